"""Text and embedding features as "estimated" numeric features.

The reference turns a text column into tokens (tokenizer -> dictionary) and then into numeric features with feature
calcers -- BoW, NaiveBayes, BM25 -- and an embedding column into LDA projections and KNN class votes
(catboost/private/libs/text_features/*, catboost/private/libs/embedding_features/*,
catboost/private/libs/feature_estimator/*); the GPU trainer consumes them as ordinary float features
(catboost/cuda/gpu_data/estimated_features_calcer.cpp).  The same is done here: ``EstimatedFeatures.fit`` learns the
dictionaries / statistics on the learn pool and returns the learn matrix, ``transform`` maps any pool.

Target-aware calcers (NaiveBayes, BM25, LDA, KNN) would leak the label of a learn document into its own feature if
they were computed from all learn documents, so the learn matrix is computed in permutation order: the documents are
cut into blocks of geometrically growing size and a block only sees the statistics of the blocks before it (the same
idea as ordered CTRs).  Applied to other pools the calcers use the statistics of the whole learn pool.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import numpy as np

_TOKEN = re.compile(r"[0-9A-Za-z_À-￿]+")


def tokenize(text, lowercasing: bool = True) -> List[str]:
    s = "" if text is None else str(text)
    if lowercasing:
        s = s.lower()
    return _TOKEN.findall(s)


class _Dictionary:
    def __init__(self, max_size=50000, occurrence_lower_bound=3, gram_order=1):
        self.max_size, self.lower, self.gram = int(max_size), int(occurrence_lower_bound), int(gram_order)
        self.ids: Dict[str, int] = {}

    def _grams(self, toks):
        if self.gram == 1:
            return toks
        return [" ".join(toks[i:i + self.gram]) for i in range(len(toks) - self.gram + 1)]

    def fit(self, docs_tokens):
        cnt: Dict[str, int] = {}
        for toks in docs_tokens:
            for g in self._grams(toks):
                cnt[g] = cnt.get(g, 0) + 1
        keep = sorted((g for g, c in cnt.items() if c >= self.lower), key=lambda g: (-cnt[g], g))[: self.max_size]
        self.ids = {g: i for i, g in enumerate(keep)}
        return self

    def encode(self, docs_tokens):
        """CSR of distinct token ids per document: (indptr, indices)."""
        indptr = [0]
        idx: List[int] = []
        ids = self.ids
        for toks in docs_tokens:
            seen = {ids[g] for g in self._grams(toks) if g in ids}
            idx.extend(sorted(seen))
            indptr.append(len(idx))
        return np.asarray(indptr, dtype=np.int64), np.asarray(idx, dtype=np.int64)


def _ordered_blocks(n: int, rng) -> List[np.ndarray]:
    """A random permutation of the rows cut into blocks of doubling size (the first holds about 1/16 of the rows)."""
    perm = rng.permutation(n)
    blocks, start, size = [], 0, max(1, n // 16)
    while start < n:
        blocks.append(perm[start:start + size])
        start += size
        size *= 2
    return blocks


class _TextCalcers:
    """BoW + (classification) NaiveBayes and BM25 over one dictionary."""

    def __init__(self, top_tokens=2000, calcers=("BoW", "NaiveBayes", "BM25")):
        self.top_tokens, self.calcers = int(top_tokens), tuple(calcers)

    def fit(self, dictionary, indptr, indices, cls, n_classes):
        self.V = len(dictionary.ids)
        self.n_classes = n_classes
        self.bow_ids = np.arange(min(self.top_tokens, self.V))          # dictionary ids are sorted by frequency
        self.counts = self._class_counts(indptr, indices, cls, np.arange(len(indptr) - 1)) if n_classes else None
        n_docs = len(indptr) - 1
        self.avg_len = float(len(indices)) / max(1, n_docs)
        self.class_docs = np.bincount(cls, minlength=n_classes).astype(np.float64) if n_classes else None
        return self

    def _class_counts(self, indptr, indices, cls, rows):
        out = np.zeros((self.n_classes, max(1, self.V)), dtype=np.float64)
        for c in range(self.n_classes):
            r = rows[cls[rows] == c]
            if len(r):
                tok = np.concatenate([indices[indptr[i]:indptr[i + 1]] for i in r]) if len(r) else np.zeros(0, np.int64)
                if len(tok):
                    out[c] += np.bincount(tok, minlength=max(1, self.V))[: max(1, self.V)]
        return out

    def names(self, prefix, id_to_token):
        out = []
        if "BoW" in self.calcers:
            out += [f"{prefix}_bow_{id_to_token[i]}" for i in self.bow_ids]
        if self.n_classes:
            if "NaiveBayes" in self.calcers:
                out += [f"{prefix}_nb_{c}" for c in range(self.n_classes)]
            if "BM25" in self.calcers:
                out += [f"{prefix}_bm25_{c}" for c in range(self.n_classes)]
        return out

    def _features(self, indptr, indices, rows, counts, class_docs):
        n = len(rows)
        cols = []
        if "BoW" in self.calcers:
            bow = np.zeros((n, len(self.bow_ids)), dtype=np.float32)
            for k, i in enumerate(rows):
                t = indices[indptr[i]:indptr[i + 1]]
                t = t[t < len(self.bow_ids)]
                bow[k, t] = 1.0
            cols.append(bow)
        if self.n_classes:
            tot = counts.sum(1, keepdims=True)
            logp = np.log((counts + 1.0) / (tot + max(1, self.V)))                 # Laplace-smoothed token likelihoods
            prior = np.log((class_docs + 1.0) / (class_docs.sum() + self.n_classes))
            k1, b = 1.5, 0.75
            idf = np.log((class_docs.sum() + 1.0) / (counts.sum(0) + 1.0)) + 1.0
            nb = np.zeros((n, self.n_classes), dtype=np.float32)
            bm = np.zeros((n, self.n_classes), dtype=np.float32)
            for k, i in enumerate(rows):
                t = indices[indptr[i]:indptr[i + 1]]
                if len(t) == 0:
                    nb[k] = prior
                    continue
                s = prior + logp[:, t].sum(1)
                s = s - s.max()
                e = np.exp(s)
                nb[k] = e / e.sum()
                tf = counts[:, t] / np.maximum(class_docs[:, None], 1.0)          # in-class document frequency
                norm = 1.0 - b + b * len(t) / max(self.avg_len, 1e-9)
                bm[k] = (idf[t] * tf * (k1 + 1.0) / (tf + k1 * norm)).sum(1)
            if "NaiveBayes" in self.calcers:
                cols.append(nb)
            if "BM25" in self.calcers:
                cols.append(bm)
        return np.concatenate(cols, 1) if cols else np.zeros((n, 0), dtype=np.float32)

    def transform(self, indptr, indices):
        rows = np.arange(len(indptr) - 1)
        return self._features(indptr, indices, rows, self.counts, self.class_docs)

    def transform_learn(self, indptr, indices, cls, blocks):
        n = len(indptr) - 1
        first = self._features(indptr, indices, np.arange(min(n, 1)), self.counts, self.class_docs) if n else None
        out = np.zeros((n, first.shape[1] if first is not None else 0), dtype=np.float32)
        if not self.n_classes:
            return self.transform(indptr, indices)
        counts = np.zeros_like(self.counts)
        class_docs = np.zeros(self.n_classes)
        for blk in blocks:
            out[blk] = self._features(indptr, indices, blk, counts, class_docs)
            counts += self._class_counts(indptr, indices, cls, blk)
            class_docs += np.bincount(cls[blk], minlength=self.n_classes)
        return out


class _EmbeddingCalcers:
    """LDA projection (classification) and KNN votes / mean target over one embedding column."""

    def __init__(self, k=5, calcers=("LDA", "KNN"), device=None):
        self.k, self.calcers = int(k), tuple(calcers)
        self.device = device          # a CUDA torch.device sends the neighbour search of large clouds to the GPU

    def _lda(self, E, cls, n_classes):
        d = E.shape[1]
        mu = E.mean(0)
        Sw = np.zeros((d, d))
        means = []
        for c in range(n_classes):
            Ec = E[cls == c]
            if len(Ec) == 0:
                continue
            m = Ec.mean(0)
            means.append(m - mu)
            Sw += (Ec - m).T @ (Ec - m)
        if not means:
            return np.zeros((d, 0))
        Sw = Sw / max(1, len(E)) + 1e-3 * np.eye(d) * max(1e-12, np.trace(Sw) / max(1, d * len(E)) + 1e-12)
        M = np.stack(means, 1)                                   # [d, classes]
        W = np.linalg.solve(Sw, M)                               # discriminant directions
        k = min(max(1, n_classes - 1), d)
        u, _, _ = np.linalg.svd(W, full_matrices=False)
        return u[:, :k]

    # clouds of at least this many rows go to the tensor-core search when the calcers were given a CUDA device
    DEVICE_MIN_CLOUD = 1024

    def _knn(self, Q, E, tgt, n_classes):
        if len(E) == 0:
            return np.zeros((len(Q), n_classes if n_classes else 1), dtype=np.float32)
        out = np.zeros((len(Q), n_classes if n_classes else 1), dtype=np.float32)
        dev = getattr(self, "device", None)
        if dev is not None and getattr(dev, "type", "") == "cuda" and len(E) >= self.DEVICE_MIN_CLOUD and len(Q):
            # neighbours from the device (ops/cuda/cb_knn_tc.cu: tcgen05 distance GEMM with a top-k epilogue, candidates
            # re-ranked by fp32 distances); the votes are counted on the host from the returned indices
            import torch
            from ..ops import api as ops
            k = min(self.k, len(E))
            nn = ops.knn_search(torch.from_numpy(np.ascontiguousarray(Q, dtype=np.float32)).to(dev),
                                torch.from_numpy(np.ascontiguousarray(E, dtype=np.float32)).to(dev), k).cpu().numpy()
            if n_classes:
                for c in range(n_classes):
                    out[:, c] = (tgt[nn] == c).mean(1)
            else:
                out[:, 0] = tgt[nn].mean(1)
            return out
        e2 = (E * E).sum(1)
        for s in range(0, len(Q), 2048):
            q = Q[s:s + 2048]
            d2 = (q * q).sum(1, keepdims=True) - 2.0 * q @ E.T + e2[None, :]
            k = min(self.k, len(E))
            nn = np.argpartition(d2, k - 1, axis=1)[:, :k]
            if n_classes:
                for c in range(n_classes):
                    out[s:s + 2048, c] = (tgt[nn] == c).mean(1)
            else:
                out[s:s + 2048, 0] = tgt[nn].mean(1)
        return out

    def fit(self, E, tgt, n_classes):
        self.n_classes = n_classes
        self.E, self.tgt = E.astype(np.float64), tgt
        self.proj = self._lda(self.E, tgt, n_classes) if (n_classes and "LDA" in self.calcers) else np.zeros((E.shape[1], 0))
        return self

    def names(self, prefix):
        out = [f"{prefix}_lda_{k}" for k in range(self.proj.shape[1])]
        if "KNN" in self.calcers:
            out += [f"{prefix}_knn_{c}" for c in range(self.n_classes if self.n_classes else 1)]
        return out

    def transform(self, E):
        E = E.astype(np.float64)
        cols = [E @ self.proj]
        if "KNN" in self.calcers:
            cols.append(self._knn(E, self.E, self.tgt, self.n_classes))
        return np.concatenate(cols, 1).astype(np.float32)

    def transform_learn(self, E, blocks):
        E = E.astype(np.float64)
        n = len(E)
        width = self.proj.shape[1] + ((self.n_classes if self.n_classes else 1) if "KNN" in self.calcers else 0)
        out = np.zeros((n, width), dtype=np.float32)
        seen = np.zeros(0, dtype=np.int64)
        for blk in blocks:
            cols = []
            if self.proj.shape[1]:
                proj = self._lda(E[seen], self.tgt[seen], self.n_classes) if len(seen) > self.n_classes else np.zeros_like(self.proj)
                if proj.shape != self.proj.shape:
                    proj = np.zeros_like(self.proj)
                # keep the orientation of the final directions so that the feature means the same thing in every block
                sign = np.sign((proj * self.proj).sum(0))
                sign[sign == 0] = 1.0
                cols.append(E[blk] @ (proj * sign))
            if "KNN" in self.calcers:
                cols.append(self._knn(E[blk], E[seen], self.tgt[seen], self.n_classes))
            out[blk] = np.concatenate(cols, 1)
            seen = np.concatenate([seen, blk])
        return out


class EstimatedFeatures:
    """All text / embedding columns of a pool -> one float matrix."""

    def set_device(self, device):
        """A CUDA ``torch.device`` sends the neighbour search of the embedding calcers to the GPU; ``None`` (the state a
        model is stored and loaded in) keeps it on the host."""
        self.device = device
        for item in self.emb:
            for obj in (item if isinstance(item, (list, tuple)) else [item]):
                if isinstance(obj, _EmbeddingCalcers):
                    obj.device = device

    def __init__(self, text_processing: Optional[dict] = None, seed: int = 0, tokenizers=None, dictionaries=None,
                 feature_calcers=None):
        """``tokenizers`` / ``dictionaries`` / ``feature_calcers`` are the estimator keywords of the same names; the same
        keys (and ``feature_processing``) may sit inside ``text_processing`` (the reference's JSON layout,
        catboost/private/libs/options/text_processing_options.cpp).  Every (dictionary, calcer list) pair of the
        processing description yields its own block of features for every text column."""
        tp = dict(text_processing or {})
        self.max_dictionary_size = int(tp.get("max_dictionary_size", 50000))
        self.occurrence_lower_bound = int(tp.get("occurrence_lower_bound", 3))
        self.top_tokens = int(tp.get("top_tokens_count", 2000))
        calc_default = feature_calcers if feature_calcers is not None else tp.get("feature_calcers", ("BoW", "NaiveBayes", "BM25"))
        self.text_calcers = tuple(self._calcer_names(calc_default))
        self.embedding_calcers = tuple(tp.get("embedding_calcers", ("LDA", "KNN")))
        self.seed = int(seed)
        self.device = None            # set_device(): where the embedding neighbour search runs during training
        self.text, self.emb, self.names = [], [], []
        # tokenizer: the first description (one tokenizer for all dictionaries)
        toks = tokenizers if tokenizers is not None else tp.get("tokenizers")
        tk = self._kv(toks[0]) if toks else {}
        self.lowercasing = str(tk.get("lowercasing", "true")).lower() in ("1", "true", "yes")
        self.delimiter = tk.get("delimiter") if str(tk.get("separator_type", "BySense")) == "ByDelimiter" else None
        # dictionaries: (id, max size, occurrence lower bound, gram order)
        self.dict_specs = []
        for d in (dictionaries if dictionaries is not None else tp.get("dictionaries") or []):
            kv = self._kv(d, id_key="dictionary_id")
            self.dict_specs.append((str(kv.get("dictionary_id", f"dict{len(self.dict_specs)}")),
                                    int(kv.get("max_dictionary_size", self.max_dictionary_size)),
                                    int(kv.get("occurrence_lower_bound", kv.get("occurence_lower_bound", self.occurrence_lower_bound))),
                                    int(kv.get("gram_order", 1))))
        if not self.dict_specs:
            self.dict_specs = [("Word", self.max_dictionary_size, self.occurrence_lower_bound, 1)]
        # processing: which calcers run on which dictionary
        self.processing = []
        fp = tp.get("feature_processing")
        if isinstance(fp, dict) and fp:
            known = {d[0] for d in self.dict_specs}
            for item in fp.get("default", next(iter(fp.values()))):
                for name in item.get("dictionaries_names", [d[0] for d in self.dict_specs]):
                    if name not in known:
                        raise ValueError(f"feature_processing names the dictionary {name!r}, which is not described")
                    self.processing.append((name, tuple(self._calcer_names(item.get("feature_calcers", self.text_calcers)))))
        else:
            self.processing = [(d[0], self.text_calcers) for d in self.dict_specs]

    @staticmethod
    def _kv(desc, id_key=None):
        """A description given as a dict or as 'Id:key=value,key=value'."""
        if isinstance(desc, dict):
            return {str(k): v for k, v in desc.items()}
        head, _, rest = str(desc).partition(":")
        out = {id_key: head} if id_key and "=" not in head else {}
        for part in ([head] if "=" in head else []) + [p for p in rest.split(",") if p]:
            k, _, v = part.partition("=")
            out[k.strip()] = v.strip()
        return out

    def _calcer_names(self, calcers):
        out = []
        for c in ([calcers] if isinstance(calcers, str) else list(calcers)):
            name, _, rest = str(c).partition(":")
            for part in [p for p in rest.split(",") if p]:
                k, _, v = part.partition("=")
                if k.strip() == "top_tokens_count":
                    self.top_tokens = int(v)
            if name not in ("BoW", "NaiveBayes", "BM25"):
                raise ValueError(f"unknown text feature calcer {name!r}")
            out.append(name)
        return out

    def _tokens(self, col):
        if self.delimiter is not None:
            return [[t for t in ("" if v is None else (str(v).lower() if self.lowercasing else str(v))).split(self.delimiter) if t]
                    for v in col]
        return [tokenize(v, self.lowercasing) for v in col]

    def fit(self, pool, target: np.ndarray, n_classes: int):
        """target: class index per row for classification (n_classes >= 2), else the numeric target (n_classes = 0)."""
        rng = np.random.default_rng(self.seed + 99)
        n = pool.num_row()
        blocks = _ordered_blocks(n, rng)
        cls = target.astype(np.int64) if n_classes else None
        mats = []
        self.text_flat = list(pool.text_feature_indices)
        self.emb_flat = list(pool.embedding_feature_indices)
        specs = {d[0]: d for d in self.dict_specs}
        for j, col in enumerate(pool.text_data):
            toks = self._tokens(col)
            built = {}
            for name, calcers in self.processing:
                _, max_size, lower, gram = specs[name]
                if name not in built:
                    d = _Dictionary(max_size, min(lower, max(1, n // 20)), gram).fit(toks)
                    built[name] = (d,) + d.encode(toks)
                d, indptr, indices = built[name]
                calc = _TextCalcers(self.top_tokens, calcers).fit(d, indptr, indices, cls, n_classes)
                self.text.append((j, d, calc))
                inv = {i: g for g, i in d.ids.items()}
                prefix = f"text{self.text_flat[j]}" if len(self.processing) == 1 else f"text{self.text_flat[j]}.{name}"
                self.names += calc.names(prefix, inv)
                mats.append(calc.transform_learn(indptr, indices, cls, blocks))
        for j, E in enumerate(pool.embedding_data):
            calc = _EmbeddingCalcers(5, self.embedding_calcers, device=self.device).fit(np.asarray(E, dtype=np.float32), cls if n_classes else target.astype(np.float64), n_classes)
            self.emb.append(calc)
            self.names += calc.names(f"emb{self.emb_flat[j]}")
            mats.append(calc.transform_learn(np.asarray(E, dtype=np.float32), blocks))
        learn = np.concatenate(mats, 1).astype(np.float32) if mats else np.zeros((n, 0), dtype=np.float32)
        return learn

    def transform(self, pool) -> np.ndarray:
        mats = []
        n_text = len({t[0] for t in self.text})
        if len(pool.text_data) != n_text or len(pool.embedding_data) != len(self.emb):
            raise ValueError("the data does not have the text / embedding columns the model was trained with")
        tok_cache = {}
        for j, d, calc in self.text:
            if j not in tok_cache:
                tok_cache[j] = self._tokens(pool.text_data[j])
            indptr, indices = d.encode(tok_cache[j])
            mats.append(calc.transform(indptr, indices))
        for calc, E in zip(self.emb, pool.embedding_data):
            mats.append(calc.transform(np.asarray(E, dtype=np.float32)))
        n = pool.num_row()
        return np.concatenate(mats, 1).astype(np.float32) if mats else np.zeros((n, 0), dtype=np.float32)
