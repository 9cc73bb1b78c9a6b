"""Public tokenizer and dictionary (catboost/python-package/catboost/text_processing.py, _text_processing.pxi;
library/cpp/text_processing): the building blocks behind text features, usable on their own.

``Tokenizer`` splits a string by a delimiter or "by sense" (runs of letters / digits / punctuation), with optional
lower-casing and number handling.  ``Dictionary`` is frequency based: it counts n-grams of words or letters over a
corpus, keeps those that occur at least ``occurence_lower_bound`` times, at most ``max_dictionary_size`` of them, and
numbers them by decreasing frequency (ties by token).
"""
from __future__ import annotations

import re
from typing import Dict, Iterable, List, Optional, Sequence

from .data.pool import CatBoostError

_SENSE = re.compile(r"(?P<Number>\d+(?:[.,]\d+)*)|(?P<Word>[^\W\d_]+(?:['’][^\W\d_]+)*)|(?P<Punctuation>[^\w\s])|(?P<Unknown>_+)",
                    re.UNICODE)


def _flag(v, default):
    if v is None:
        return default
    if isinstance(v, str):
        return v.strip().lower() in ("true", "1", "yes")
    return bool(v)


class Tokenizer:
    def __init__(self, lowercasing=None, lemmatizing=None, number_process_policy=None, number_token=None,
                 separator_type=None, delimiter=None, split_by_set=None, skip_empty=None, token_types=None,
                 sub_tokens_policy=None, languages=None):
        if _flag(lemmatizing, False):
            raise CatBoostError("lemmatizing needs language models that are not part of this package")
        self.lowercasing = _flag(lowercasing, False)
        self.number_process_policy = number_process_policy or "LeaveAsIs"
        if self.number_process_policy not in ("Skip", "LeaveAsIs", "Replace"):
            raise CatBoostError("number_process_policy must be 'Skip', 'LeaveAsIs' or 'Replace'")
        self.number_token = "🔢" if number_token is None else str(number_token)
        self.separator_type = separator_type or "ByDelimiter"
        if self.separator_type not in ("ByDelimiter", "BySense"):
            raise CatBoostError("separator_type must be 'ByDelimiter' or 'BySense'")
        self.delimiter = " " if delimiter is None else str(delimiter)
        self.split_by_set = _flag(split_by_set, False)
        self.skip_empty = _flag(skip_empty, True)
        self.token_types = list(token_types) if token_types is not None else ["Word", "Number", "Unknown"]

    def _number(self, tok: str) -> Optional[str]:
        if self.number_process_policy == "LeaveAsIs":
            return tok
        return None if self.number_process_policy == "Skip" else self.number_token

    def tokenize(self, s, types: bool = False):
        """List of tokens; with ``types=True`` a pair (tokens, token types)."""
        text = "" if s is None else str(s)
        if self.lowercasing:
            text = text.lower()
        toks, kinds = [], []
        if self.separator_type == "BySense":
            for mt in _SENSE.finditer(text):
                kind = mt.lastgroup
                if kind not in self.token_types:
                    continue
                tok = mt.group()
                if kind == "Number":
                    tok = self._number(tok)
                    if tok is None:
                        continue
                toks.append(tok)
                kinds.append(kind)
        else:
            if self.split_by_set and self.delimiter:
                parts = re.split("[" + re.escape(self.delimiter) + "]", text)
            else:
                parts = text.split(self.delimiter) if self.delimiter else list(text)
            for tok in parts:
                if tok == "" and self.skip_empty:
                    continue
                kind = "Number" if re.fullmatch(r"\d+(?:[.,]\d+)*", tok) else "Word"
                if kind == "Number":
                    tok = self._number(tok)
                    if tok is None:
                        continue
                toks.append(tok)
                kinds.append(kind)
        return (toks, kinds) if types else toks


class Dictionary:
    def __init__(self, token_level_type=None, gram_order=None, skip_step=None, start_token_id=None, end_of_word_policy=None,
                 end_of_sentence_policy=None, occurence_lower_bound=None, max_dictionary_size=None, num_bpe_units=None,
                 skip_unknown=None, dictionary_type="FrequencyBased"):
        if dictionary_type not in ("FrequencyBased", "Bpe"):
            raise CatBoostError("dictionary_type must be 'FrequencyBased' or 'Bpe'")
        self.dictionary_type = dictionary_type
        self.num_bpe_units = int(num_bpe_units or 0)
        if dictionary_type == "Bpe" and self.num_bpe_units <= 0:
            raise CatBoostError("a Bpe dictionary needs num_bpe_units > 0")
        if dictionary_type == "Bpe" and int(gram_order or 1) != 1:
            raise CatBoostError("a Bpe dictionary is built over single tokens (gram_order = 1)")
        self.skip_unknown = bool(skip_unknown)
        self._merges: List[tuple] = []              # (left id, right id, count) in the order they were learned
        self.token_level_type = token_level_type or "Word"
        if self.token_level_type not in ("Word", "Letter"):
            raise CatBoostError("token_level_type must be 'Word' or 'Letter'")
        self.gram_order = int(gram_order or 1)
        self.skip_step = int(skip_step or 0)
        self.start_token_id = int(start_token_id or 0)
        self.end_of_word_policy = end_of_word_policy or "Insert"
        self.end_of_sentence_policy = end_of_sentence_policy or "Skip"
        self.occurence_lower_bound = 50 if occurence_lower_bound is None else int(occurence_lower_bound)
        self.max_dictionary_size = -1 if max_dictionary_size is None else int(max_dictionary_size)
        self._token_to_id: Dict[str, int] = {}
        self._tokens: List[str] = []
        self._counts: List[int] = []
        self._fitted = False

    # ---- helpers -------------------------------------------------------------------------------------------
    def _units(self, tokens: Sequence[str]) -> List[str]:
        if self.token_level_type == "Word":
            return list(tokens)
        units: List[str] = []
        for tok in tokens:                                     # letters, with an end-of-word mark between words
            units.extend(tok)
            if self.end_of_word_policy == "Insert":
                units.append(" ")
        return units

    def _grams(self, tokens: Sequence[str]) -> List[str]:
        units = self._units(tokens)
        k, step = self.gram_order, self.skip_step + 1
        if k == 1:
            return units
        span = (k - 1) * step
        sep = " " if self.token_level_type == "Word" else ""
        return [sep.join(units[i:i + span + 1:step]) for i in range(len(units) - span)]

    @staticmethod
    def _sentences(data, tokenizer):
        if isinstance(data, str):
            data = [data]
        for item in data:
            if isinstance(item, str):
                yield (tokenizer or Tokenizer()).tokenize(item)
            else:
                yield [str(t) for t in item]

    def _need_fit(self):
        if not self._fitted:
            raise CatBoostError("the dictionary is not built: call fit or load first")

    # ---- building and applying ----------------------------------------------------------------------------------
    def fit(self, data, tokenizer: Optional[Tokenizer] = None, verbose=False):
        """``data``: a path to a text file (one document per line), a string, a list of strings, or a list of token
        lists."""
        if isinstance(data, str) and "\n" not in data:
            try:
                with open(data, encoding="utf-8") as fh:
                    data = [line.rstrip("\n") for line in fh]
            except OSError:
                pass
        counts: Dict[str, int] = {}
        for toks in self._sentences(data, tokenizer):
            for g in self._grams(toks):
                counts[g] = counts.get(g, 0) + 1
        keep = sorted((g for g, c in counts.items() if c >= self.occurence_lower_bound), key=lambda g: (-counts[g], g))
        if self.max_dictionary_size >= 0:
            keep = keep[: self.max_dictionary_size]
        self._tokens = keep
        self._counts = [counts[g] for g in keep]
        self._token_to_id = {g: self.start_token_id + i for i, g in enumerate(keep)}
        self._fitted = True
        if self.dictionary_type == "Bpe":
            self._fit_bpe(data, tokenizer)
        return self

    # ---- byte-pair encoding ------------------------------------------------------------------------------------------
    # Behaviour follows library/cpp/text_processing/dictionary/bpe_builder.cpp: the alphabet is the frequency dictionary
    # of single units; ``num_bpe_units`` times the most frequent pair of neighbouring ids (ties: the smaller pair of
    # ids) becomes a new unit with the next free id and every non-overlapping occurrence is replaced left to right.
    # Unknown units break a sentence (no pair spans them) unless ``skip_unknown`` drops them first.
    def _base_ids(self, toks):
        ids = []
        for g in self._units(toks):
            i = self._token_to_id.get(g)
            if i is not None:
                ids.append(i)
            elif not self.skip_unknown:
                ids.append(-1)
        return ids

    @staticmethod
    def _merge_pair(arr, a, b, new_id):
        import numpy as np
        hit = np.nonzero((arr[:-1] == a) & (arr[1:] == b))[0]
        if a == b and len(hit) > 1:                       # runs "a a a": the pairs must not overlap
            keep, last = [], -2
            for i in hit.tolist():
                if i - last >= 2:
                    keep.append(i)
                    last = i
            hit = np.asarray(keep, dtype=np.int64)
        if len(hit) == 0:
            return arr
        arr = arr.copy()
        arr[hit] = new_id
        mask = np.ones(len(arr), dtype=bool)
        mask[hit + 1] = False
        return arr[mask]

    def _fit_bpe(self, data, tokenizer):
        import numpy as np
        flat: List[int] = []
        for toks in self._sentences(data, tokenizer):
            flat.extend(self._base_ids(toks))
            flat.append(-1)                                # sentence boundary: never part of a pair
        arr = np.asarray(flat, dtype=np.int64)
        self._merges = []
        sep = " " if self.token_level_type == "Word" else ""
        next_id = self.start_token_id + len(self._tokens)
        for _ in range(self.num_bpe_units):
            ok = (arr[:-1] >= 0) & (arr[1:] >= 0)
            if not ok.any():
                break
            key = (arr[:-1][ok] << 32) | arr[1:][ok]
            uniq, cnt = np.unique(key, return_counts=True)
            # occurrences of (a, a) overlap in runs; count them as the replacement will see them
            same = (uniq >> 32) == (uniq & 0xFFFFFFFF)
            for k in np.nonzero(same & (cnt > 1))[0].tolist():
                a = int(uniq[k] >> 32)
                cnt[k] = (len(arr) - len(self._merge_pair(arr, a, a, -2)))
            best = int(np.argmax(cnt))                     # np.unique sorts the keys: ties go to the smaller pair
            if cnt[best] < 2:
                break
            a, b = int(uniq[best] >> 32), int(uniq[best] & 0xFFFFFFFF)
            arr = self._merge_pair(arr, a, b, next_id)
            self._merges.append((a, b, int(cnt[best])))
            tok = self.get_token(a) + sep + self.get_token(b)
            self._tokens.append(tok)
            self._counts.append(int(cnt[best]))
            self._token_to_id.setdefault(tok, next_id)
            next_id += 1

    def _apply_bpe(self, toks):
        import numpy as np
        arr = np.asarray(self._base_ids(toks) + [-1], dtype=np.int64)
        first_new = self.start_token_id + len(self._tokens) - len(self._merges)
        for k, (a, b, _) in enumerate(self._merges):
            if len(arr) < 3:
                break
            arr = self._merge_pair(arr, a, b, first_new + k)
        return arr[:-1].tolist()

    def apply(self, data, tokenizer: Optional[Tokenizer] = None, unknown_token_policy=None):
        """Token ids per document.  Unknown tokens are dropped ('Skip', default) or mapped to ``unknown_token_id``
        ('Insert')."""
        self._need_fit()
        policy = unknown_token_policy or "Skip"
        if policy not in ("Skip", "Insert"):
            raise CatBoostError("unknown_token_policy must be 'Skip' or 'Insert'")
        single = isinstance(data, str) or (len(data) > 0 and not isinstance(data[0], (str, list, tuple)))
        out = []
        for toks in self._sentences([data] if isinstance(data, str) else data, tokenizer):
            ids = []
            if self.dictionary_type == "Bpe":
                for i in self._apply_bpe(toks):
                    if i >= 0:
                        ids.append(i)
                    elif policy == "Insert":
                        ids.append(self.unknown_token_id)
                out.append(ids)
                continue
            for g in self._grams(toks):
                i = self._token_to_id.get(g)
                if i is not None:
                    ids.append(i)
                elif policy == "Insert":
                    ids.append(self.unknown_token_id)
            out.append(ids)
        return out[0] if single and isinstance(data, str) else out

    # ---- inspection ----------------------------------------------------------------------------------------------------
    @property
    def size(self) -> int:
        self._need_fit()
        return len(self._tokens)

    def get_token(self, token_id) -> str:
        self._need_fit()
        k = int(token_id) - self.start_token_id
        if not 0 <= k < len(self._tokens):
            raise CatBoostError(f"no token with id {token_id}")
        return self._tokens[k]

    def get_tokens(self, token_ids: Iterable[int]) -> List[str]:
        return [self.get_token(t) for t in token_ids]

    def get_top_tokens(self, top_size=None) -> List[str]:
        self._need_fit()
        return list(self._tokens if top_size is None else self._tokens[: int(top_size)])

    @property
    def unknown_token_id(self) -> int:
        self._need_fit()
        return self.start_token_id + len(self._tokens)

    @property
    def end_of_sentence_token_id(self) -> int:
        return self.unknown_token_id + 1

    @property
    def min_unused_token_id(self) -> int:
        return self.unknown_token_id + 2

    # ---- files ---------------------------------------------------------------------------------------------------------
    def save(self, frequency_dict_path, bpe_path=None):
        """Text file: a JSON line with the options, then one ``id<TAB>count<TAB>token`` line per entry."""
        import json
        self._need_fit()
        opts = {"token_level_type": self.token_level_type, "gram_order": self.gram_order, "skip_step": self.skip_step,
                "start_token_id": self.start_token_id, "end_of_word_policy": self.end_of_word_policy,
                "end_of_sentence_policy": self.end_of_sentence_policy, "dictionary_format": "id_count_token"}
        with open(frequency_dict_path, "w", encoding="utf-8") as fh:
            fh.write(json.dumps(opts) + "\n" + str(len(self._tokens)) + "\n")
            for i, (tok, c) in enumerate(zip(self._tokens, self._counts)):
                fh.write(f"{self.start_token_id + i}\t{c}\t{tok}\n")
        if self.dictionary_type == "Bpe":
            if bpe_path is None:
                raise CatBoostError("a Bpe dictionary is saved to two files: pass bpe_path")
            first_new = self.start_token_id + len(self._tokens) - len(self._merges)
            with open(bpe_path, "w", encoding="utf-8") as fh:          # left id, right id, count, text of the new unit
                for k, (a, b, c) in enumerate(self._merges):
                    fh.write(f"{a}\t{b}\t{c}\t{self.get_token(first_new + k)}\n")
        return self

    def load(self, frequency_dict_path, bpe_path=None):
        import json
        with open(frequency_dict_path, encoding="utf-8") as fh:
            opts = json.loads(fh.readline())
            n = int(fh.readline())
            self.token_level_type = opts.get("token_level_type", "Word")
            self.gram_order = int(opts.get("gram_order", 1))
            self.skip_step = int(opts.get("skip_step", 0))
            self.start_token_id = int(opts.get("start_token_id", 0))
            self.end_of_word_policy = opts.get("end_of_word_policy", "Insert")
            self.end_of_sentence_policy = opts.get("end_of_sentence_policy", "Skip")
            self._tokens, self._counts = [], []
            for _ in range(n):
                _id, c, tok = fh.readline().rstrip("\n").split("\t", 2)
                self._tokens.append(tok)
                self._counts.append(int(c))
        self._token_to_id = {}
        for i, g in enumerate(self._tokens):
            self._token_to_id.setdefault(g, self.start_token_id + i)
        self._fitted = True
        self._merges = []
        if bpe_path is not None:
            self.dictionary_type = "Bpe"
            with open(bpe_path, encoding="utf-8") as fh:
                for line in fh:
                    a, b, c, _tok = line.rstrip("\n").split("\t", 3)
                    self._merges.append((int(a), int(b), int(c)))
            self.num_bpe_units = len(self._merges)
        return self
        return self
