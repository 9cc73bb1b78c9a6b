"""Device-dispatching wrappers around the native kernels, plus plain-PyTorch reference implementations.

``hist`` / ``update_leaf`` / ``update_nodes`` / ``leaf_index`` run the hand-written CUDA kernel when the store
is on a GPU and the OpenMP implementation when it is on the CPU.  The ``*_reference`` functions are
straightforward fp32 PyTorch restatements of the same operation; tests compare the kernels against them.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from ..data.quantization import BinnedStore
from . import native


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


_dev_info = {}


def device_info(dev):
    key = str(dev)
    if key not in _dev_info:
        sm, smem = ctypes.c_int(0), ctypes.c_int(0)
        with torch.cuda.device(dev):
            native.cuda_check(native.cuda_lib().cb_device_info(ctypes.byref(sm), ctypes.byref(smem)), "cb_device_info")
        _dev_info[key] = (sm.value, smem.value)
    return _dev_info[key]


def hist(store: BinnedStore, leaf: torch.Tensor, stats: torch.Tensor, slot_table: torch.Tensor, nslots: int,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[slot, s, feat_off[f] + bin] = sum of stats[s, i] over documents with slot_table[leaf[i]] == slot.

    leaf: int16 [npad]; stats: float32 [S, npad]; slot_table: int16 [n_leaf_ids] (-1 = skip)."""
    S = stats.shape[0]
    TB = store.TB
    dev = store.bins.device
    if out is None:
        out = torch.zeros((nslots, S, TB), dtype=torch.float32, device=dev)
    else:
        out.zero_()
    if dev.type == "cpu":
        native.cpu_lib().cbc_hist(_p(store.bins), ctypes.c_longlong(store.npad), ctypes.c_longlong(store.n),
                                  ctypes.c_int(store.F), _p(store.feat_off), ctypes.c_int(TB), _p(leaf), _p(stats),
                                  ctypes.c_int(S), _p(slot_table), ctypes.c_int(nslots), _p(out))
        return out
    lib = native.cuda_lib()
    sm, max_smem = device_info(dev)
    B = max(4, (store.max_bins + 3) // 4 * 4)
    per_slot = S * 4 * B * 4
    max_smem -= 2048
    spp = max(1, min(nslots, max_smem // per_slot))
    if per_slot > max_smem:
        # too many statistic columns for one shared-memory pass: process them in chunks
        smax = max(1, max_smem // (4 * B * 4))
        for s0 in range(0, S, smax):
            s1 = min(S, s0 + smax)
            out[:, s0:s1] = hist(store, leaf, stats[s0:s1].contiguous(), slot_table, nslots)
        return out
    occ = max(1, min(4, (max_smem) // max(1, spp * per_slot + 1024)))
    grid = sm * occ
    # integer cells: every statistic is scaled by its largest magnitude (shared fp32 atomics are compare-and-swap loops)
    statmax = stats[:, : store.n].abs().amax(dim=1).clamp_min(1e-30).contiguous()
    native.cuda_check(lib.cb_hist_n(ctypes.c_void_p(store.handle), _p(leaf), _p(stats), S, 0, None, _p(slot_table),
                                    nslots, spp, B, _p(out), _p(statmax), grid, 512, _stream(dev)), "cb_hist_n")
    return out


def sort_pairs(keys: torch.Tensor):
    """Stable ascending sort of int64 keys: ``(sorted_keys, order)`` with ``order`` int64 such that
    ``sorted_keys == keys[order]`` and equal keys keep their input order.  On the GPU this is the hand-written radix sort
    of ``cb_sort.cu`` (8 passes of 8 bits); on the CPU the framework's stable sort."""
    if not keys.is_cuda:
        return torch.sort(keys, stable=True)
    dev = keys.device
    n = int(keys.numel())
    ka = keys.contiguous().clone()
    kb = torch.empty_like(ka)
    va = torch.empty(n, dtype=torch.int32, device=dev)
    vb = torch.empty(n, dtype=torch.int32, device=dev)
    lib = native.cuda_lib()
    scratch = torch.empty(max(1, int(lib.cb_sort_scratch_bytes(n))), dtype=torch.uint8, device=dev)
    native.cuda_check(lib.cb_sort_pairs_i64(_p(ka), _p(va), _p(kb), _p(vb), n, _p(scratch), 1, _stream(dev)),
                      "cb_sort_pairs_i64")
    return ka, va.long()


KNN_TIMEOUT = 0x61


def knn_candidates(Q: torch.Tensor, E: torch.Tensor, cand: int = 16):
    """Approximate nearest rows of ``E`` for every row of ``Q`` on the tensor cores (ops/cuda/cb_knn_tc.cu: TMA-fed
    tcgen05 GEMM with the accumulator in TMEM, top-k selection in the epilogue).  Q [nq, d], E [ne, d] float tensors on
    one CUDA device, d <= cb_knn_max_dim().  Returns (idx int64 [nq, C], score float32 [nq, C]) with
    score = |e|^2 - 2 q.e computed from bf16-rounded inputs, ascending; C = 2 * cand: the kernel keeps a list of ``cand``
    (8 or 16) per half of a cloud tile and the two halves are merged here; idx is -1 where the cloud has fewer rows.
    Returns None when the shape does not qualify."""
    lib = native.cuda_lib()
    dev = Q.device
    nq, d = int(Q.shape[0]), int(Q.shape[1])
    ne = int(E.shape[0])
    C = int(cand)
    if d > int(lib.cb_knn_max_dim()) or nq == 0 or ne == 0 or nq >= (1 << 31) or ne >= (1 << 31):
        return None
    dpad = (d + 63) // 64 * 64
    qb = torch.zeros((nq, dpad), dtype=torch.bfloat16, device=dev)
    eb = torch.zeros((ne, dpad), dtype=torch.bfloat16, device=dev)
    qb[:, :d] = Q
    eb[:, :d] = E
    e2 = (eb.float() ** 2).sum(1).contiguous()
    splits = int(lib.cb_knn_splits(nq, ne))
    lists = 2 * splits                       # the kernel keeps one list per column half of a cloud tile
    out_idx = torch.empty((nq, lists, C), dtype=torch.int32, device=dev)
    out_val = torch.empty((nq, lists, C), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.cb_knn_tc(_p(qb), nq, _p(eb), ne, dpad, _p(e2), splits, C, _p(out_idx), _p(out_val), _p(status), _stream(dev))
    if rc == -2:
        return None
    native.cuda_check(rc, "cb_knn_tc")
    if int(status.item()) != 0:
        raise RuntimeError(f"cb_knn_tc: a wait inside the kernel ran out (status {int(status.item()):#x})")
    val = out_val.reshape(nq, lists * C)
    idx = out_idx.reshape(nq, lists * C).long()
    val, pos = torch.topk(val, min(2 * C, val.shape[1]), dim=1, largest=False, sorted=True)
    return idx.gather(1, pos), val


def knn_search(Q: torch.Tensor, E: torch.Tensor, k: int):
    """Indices [nq, k] of the k nearest rows of ``E`` (Euclidean) for every row of ``Q``: tensor-core candidates
    re-ranked by fp32 distances.  Falls back to a chunked fp32 distance matrix (library GEMM) when the shape does not
    qualify for the tensor-core kernel (more than cb_knn_max_dim() dimensions, k above 8)."""
    k = min(int(k), int(E.shape[0]))
    cand = None
    if Q.is_cuda and k <= 8:
        # lists of 8 hold the 5 nearest of a tile half with room for the reordering bf16 rounding causes; longer lists
        # for k up to 8
        cand = knn_candidates(Q, E, 8 if k <= 5 else 16)
    if cand is not None:
        idx, _ = cand
        Qf, Ef = Q.float(), E.float()
        out = torch.empty((Q.shape[0], k), dtype=torch.long, device=Q.device)
        step = max(1, (64 << 20) // max(1, idx.shape[1] * Ef.shape[1] * 4))
        for s in range(0, Q.shape[0], step):
            ii = idx[s:s + step]
            g = Ef[ii.clamp_min(0)]                                    # [b, C, d]
            d2 = ((g - Qf[s:s + step].unsqueeze(1)) ** 2).sum(2)
            d2 = torch.where(ii >= 0, d2, torch.full_like(d2, float("inf")))
            pos = torch.topk(d2, k, dim=1, largest=False, sorted=True).indices
            out[s:s + step] = ii.gather(1, pos)
        return out
    Qf, Ef = Q.float(), E.float()
    e2 = (Ef * Ef).sum(1)
    out = torch.empty((Q.shape[0], k), dtype=torch.long, device=Q.device)
    step = max(1, (256 << 20) // max(1, Ef.shape[0] * 4))
    for s in range(0, Q.shape[0], step):
        d2 = e2.unsqueeze(0) - 2.0 * Qf[s:s + step] @ Ef.t()
        out[s:s + step] = torch.topk(d2, k, dim=1, largest=False, sorted=True).indices
    return out


_LEAF_NEWTON_STATE = {}


def leaf_newton(loss_id: int, p0: float, p1: float, approx: torch.Tensor, target: torch.Tensor, weight, leaf: torch.Tensor,
                n: int, n_leaves: int, steps: int, newton: bool, l2: float, lr: float, backtracking: str = "No"):
    """All leaf-estimation steps of one tree in one cooperative launch (ops/cuda/cb_leaf.cu, the kernel of the device
    trainer) for a tree of any shape: ``leaf`` holds the leaf number of every document.  Returns (leaf values times the
    learning rate [n_leaves], leaf weights [n_leaves]) on the device, or None when the tree has too many leaves for the
    kernel's shared-memory cells.  One rank only."""
    dev = approx.device
    lib = native.cuda_lib()
    L = int(n_leaves)
    grid = int(lib.cb_leaf_newton_max_grid(L))
    if grid <= 0:
        return None
    key = (str(dev), L)
    st = _LEAF_NEWTON_STATE.get(key)
    if st is None:
        if len(_LEAF_NEWTON_STATE) > 16:
            _LEAF_NEWTON_STATE.clear()
        st = (torch.zeros(int(lib.cb_leaf_newton_sums_doubles(L)), dtype=torch.float64, device=dev),
              torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(2, dtype=torch.float32, device=dev),
              torch.zeros(1, dtype=torch.int32, device=dev))
        _LEAF_NEWTON_STATE[key] = st
    sums, counter, vmax, iter_ptr = st
    delta = torch.zeros(L, dtype=torch.float32, device=dev)
    cur = torch.zeros(L, dtype=torch.float32, device=dev)
    leaf_w = torch.zeros(L, dtype=torch.float32, device=dev)
    a, t = approx.contiguous().float(), target.contiguous().float()
    w = None if weight is None else weight.contiguous().float()
    bt = {"No": 0, "AnyImprovement": 1, "Armijo": 2}[str(backtracking or "No")]
    rc = lib.cb_leaf_newton(int(loss_id), float(p0), float(p1), _p(a), _p(t), _p(w), _p(leaf), int(n), L, _p(delta), _p(sums),
                            _p(counter), _p(vmax), int(steps), 1 if newton else 0, float(l2), float(lr), _p(cur), None, None, L,
                            _p(iter_ptr), _p(leaf_w), None, bt, grid, _stream(dev))
    if rc == -2:
        return None
    native.cuda_check(rc, "cb_leaf_newton")
    return cur, leaf_w


def query_der(kind: str, approx: torch.Tensor, target: torch.Tensor, weight, offsets: torch.Tensor, beta: float = 1.0):
    """(der, hess) [n] of a query-wise objective on the GPU (ops/cuda/cb_querywise.cu).  ``kind``: 'QueryRMSE',
    'QuerySoftMax' or 'PairLogit' (all pairs of a query whose labels differ); ``offsets``: int64 [Q + 1] row offsets."""
    dev = approx.device
    n = int(approx.shape[0])
    a, t = approx.contiguous().float(), target.contiguous().float()
    w = None if weight is None else weight.contiguous().float()
    off = offsets.contiguous().long()
    Q = int(off.numel()) - 1
    der, hess = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    lib = native.cuda_lib()
    if kind == "QueryRMSE":
        rc = lib.cb_query_rmse_der(_p(a), _p(t), _p(w), _p(off), Q, _p(der), _p(hess), _stream(dev))
    elif kind == "QuerySoftMax":
        rc = lib.cb_query_softmax_der(_p(a), _p(t), _p(w), _p(off), Q, float(beta), _p(der), _p(hess), _stream(dev))
    elif kind == "PairLogit":
        rc = lib.cb_pair_logit_labels_der(_p(a), _p(t), _p(off), Q, _p(der), _p(hess), _stream(dev))
    else:
        raise ValueError(kind)
    native.cuda_check(rc, "cb_querywise")
    return der, hess


def pair_metric(approx: torch.Tensor, target, offsets, pairs=None, pair_weight=None):
    """(PairLogit loss, PairAccuracy) of the approximations on the GPU: explicit (winner, loser) pairs, or every pair of a
    query whose labels differ."""
    dev = approx.device
    out = torch.zeros(3, dtype=torch.float64, device=dev)
    a = approx.contiguous().float()
    if pairs is not None:
        pr = pairs.contiguous().long()
        pw = None if pair_weight is None else pair_weight.contiguous().float()
        rc = native.cuda_lib().cb_pair_metric(_p(a), None, None, 0, _p(pr), _p(pw), int(pr.shape[0]), _p(out), _stream(dev))
    else:
        t, off = target.contiguous().float(), offsets.contiguous().long()
        rc = native.cuda_lib().cb_pair_metric(_p(a), _p(t), _p(off), int(off.numel()) - 1, None, None, 0, _p(out), _stream(dev))
    native.cuda_check(rc, "cb_pair_metric")
    l, w, c = (float(v) for v in out.tolist())
    return (l / w if w > 0 else 0.0), (c / w if w > 0 else 1.0)


def pair_logit_der(approx: torch.Tensor, pairs: torch.Tensor, pair_weight):
    """(der, hess) [n] of PairLogit from explicit (winner, loser) pairs [P, 2] (int64) on the GPU."""
    dev = approx.device
    n = int(approx.shape[0])
    a = approx.contiguous().float()
    pr = pairs.contiguous().long()
    pw = None if pair_weight is None else pair_weight.contiguous().float()
    der, hess = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    native.cuda_check(native.cuda_lib().cb_pair_logit_pairs_der(_p(a), _p(pr), _p(pw), int(pr.shape[0]), _p(der), _p(hess),
                                                                _stream(dev)), "cb_pair_logit_pairs_der")
    return der, hess.clamp_min_(1e-16)


_SCORE_FN_ID = {"Cosine": 0, "NewtonCosine": 0, "L2": 1, "NewtonL2": 1, "SolarL2": 2, "LOOL2": 3, "SatL2": 4}


def leaf_search(store: BinnedStore, hist_: torch.Tensor, K: int, l2: float, score_function: str, noise_std: float = 0.0,
                seed: int = 0, leaf_id: Optional[torch.Tensor] = None, fmask: Optional[torch.Tensor] = None,
                min_data: float = 0.0):
    """Best split of every leaf from its complete histogram ``hist_[leaf, S, TB]`` (K derivative columns, the weight
    column, optionally a document-count column) on the GPU: ``(score, feature, bin, gain)`` arrays on the host, feature
    -1 where a leaf has no admissible candidate.  One warp per (leaf, feature), then one warp per leaf."""
    dev = store.bins.device
    nleaf, S = int(hist_.shape[0]), int(hist_.shape[1])
    F = store.F
    sc = torch.empty((nleaf, F), dtype=torch.float32, device=dev)
    bn = torch.empty((nleaf, F), dtype=torch.int32, device=dev)
    gn = torch.empty((nleaf, F), dtype=torch.float32, device=dev)
    best = torch.empty((nleaf, 4), dtype=torch.float32, device=dev)
    fm = None if fmask is None else fmask.to(torch.float32).contiguous()
    lid = None if leaf_id is None else leaf_id.to(torch.int32).contiguous()
    native.cuda_check(native.cuda_lib().cb_leaf_search(
        ctypes.c_void_p(store.handle), _p(hist_.contiguous()), nleaf, S, int(K), float(l2), _SCORE_FN_ID[score_function],
        float(noise_std), int(seed) & 0xFFFFFFFFFFFFFFFF, _p(lid), _p(fm), float(min_data), _p(sc), _p(bn), _p(gn), _p(best),
        _stream(dev)), "cb_leaf_search")
    b = best.cpu()
    ints = b.view(torch.int32)
    return b[:, 0].numpy(), ints[:, 1].numpy(), ints[:, 2].numpy(), b[:, 3].numpy()


def hist_reference(store: BinnedStore, leaf: torch.Tensor, stats: torch.Tensor, slot_table: torch.Tensor,
                   nslots: int) -> torch.Tensor:
    n, S, TB = store.n, stats.shape[0], store.TB
    out = torch.zeros((nslots, S, TB), dtype=torch.float32, device=store.bins.device)
    slot = slot_table.long()[(leaf[:n].long() & 0xFFFF)]
    keep = slot >= 0
    flat = out.view(nslots * S, TB)
    for f in range(store.F):
        col = store.column(f).long() + int(store.feat_off_host[f])
        for s in range(S):
            idx = (slot[keep] * S + s) * TB + col[keep]
            flat.view(-1).index_add_(0, idx, stats[s, :n][keep])
    return out


def update_leaf(store: BinnedStore, leaf: torch.Tensor, feature: int, bin_: int, onehot: bool, level: int):
    """leaf |= (bin(feature) > bin_) << level   (one-hot: ==)."""
    dev = store.bins.device
    if dev.type == "cpu":
        native.cpu_lib().cbc_update_leaf(_p(store.bins), ctypes.c_longlong(store.npad), ctypes.c_longlong(store.n),
                                         ctypes.c_int(feature), ctypes.c_int(bin_), ctypes.c_int(1 if onehot else 0),
                                         ctypes.c_int(level), _p(leaf))
        return
    # the kernel reads splits[iter * depth + level]; place the record at index `level` of a (level+1)-deep tree
    recs = torch.zeros((level + 1, 4), dtype=torch.int32, device=dev)
    recs[:, 0] = -1
    recs[level] = torch.tensor([feature, bin_, 0, 1 if onehot else 0], dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    sm, _ = device_info(dev)
    native.cuda_check(native.cuda_lib().cb_update_leaf(ctypes.c_void_p(store.handle), _p(leaf), _p(recs), _p(zero),
                                                       level + 1, level, sm * 8, _stream(dev)), "cb_update_leaf")


def update_nodes(store: BinnedStore, leaf: torch.Tensor, node_split: torch.Tensor):
    """Non-symmetric step: node_split int32 [n_nodes, 4] = (feature, bin, flags, left_child); documents of a node
    with feature >= 0 move to left_child (+1 when the condition holds)."""
    dev = store.bins.device
    n_nodes = node_split.shape[0]
    if dev.type == "cpu":
        native.cpu_lib().cbc_update_nodes(_p(store.bins), ctypes.c_longlong(store.npad), ctypes.c_longlong(store.n),
                                          _p(node_split), ctypes.c_int(n_nodes), _p(leaf))
        return
    sm, _ = device_info(dev)
    native.cuda_check(native.cuda_lib().cb_update_nodes(ctypes.c_void_p(store.handle), _p(leaf), _p(node_split), n_nodes,
                                                        sm * 8, _stream(dev)), "cb_update_nodes")


def update_one_node(store: BinnedStore, leaf: torch.Tensor, node: int, feature: int, bin_: int, onehot: bool, left_child: int):
    """The documents of ``node`` move to ``left_child`` (+1 when the split condition holds); GPU only (the split travels as
    kernel arguments, nothing is uploaded)."""
    dev = store.bins.device
    sm, _ = device_info(dev)
    native.cuda_check(native.cuda_lib().cb_update_one_node(ctypes.c_void_p(store.handle), _p(leaf), int(node), int(feature),
                                                           int(bin_), 1 if onehot else 0, int(left_child), sm * 8,
                                                           _stream(dev)), "cb_update_one_node")


def leaf_index(store: BinnedStore, splits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Oblivious leaf index of every document for int32 split records [depth, 4] = (feature, bin, _, flags)."""
    dev = store.bins.device
    depth = splits.shape[0]
    if out is None:
        out = torch.zeros(store.npad, dtype=torch.int16, device=dev)
    if dev.type == "cpu":
        native.cpu_lib().cbc_leaf_index(_p(store.bins), ctypes.c_longlong(store.npad), ctypes.c_longlong(store.n),
                                        _p(splits.contiguous()), ctypes.c_int(depth), _p(out))
        return out
    sm, _ = device_info(dev)
    native.cuda_check(native.cuda_lib().cb_leaf_index(ctypes.c_void_p(store.handle), _p(out), _p(splits.contiguous()),
                                                      depth, sm * 8, _stream(dev)), "cb_leaf_index")
    return out


def leaf_index_reference(store: BinnedStore, splits) -> torch.Tensor:
    idx = torch.zeros(store.n, dtype=torch.long, device=store.bins.device)
    for k, (f, b, _, flags) in enumerate(np.asarray(splits).tolist()):
        if f < 0:
            continue
        col = store.column(f).long()
        bit = (col == b) if (flags & 1) else (col > b)
        idx |= bit.long() << k
    return idx


def leaf_sums(leaf: torch.Tensor, cols: torch.Tensor, L: int, n: int) -> torch.Tensor:
    """float64 [L, C]: per-leaf sums of the C columns ``cols`` [C, >= n]."""
    C = cols.shape[0]
    if leaf.device.type == "cpu":
        out = torch.zeros((L, C), dtype=torch.float64)
        cols = cols.contiguous()
        native.cpu_lib().cbc_leaf_sums(_p(leaf), ctypes.c_longlong(n), _p(cols), ctypes.c_longlong(cols.stride(0)),
                                       ctypes.c_int(C), ctypes.c_int(L), _p(out))
        return out
    idx = leaf[:n].long() & 0xFFFF
    out = torch.zeros((C, L), dtype=torch.float64, device=leaf.device)
    out.index_add_(1, idx, cols[:, :n].double())
    return out.t().contiguous()


# ---- CTR engine (ops/cuda/cb_ctr.cu) ---------------------------------------------------------------------------
CTR_MAX_SPECS = 16
CTR_MAX_TB = 4


def ctr_scan(sorted_h: torch.Tensor, rows: torch.Tensor, cls_u8: torch.Tensor, need_tb):
    """Segmented exclusive scans over documents sorted by (projection hash, permutation position).

    Returns (excl int32 [1 + len(need_tb), n] per sorted position, seg_id int32 [n], distinct hashes int64 [U],
    per-segment totals int32 [1 + len(need_tb), U])."""
    lib = native.cuda_lib()
    dev = sorted_h.device
    n = int(sorted_h.shape[0])
    nb = len(need_tb)
    if nb > CTR_MAX_TB:
        raise ValueError(f"at most {CTR_MAX_TB} target borders per projection")
    C = 1 + nb
    tile, agg = lib.cb_ctr_tile(), lib.cb_ctr_agg_bytes()
    excl = torch.empty((C, n), dtype=torch.int32, device=dev)
    seg_id = torch.empty(n, dtype=torch.int32, device=dev)
    open_ = torch.empty(n, dtype=torch.uint8, device=dev)
    tile_agg = torch.empty(((n + tile - 1) // tile) * agg, dtype=torch.uint8, device=dev)
    uniq = torch.empty(n, dtype=torch.int64, device=dev)
    totals = torch.empty((C, n), dtype=torch.int32, device=dev)
    nseg = torch.zeros(1, dtype=torch.int32, device=dev)
    tb = (ctypes.c_int * max(1, nb))(*[int(t) for t in need_tb])
    with torch.cuda.device(dev):
        native.cuda_check(lib.cb_ctr_scan(_p(sorted_h.contiguous()), _p(rows.contiguous()), _p(cls_u8.contiguous()),
                                          ctypes.c_longlong(n), ctypes.c_int(nb), tb, _p(excl), _p(seg_id), _p(open_),
                                          _p(tile_agg), _p(uniq), _p(totals), _p(nseg), _stream(dev)), "cb_ctr_scan")
    U = int(nseg.item())
    return excl, seg_id, uniq[:U].clone(), totals[:, :U].contiguous()


def _ctr_spec_arrays(descs):
    S = len(descs)
    ci = (ctypes.c_int * S)
    cf = (ctypes.c_float * S)
    return (ci(*[int(d[0]) for d in descs]), ci(*[int(d[1]) for d in descs]), cf(*[float(d[2]) for d in descs]),
            cf(*[float(d[3]) for d in descs]), cf(*[float(d[4]) for d in descs]))


def ctr_minmax(descs, excl, totals, seg_id):
    """[(min, max)] of the CTR values of ``descs`` over all documents (float32)."""
    lib = native.cuda_lib()
    dev = excl.device
    S = len(descs)
    if S == 0:
        return []
    mm = torch.tensor([-1, 0] * S, dtype=torch.int32, device=dev)       # bit patterns: min starts at all ones, max at 0
    kind, col, pn, pd, den = _ctr_spec_arrays(descs)
    n = int(excl.shape[1])
    # the kernel reads only row 0 of ``totals`` (the counts), so the row stride does not matter
    with torch.cuda.device(dev):
        native.cuda_check(lib.cb_ctr_minmax(ctypes.c_int(S), kind, col, pn, pd, den, _p(excl), _p(totals), _p(seg_id),
                                            ctypes.c_longlong(n), _p(mm), _stream(dev)), "cb_ctr_minmax")
    vals = mm.cpu().numpy().view(np.float32)
    return [(np.float32(vals[2 * s]), np.float32(vals[2 * s + 1])) for s in range(S)]


def ctr_binarize(descs, borders, excl, totals, seg_id, rows, row_lo: int, n_out: int) -> torch.Tensor:
    """uint8 [len(descs), n_out]: border bucket of every CTR for documents row_lo .. row_lo + n_out."""
    lib = native.cuda_lib()
    dev = excl.device
    S = len(descs)
    out = torch.empty((S, n_out), dtype=torch.uint8, device=dev)
    if S == 0 or n_out == 0:
        return out
    kind, col, pn, pd, den = _ctr_spec_arrays(descs)
    offs, cnts, flat = [], [], []
    for b in borders:
        offs.append(len(flat))
        cnts.append(len(b))
        flat.extend(float(x) for x in b)
    bt = torch.tensor(flat, dtype=torch.float32, device=dev)
    n = int(excl.shape[1])
    with torch.cuda.device(dev):
        native.cuda_check(lib.cb_ctr_binarize(ctypes.c_int(S), kind, col, pn, pd, den, (ctypes.c_int * S)(*offs),
                                              (ctypes.c_int * S)(*cnts), _p(bt), ctypes.c_int(len(flat)), _p(excl),
                                              _p(totals), _p(seg_id), _p(rows.contiguous()), ctypes.c_longlong(n),
                                              ctypes.c_longlong(row_lo), ctypes.c_longlong(n_out), _p(out), _stream(dev)),
                          "cb_ctr_binarize")
    return out
