"""The allocation-free leaf pass (cb_leaf_pass_noalloc) against the regular entry point (cb_leaf_pass).

Some hosts of the library cannot allocate device memory at call time -- they run inside a pool that already owns the
whole GPU, or on a path where an allocation would stall them -- so one entry point keeps its scratch in a fixed array
inside the library.  The test calls it through its exported C symbol, twice in a row (the two Newton passes of one
tree, which also proves that the second call is not disturbed by what the first left in the shared array), and checks
every output against the regular entry point fed with caller-allocated scratch.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from catboost_b200.ops import native
    native.cuda_lib()                                   # builds / loads the library the package uses
    lib = ctypes.CDLL(str(native.CUDA_LIB))
    vp, i, f, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    fn = lib.cb_leaf_pass_noalloc
    fn.restype = i
    fn.argtypes = [i, f, f, vp, vp, vp, vp, vp, vp, ll, i, vp, i, i, i, f, f, vp, vp, vp, i, vp, vp, i, vp]
    err = lib.cb_noalloc_last_error
    err.restype = ctypes.c_char_p
    return native.cuda_lib(), fn, err


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _compare_with_regular(n, L):
    lib, noalloc, last_error = _symbols()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    npad = (n + 255) // 256 * 256
    approx = torch.zeros(npad)
    approx[:n] = torch.randn(n, generator=g)
    target = torch.zeros(npad)
    target[:n] = (torch.rand(n, generator=g) < 0.4).float()
    weight = torch.zeros(npad)
    weight[:n] = torch.rand(n, generator=g) + 0.5
    leaf = torch.zeros(npad, dtype=torch.int16)
    leaf[:n] = torch.randint(0, L, (n,), generator=g).short()
    approx, target, weight, leaf = approx.to(dev), target.to(dev), weight.to(dev), leaf.to(dev)
    it = torch.zeros(1, dtype=torch.int32, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    grid = 2 * torch.cuda.get_device_properties(dev).multi_processor_count
    l2, lr = 3.0, 0.5

    def outputs():
        return dict(delta=torch.zeros(L, device=dev), cur=torch.zeros(L, device=dev), mv=torch.zeros((1, L), device=dev),
                    mw=torch.zeros((1, L), device=dev), lw=torch.zeros(L, device=dev))

    # plain fp32/fp64 restatement of one Newton pass at approx + shift[leaf], independent of both entry points
    idx = leaf[:n].long() & 0xFFFF

    def newton_step(shift):
        p = torch.sigmoid(approx[:n] + shift[idx])
        d = torch.zeros(L, dtype=torch.float64, device=dev).index_add_(0, idx, ((target[:n] - p) * weight[:n]).double())
        h = torch.zeros(L, dtype=torch.float64, device=dev).index_add_(0, idx, (p * (1 - p) * weight[:n]).double())
        return (d / (h + l2)).float()

    ref, got = outputs(), outputs()
    sums = torch.zeros(3 * L, dtype=torch.float64, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    step1 = newton_step(torch.zeros(L, device=dev))
    for first, last in ((1, 0), (0, 1)):                 # two calls in a row: both passes of a two-step Newton
        rc = lib.cb_leaf_pass(1, 0.0, 0.0, _p(approx), _p(target), _p(weight), _p(leaf), None, None, n, L,
                              _p(ref["delta"]), _p(sums), _p(counter), first, last, 1, l2, lr, _p(ref["cur"]),
                              _p(ref["mv"]), _p(ref["mw"]), L, _p(it), _p(ref["lw"]), None, grid, st)
        assert rc == 0
        rc = noalloc(1, 0.0, 0.0, _p(approx), _p(target), _p(weight), _p(leaf), None, None, n, L, _p(got["delta"]),
                     first, last, 1, l2, lr, _p(got["cur"]), _p(got["mv"]), _p(got["mw"]), L, _p(it), _p(got["lw"]),
                     grid, st)
        assert rc == 0, last_error().decode()
        torch.cuda.synchronize(dev)
        for k in ref:
            assert torch.allclose(ref[k], got[k], rtol=1e-4, atol=1e-5), (first, k, float((ref[k] - got[k]).abs().max()))
        if first:
            assert torch.allclose(got["delta"], step1, rtol=1e-4, atol=1e-5), float((got["delta"] - step1).abs().max())
    assert float(ref["delta"].abs().sum()) > 0 and float(ref["cur"].abs().sum()) > 0
    w = torch.zeros(L, dtype=torch.float64, device=dev).index_add_(0, idx, weight[:n].double())
    assert torch.allclose(got["lw"].double(), w, rtol=1e-4)
    want = lr * (step1 + newton_step(step1))
    assert torch.allclose(got["cur"], want, rtol=2e-4, atol=2e-5), float((got["cur"] - want).abs().max())
    assert torch.allclose(got["mv"][0], want, rtol=2e-4, atol=2e-5)


def test_noalloc_leaf_pass_matches_regular_entry_point():
    _compare_with_regular(50001, 64)


def test_noalloc_leaf_pass_at_the_largest_supported_size():
    # 4096 leaves: the whole built-in array is in use and the kernel runs with its smallest replica count
    _compare_with_regular(30011, 4096)


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    lib, noalloc, last_error = _symbols()
    dev = torch.device("cuda", 0)
    z = torch.zeros(256, device=dev)
    leaf = torch.zeros(256, dtype=torch.int16, device=dev)
    it = torch.zeros(1, dtype=torch.int32, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = noalloc(1, 0.0, 0.0, _p(z), _p(z), None, _p(leaf), None, None, 16, 4097, _p(z), 1, 1, 1, 3.0, 0.5, _p(z), None,
                 None, 4097, _p(it), _p(z), 8, st)
    assert rc == -2
    assert b"at most 4096" in last_error()
    torch.cuda.synchronize(dev)
