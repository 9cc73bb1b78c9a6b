"""Build and load the native libraries of catboost_b200.

Two shared objects live next to this file:

* ``libcb200_cuda.so`` -- the hand-written sm_100a kernels (``ops/cuda/*.cu``), compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``; plain C ABI, no torch headers, so a rebuild takes seconds.
* ``libcb200_cpu.so``  -- the OpenMP CPU backend (``ops/cpu/*.cpp``).

Both are loaded with :mod:`ctypes`; tensors are passed as raw pointers (``tensor.data_ptr()``) together with
the current CUDA stream handle, so every launch is asynchronous and can be captured in a CUDA graph.
On a machine with a GPU the CUDA library is mandatory: if it cannot be loaded the import fails loudly
instead of falling back to a slow path.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
from pathlib import Path

_HERE = Path(__file__).resolve().parent
CUDA_SRC = [_HERE / "cuda" / "cb_kernels.cu", _HERE / "cuda" / "cb_fused.cu", _HERE / "cuda" / "cb_leaf.cu",
            _HERE / "cuda" / "cb_quantize_tma.cu", _HERE / "cuda" / "cb_ranking.cu", _HERE / "cuda" / "cb_ctr.cu",
            _HERE / "cuda" / "cb_multiclass.cu", _HERE / "cuda" / "cb_search.cu", _HERE / "cuda" / "cb_pairwise.cu", _HERE / "cuda" / "cb_sort.cu", _HERE / "cuda" / "cb_mvs.cu", _HERE / "cuda" / "cb_predict_wide.cu", _HERE / "cuda" / "cb_querywise.cu",
            _HERE / "cuda" / "cb_knn_tc.cu"]
CUDA_HDR = sorted((_HERE / "cuda").glob("*.cuh")) + sorted((_HERE / "cuda").glob("*.h"))
CPU_SRC = [_HERE / "cpu" / "cb_cpu.cpp", _HERE / "cpu" / "cb_cityhash.h"]
MODEL_SRC = [_HERE / "cpu" / "cb_model_capi.cpp", _HERE / "cpu" / "cb_model_capi.h", _HERE / "cpu" / "cb_cityhash.h"]
CUDA_LIB = _HERE / "libcb200_cuda.so"
CPU_LIB = _HERE / "libcb200_cpu.so"
MODEL_LIB = _HERE / "libcb200model.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-shared",
]


def _newer(srcs, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.exists() and s.stat().st_mtime > t for s in srcs)


def _nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for p in ("/usr/local/cuda/bin/nvcc",):
        if os.path.exists(p):
            return p
    return None


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a into one shared object (cross-compiles without a GPU)."""
    srcs = [s for s in CUDA_SRC if s.exists()]
    if not force and not _newer(srcs + CUDA_HDR, CUDA_LIB):
        return CUDA_LIB
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(_HERE / "cuda"), *map(str, srcs), "-o", str(CUDA_LIB)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stderr)
    return CUDA_LIB


def build_cpu(force: bool = False) -> Path:
    if not force and not _newer(CPU_SRC, CPU_LIB):
        return CPU_LIB
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found: cannot build the CPU backend")
    cmd = [cxx, "-O3", "-march=x86-64-v3", "-std=c++17", "-fopenmp", "-fPIC", "-shared", str(CPU_SRC[0]),
           "-o", str(CPU_LIB)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return CPU_LIB


def build_model_lib(force: bool = False) -> Path:
    """The stand-alone evaluator with the C interface of ``cpu/cb_model_capi.h`` (no Python, torch or CUDA inside)."""
    if not force and not _newer(MODEL_SRC, MODEL_LIB):
        return MODEL_LIB
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found: cannot build the model evaluator")
    cmd = [cxx, "-O3", "-march=x86-64-v3", "-std=c++17", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden",
           str(MODEL_SRC[0]), "-o", str(MODEL_LIB)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return MODEL_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cpu(force)
    build_model_lib(force)
    build_cuda(force, verbose)


_cpu = None
_cuda = None

c_void_p, c_int, c_ll, c_float, c_ull, c_double = (ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float,
                                                  ctypes.c_ulonglong, ctypes.c_double)


def cpu_lib() -> ctypes.CDLL:
    """The CPU backend (built on first use if the tool chain is present)."""
    global _cpu
    if _cpu is None:
        if _newer(CPU_SRC, CPU_LIB):
            build_cpu()
        lib = ctypes.CDLL(str(CPU_LIB))
        lib.cbc_select_borders.restype = c_int
        lib.cbc_num_threads.restype = c_int
        lib.cbc_leaf_newton.restype = c_int
        _cpu = lib
    return _cpu


_SIGS = {
    # name: (restype, argtypes)
    "cb_quantize": (c_int, [c_void_p, c_ll, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_void_p]),
    "cb_pack_bins": (c_int, [c_void_p, c_ll, c_ll, c_int, c_int, c_void_p, c_ll, c_ll, c_void_p]),
    "cb_grad_pointwise": (c_int, [c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll,
                                  c_void_p, c_int, c_int, c_float, c_ull, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p]),
    "cb_data_create": (c_void_p, [c_void_p, c_ll, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int]),
    "cb_data_destroy": (None, [c_void_p]),
    "cb_comm_create": (c_void_p, [c_int, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_ll]),
    "cb_comm_destroy": (None, [c_void_p]),
    "cb_update_leaf": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cb_update_nodes": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "cb_update_one_node": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "cb_hist_smem_bytes": (c_int, [c_int, c_int, c_int]),
    "cb_hist": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                        c_int, c_int, c_void_p]),
    "cb_ctr_tile": (c_int, []),
    "cb_ctr_agg_bytes": (c_int, []),
    "cb_ctr_max_tb": (c_int, []),
    "cb_ctr_max_specs": (c_int, []),
    "cb_ctr_scan": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_ctr_minmax": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll,
                              c_void_p, c_void_p]),
    "cb_ctr_binarize": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_void_p, c_void_p]),
    "cb_hist_n": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                          c_void_p, c_int, c_int, c_void_p]),
    "cb_score": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_void_p, c_float, c_int, c_float, c_void_p, c_void_p, c_ull, c_float, c_void_p, c_void_p]),
    "cb_select_local_launch": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "cb_select_final_launch": (c_int, [c_void_p, c_void_p, c_int, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_void_p]),
    "cb_select_msg_bytes": (c_int, []),
    "cb_allreduce_sum": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
    "cb_leaf_pass": (c_int, [c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll,
                             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p,
                             c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cb_leaf_pass_q": (c_int, [c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll,
                               c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p,
                               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cb_quantize_tma": (c_int, [c_void_p, c_ll, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_void_p,
                                c_void_p]),
    "cb_yetirank_max_group": (c_int, []),
    "cb_yetirank": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_ll, c_int, c_float, c_ull, c_void_p, c_void_p,
                            c_void_p, c_int, c_void_p]),
    "cb_leaf_newton_max_grid": (c_int, [c_int]),
    "cb_leaf_newton": (c_int, [c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "cb_leaf_newton_sums_doubles": (c_int, [c_int]),
    "cb_leaf_newton_msg_bytes": (c_int, [c_int]),
    "cb_iter_end": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "cb_leaf_search": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_ull, c_void_p, c_void_p,
                               c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_pair_hist_floats": (c_ll, [c_int, c_int, c_int]),
    "cb_pair_hist_sorted": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                    c_void_p, c_float, c_void_p]),
    "cb_pair_chunk_pairs": (c_int, []),
    "cb_pair_hist": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_int,
                             c_void_p, c_void_p, c_float, c_int, c_void_p]),
    "cb_pair_scan": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "cb_pair_solve_smem_bytes": (c_int, [c_int]),
    "cb_pair_solve": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p]),
    "cb_sort_scratch_bytes": (c_ll, [c_ll]),
    "cb_sort_pairs_i64": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_void_p]),
    "cb_predict_wide_fits": (c_int, [c_int, c_int, c_int, c_int, c_ll]),
    "cb_predict_oblivious_wide": (c_int, [c_void_p, c_ll, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_float, c_void_p, c_void_p, c_void_p,
                                          c_void_p]),
    "cb_query_rmse_der": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p]),
    "cb_query_softmax_der": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_void_p, c_void_p, c_void_p]),
    "cb_pair_logit_pairs_der": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p]),
    "cb_pair_logit_labels_der": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p]),
    "cb_pair_metric": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_void_p, c_void_p]),
    "cb_knn_candidates": (c_int, []),
    "cb_knn_max_dim": (c_int, []),
    "cb_knn_splits": (c_int, [c_int, c_int]),
    "cb_knn_tc": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_mvs_block_docs": (c_int, []),
    "cb_mvs_sample": (c_int, [c_void_p, c_ll, c_ll, c_float, c_float, c_ull, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_mc_max_classes": (c_int, []),
    "cb_mc_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_void_p, c_int, c_int, c_float,
                           c_ull, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cb_mc_leaf_sums_doubles": (c_int, [c_int, c_int]),
    "cb_mc_leaf_msg_bytes": (c_int, [c_int, c_int]),
    "cb_mc_leaf_smem_bytes": (c_int, [c_int, c_int]),
    "cb_mc_leaf_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_float, c_int, c_void_p]),
    "cb_mc_metric": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cb_apply_tree_bins": (c_int, [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                   c_void_p]),
    "cb_leaf_index": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "cb_predict_oblivious": (c_int, [c_void_p, c_ll, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
                                     c_void_p, c_int, c_ll, c_void_p]),
    "cb_metric_sum": (c_int, [c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                             c_int, c_void_p]),
    "cb_device_info": (c_int, [c_void_p, c_void_p]),
    "cb_fused_create": (c_void_p, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int,
                                   c_float, c_void_p, c_void_p, c_ull, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "cb_fused_set_fuse_leaf": (None, [c_void_p, c_int]),
    "cb_fused_set_dominant": (None, [c_void_p, c_void_p]),
    "cb_fused_set_features": (None, [c_void_p, c_int, c_int]),
    "cb_fused_set_phase_ts": (None, [c_void_p, c_void_p]),
    "cb_fused_set_work": (None, [c_void_p, c_void_p]),
    "cb_fused_set_narrow": (None, [c_void_p, c_int, c_int]),
    "cb_fused_set_max_copies": (None, [c_void_p, c_int]),
    "cb_fused_set_priv": (None, [c_void_p, c_void_p, c_void_p]),
    "cb_fused_destroy": (None, [c_void_p]),
    "cb_fused_set_group_bins": (None, [c_void_p, c_void_p, c_int]),
    "cb_fused_geometry": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "cb_fused_launch": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_int, c_void_p]),
}


def cuda_lib() -> ctypes.CDLL:
    """The sm_100a kernel library.  Raises if it is missing: there is no eager fallback on a GPU box."""
    global _cuda
    if _cuda is None:
        if not CUDA_LIB.exists() or (_nvcc() is not None and _newer([s for s in CUDA_SRC if s.exists()] + CUDA_HDR,
                                                                     CUDA_LIB)):
            build_cuda()
        lib = ctypes.CDLL(os.environ.get("CB200_CUDA_LIB") or str(CUDA_LIB))     # the variable names another build to load
        for name, (res, args) in _SIGS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _cuda = lib
    return _cuda


def cuda_check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"CUDA launch of {what} failed with cudaError {code}")
