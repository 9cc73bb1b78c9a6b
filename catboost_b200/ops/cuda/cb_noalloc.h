// Leaf-estimation pass for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library that cannot call
// cudaMalloc themselves and cannot let the library do it either: code running inside a memory pool that owns the
// whole device (an inference server or a training framework that pre-reserved all free memory, so a fresh
// allocation fails or fragments the pool), and code on a path where an allocation would be a synchronisation point
// it cannot afford.  Such a caller still owns its inputs and outputs; what it lacks is the scratch that
// cb_leaf_pass needs between its blocks (per-leaf partial sums and the block counter).
//
// cb_leaf_pass_noalloc is cb_leaf_pass with that scratch taken from a fixed array that lives in the library's own
// device image: CB_NOALLOC_MAX_LEAVES * 3 doubles plus one counter (about 96 KiB).  Every GPU that loads the
// library holds the array until the process exits.
//
// Rules of use:
//   * L (number of leaves) must be <= CB_NOALLOC_MAX_LEAVES; a larger L is rejected with CB_NOALLOC_TOO_LARGE and a
//     message from cb_noalloc_last_error().  Nothing is launched in that case.
//   * The first call on each device looks up the address of the array (cudaGetSymbolAddress) with that device current.
//     Make that first call outside of any stream capture.
//   * The array is shared by all calls on a device and keeps what the last call left in it.  Each call clears the part
//     it uses on the caller's stream before launching, so calls on one stream are safe back to back; two calls that
//     can overlap on the GPU (different streams, no dependency) race on the array and must be ordered by the caller.
//   * Not thread-safe: the per-device address cache and the error text are plain process-wide variables.  A host with
//     several threads serialises its calls (one lock around cb_leaf_pass_noalloc and cb_noalloc_last_error); in
//     particular two threads must not make the first call on a device at the same time.
//   * Devices with an ordinal of 64 or more are rejected with CB_NOALLOC_SETUP_FAILED.
//   * No cudaMalloc, cudaFree or other allocating routine is called.  Single-GPU only (no peer exchange).
#pragma once
#include <cuda_runtime.h>

#define CB_NOALLOC_MAX_LEAVES 4096
#define CB_NOALLOC_TOO_LARGE (-2)
#define CB_NOALLOC_SETUP_FAILED (-3)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as cb_leaf_pass, without the scratch pointers (sums, counter) and without a communicator.
// Returns 0, a cudaError_t value (> 0) of the failing runtime call, or one of the negative codes above.
int cb_leaf_pass_noalloc(int loss, float p0, float p1, const float* approx, const float* target, const float* weight,
                         const unsigned short* leaf, const float* ext_der, const float* ext_hess, long long n, int L,
                         float* delta, int first, int last, int newton, float l2, float lr, float* cur_vals,
                         float* model_vals, float* model_wts, int Lstride, const int* iter_ptr, float* leaf_w, int grid,
                         cudaStream_t stream);

// Text of the last error reported by cb_leaf_pass_noalloc in this process ("" when there was none).
const char* cb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
