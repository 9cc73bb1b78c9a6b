// Shared device helpers for the sm_100a kernels of catboost_b200.
//
// Conventions used by every kernel in this directory:
//   * bins      : uint32 [G][npad]   four one-byte feature bins per word (feature 4g+j in byte j),
//                                    feature-group-major so a group streams with coalesced 16-byte loads.
//   * stats     : float  [S][npad]   per-document statistic columns (weighted der, weight / hessian, ...).
//   * leaf      : uint16 [npad]      current leaf (or tree-node) index of each document.
//   * histogram : float  [slot][S][TB]  TB = sum over features of the padded bin count; feat_off[f] is the
//                                    first bin of feature f (always a multiple of 4 floats = 16 bytes).
// Documents are never re-ordered: a level streams all rows once per feature group and the leaf index picks
// the histogram slot, so the only random access is into shared memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define CB_API extern "C" __attribute__((visibility("default")))
#define CB_MAX_RANKS 8
#define CB_WARP 32

// ---- error / status words (device -> host), never a trap ------------------------------------------------
enum CbStatus : int {
    CB_OK = 0,
    CB_TIMEOUT_HIST_ARRIVE = 1,   // bounded wait for peers' histogram pushes ran out
    CB_TIMEOUT_MAILBOX = 2,       // bounded wait for a small all-reduce message ran out
    CB_BAD_ARGUMENT = 3,
};

// Per-rank view of the cross-GPU exchange arena.  Every pointer in `peer_*` is the address of rank r's
// buffer as mapped into THIS process (peer-to-peer over NVLink); index `rank` is the local buffer.
struct CbComm {
    int rank;
    int nranks;
    long long timeout_ns;            // bound of every device-side wait
    int* status;                     // local status words: [0]=code, [1]=detail (epoch/peer), sticky
    unsigned long long* epoch;       // local device counters: [0]=mailbox epoch, [1]=hist epoch
    // mailbox: [2 parity][nranks src][mbox_bytes] payload, then flags [2][nranks] (uint64 epoch tags)
    char* peer_mbox[CB_MAX_RANKS];
    unsigned long long* peer_mbox_flag[CB_MAX_RANKS];
    int mbox_bytes;
    // histogram slots: [nranks src][slot_floats] floats on each owner, plus arrive tags [nranks] (uint64)
    float* peer_slot[CB_MAX_RANKS];
    unsigned long long* peer_slot_flag[CB_MAX_RANKS];
    long long slot_floats;
};

__device__ __forceinline__ unsigned long long cb_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned long long cb_ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void cb_st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Bounded wait until *flag >= want.  Returns true on success; on timeout records the status and returns
// false so that the caller carries on (results are garbage, the host raises after reading the status).
__device__ __forceinline__ bool cb_wait_flag(const unsigned long long* flag, unsigned long long want,
                                             long long timeout_ns, int* status, int code, int detail) {
    unsigned long long t0 = cb_globaltimer();
    unsigned int spins = 0;
    while (cb_ld_acquire_sys(flag) < want) {
        if ((++spins & 63u) == 0) {
            if ((long long)(cb_globaltimer() - t0) > timeout_ns) {
                if (atomicCAS(status, CB_OK, code) == CB_OK) status[1] = detail;
                return false;
            }
        }
        __nanosleep(64);
    }
    return true;
}

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) belong to a device, not to the process:
// `seen` is one static word per call site with a bit per device ordinal; true the first time the current device asks.
static inline bool cb_first_on_device(unsigned long long* seen) {
    int dev = 0;
    cudaGetDevice(&dev);
    const unsigned long long bit = 1ull << (dev & 63);
    return (__atomic_fetch_or(seen, bit, __ATOMIC_ACQ_REL) & bit) == 0ull;
}

// float -> uint32 whose unsigned order equals the float order (NaN excluded by the callers)
__device__ __forceinline__ unsigned int cb_float_to_ordered(float x) {
    unsigned int u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float cb_ordered_to_float(unsigned int u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// counter-based RNG (splitmix64 finaliser); good enough for bootstrap weights and score noise
__host__ __device__ __forceinline__ unsigned long long cb_mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float cb_uniform01(unsigned long long h) {
    return ((unsigned int)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);   // (0,1)
}
__device__ __forceinline__ float cb_normal(unsigned long long h) {
    float u1 = cb_uniform01(h);
    float u2 = cb_uniform01(cb_mix64(h));
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.28318530718f * u2);
}

__device__ __forceinline__ float cb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double cb_warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
