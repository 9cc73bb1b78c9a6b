// Stable least-significant-digit radix sort of (int64 key, int32 value) pairs, 8 bits per pass, written for the CTR
// engine: the keys are projection hashes taken in permutation order and the sort has to keep that order inside a
// group of equal hashes (catboost/cuda/ctrs/ctr_bins_builder.h:217-245 sorts the same pairs with a library radix sort,
// catboost/cuda/cuda_util/kernel/sort_templ.cuh:10-39).
//
// One pass = three launches:
//   count   one warp per tile of CB_SORT_TILE consecutive elements counts its digits  -> counts[digit][tile]
//   scan    block d turns row d into exclusive offsets and leaves the row total        -> counts (in place), totals[d]
//           (+ one small block that turns the 256 totals into digit bases)
//   scatter the warp of a tile walks its elements 32 at a time in order; lanes with equal digits find each other with
//           match.any, the lowest of them advances the tile's running offset of that digit, and every lane writes its
//           pair to offset + its rank inside the group -- elements of equal digit keep their order, so the sort is stable.
// Keys are ordered as signed integers (the top byte is biased in the last pass).
#include "cb_common.cuh"

#define CB_SORT_TILE 2048          // elements per warp tile
#define CB_SORT_WARPS 8            // tiles per block

__device__ __forceinline__ unsigned int cb_sort_digit(long long key, int shift) {
    unsigned int d = (unsigned int)(((unsigned long long)key >> shift) & 255ull);
    return shift == 56 ? d ^ 0x80u : d;
}

__global__ void __launch_bounds__(CB_SORT_WARPS * 32) cb_sort_count_kernel(const long long* keys, long long n, int shift,
                                                                           long long ntiles, unsigned int* counts) {
    __shared__ unsigned int cnt[CB_SORT_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long tile = (long long)blockIdx.x * CB_SORT_WARPS + warp;
    for (int d = lane; d < 256; d += 32) cnt[warp][d] = 0u;
    __syncwarp();
    if (tile < ntiles) {
        const long long b = tile * CB_SORT_TILE, e = min(n, b + CB_SORT_TILE);
        for (long long i = b + lane; i < e; i += 32) atomicAdd(&cnt[warp][cb_sort_digit(keys[i], shift)], 1u);
        __syncwarp();
        for (int d = lane; d < 256; d += 32) counts[(size_t)d * ntiles + tile] = cnt[warp][d];
    }
}

// Block d: exclusive scan of counts[d][0 .. ntiles) in place; totals[d] = row sum.
__global__ void __launch_bounds__(256) cb_sort_scan_rows_kernel(unsigned int* counts, long long ntiles, unsigned int* totals) {
    __shared__ unsigned int warp_sum[8];
    __shared__ unsigned int carry;
    unsigned int* row = counts + (size_t)blockIdx.x * ntiles;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0u;
    __syncthreads();
    for (long long base = 0; base < ntiles; base += 256) {
        const long long i = base + threadIdx.x;
        const unsigned int v = i < ntiles ? row[i] : 0u;
        unsigned int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_sum[warp] = inc;
        __syncthreads();
        unsigned int before = carry;
        for (int w = 0; w < warp; ++w) before += warp_sum[w];
        if (i < ntiles) row[i] = before + inc - v;
        __syncthreads();
        if (threadIdx.x == 255) carry = before + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

// One block: totals[256] -> exclusive digit bases (64-bit: n may exceed 2^32 in principle, offsets of a tile do not).
__global__ void __launch_bounds__(256) cb_sort_scan_totals_kernel(const unsigned int* totals, unsigned long long* bases) {
    __shared__ unsigned long long s[256];
    s[threadIdx.x] = totals[threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long run = 0ull;
        for (int d = 0; d < 256; ++d) { const unsigned long long v = s[d]; s[d] = run; run += v; }
    }
    __syncthreads();
    bases[threadIdx.x] = s[threadIdx.x];
}

__global__ void __launch_bounds__(CB_SORT_WARPS * 32) cb_sort_scatter_kernel(const long long* keys_in, const int* vals_in,
                                                                             long long n, int shift, long long ntiles,
                                                                             const unsigned int* within,
                                                                             const unsigned long long* bases,
                                                                             long long* keys_out, int* vals_out) {
    __shared__ unsigned long long off[CB_SORT_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long tile = (long long)blockIdx.x * CB_SORT_WARPS + warp;
    if (tile >= ntiles) return;
    for (int d = lane; d < 256; d += 32) off[warp][d] = bases[d] + (unsigned long long)within[(size_t)d * ntiles + tile];
    __syncwarp();
    const long long b = tile * CB_SORT_TILE, e = min(n, b + CB_SORT_TILE);
    const unsigned int lt = (1u << lane) - 1u;
    for (long long i0 = b; i0 < e; i0 += 32) {
        const long long i = i0 + lane;
        const bool live = i < e;
        const long long key = live ? keys_in[i] : 0ll;
        const int val = live ? (vals_in ? vals_in[i] : (int)i) : 0;
        // dead lanes get a digit of their own (256 + lane) so that they match nobody
        const unsigned int d = live ? cb_sort_digit(key, shift) : 256u + (unsigned int)lane;
        const unsigned int peers = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(peers) - 1;
        unsigned long long start = 0ull;
        if (live && lane == leader) {
            start = off[warp][d];
            off[warp][d] = start + (unsigned long long)__popc(peers);
        }
        start = __shfl_sync(0xffffffffu, start, leader);
        if (live) {
            const unsigned long long dst = start + (unsigned long long)__popc(peers & lt);
            keys_out[dst] = key;
            vals_out[dst] = val;
        }
        __syncwarp();
    }
}

CB_API long long cb_sort_scratch_bytes(long long n) {
    const long long ntiles = (n + CB_SORT_TILE - 1) / CB_SORT_TILE;
    return 256ll * ntiles * 4 + 256 * 4 + 256 * 8 + 256;
}

// Sorts n pairs.  keys_a / vals_a hold the input (vals_a may be null: the values are then the positions 0 .. n-1) and
// are overwritten; keys_b / vals_b are work buffers of the same size.  After the 8 passes the result is back in the _a
// buffers.  scratch: cb_sort_scratch_bytes(n) bytes.  Returns 0 or a CUDA error code.
CB_API int cb_sort_pairs_i64(long long* keys_a, int* vals_a, long long* keys_b, int* vals_b, long long n, void* scratch,
                             int first_values_are_positions, cudaStream_t st) {
    if (n <= 0) return 0;
    const long long ntiles = (n + CB_SORT_TILE - 1) / CB_SORT_TILE;
    unsigned int* counts = reinterpret_cast<unsigned int*>(scratch);
    unsigned int* totals = counts + 256ll * ntiles;
    unsigned long long* bases = reinterpret_cast<unsigned long long*>(
        (reinterpret_cast<uintptr_t>(totals + 256) + 255) & ~(uintptr_t)255);
    const unsigned int blocks = (unsigned int)((ntiles + CB_SORT_WARPS - 1) / CB_SORT_WARPS);
    long long* kin = keys_a; long long* kout = keys_b;
    int* vin = vals_a; int* vout = vals_b;
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = pass * 8;
        cb_sort_count_kernel<<<blocks, CB_SORT_WARPS * 32, 0, st>>>(kin, n, shift, ntiles, counts);
        cb_sort_scan_rows_kernel<<<256, 256, 0, st>>>(counts, ntiles, totals);
        cb_sort_scan_totals_kernel<<<1, 256, 0, st>>>(totals, bases);
        cb_sort_scatter_kernel<<<blocks, CB_SORT_WARPS * 32, 0, st>>>(
            kin, (pass == 0 && first_values_are_positions) ? nullptr : vin, n, shift, ntiles, counts, bases, kout, vout);
        long long* tk = kin; kin = kout; kout = tk;
        int* tv = vin; vin = vout; vout = tv;
    }
    return (int)cudaGetLastError();
}
