// Batch apply of an oblivious-tree ensemble that uses many features (hundreds): no quantisation step at all.
//
// A split "bin of feature f > k" is the same test as "value of f > border k of f", so a row can be evaluated from its
// raw float values.  The narrow-model kernel (cb_predict_kernel) first turns every used feature of a row into a bin by
// a binary search over its borders -- 7 shared-memory reads per (row, used feature), which for a 700-feature model is
// 4900 reads per row before the first tree is walked, more than the 1200 reads the 200 trees themselves need.  Here the
// float values of a tile of 16 rows sit in shared memory (row stride odd, so that lanes on different rows never share a
// bank) next to the whole split table (column, border), the tree table and, when they fit, all leaf values.  A lane is
// (row, half); the 32 (warp, half) pairs of a group deal the trees among themselves, a lane adds the leaf values of its
// row over its trees, and the partial sums are added in a fixed order.  The reference's GPU evaluator quantises into a
// byte buffer in one kernel and walks the trees in a second (catboost/libs/model/cuda/evaluator.cu:85-343).
//
// Persistent blocks (one per SM, 1024 threads) in two groups of 16 warps.  The model is staged once per block; each
// group takes its own row tiles in a grid-stride loop with its own buffer and its own named barrier, so while one group
// waits for its rows (a warp reads one row with up to 24 independent 128-byte requests in flight) the other one walks
// trees.  Measured on a 700-feature, 200-tree model, rows resident on the device: 1.5e8 rows/s with the quantising
// kernel, 6.1e8 with one 32-row tile per block and no overlap.
#include "cb_common.cuh"

#define CB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

struct CbPredictWideArgs {
    const float* X; long long n; long long ldx; int F;     // F leading columns of a row are staged
    const unsigned char* col_nanmax;   // [F] 1: a NaN in this column counts as +inf (largest bin), else as the smallest; or null
    const int* tree_depth;             // [T]
    const int* tree_split_off;         // [T]
    const int* split_col;              // [S] column of X
    const float* split_border;         // [S] go right when value > border
    const long long* tree_leaf_off;    // [T] first leaf value (in units of dims)
    const float* leaf_vals;            // [sum leaves][dims]
    int T, S, dims;
    long long total_leaf_floats;       // all leaf values * dims
    int stage_leaves;                  // 1: all leaf values sit in shared memory
    float scale; const float* bias;
    float* out;                        // [dims][n]
};

#ifndef CB_PW_NG
#define CB_PW_NG 2               // groups per block
#endif
#define CB_PW_GW (32 / CB_PW_NG) // warps per group
#ifndef CB_PW_ROWS
#define CB_PW_ROWS 32            // rows per tile (32: one per lane; 16 or 8: several lanes share a row and split the trees)
#endif
#define CB_PW_SUB (32 / CB_PW_ROWS)   // lanes of a warp that share a row (each takes its own trees)
#define CB_PW_NSL (CB_PW_GW * CB_PW_SUB)   // tree slices of a group
#define CB_PW_BATCH 24

__device__ __forceinline__ void cb_pw_group_sync(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(CB_PW_GW * 32) : "memory");
}

template <bool NANMAX, int DEPTH>
__device__ __forceinline__ int cb_pw_leaf(const CbPredictWideArgs& a, const float2* sp, const float* xrow, int depth) {
    int leaf = 0;
    if (DEPTH > 0) {
        // all levels at once: the split entries, then the values, are independent loads
        float2 e[DEPTH > 0 ? DEPTH : 1];
#pragma unroll
        for (int k = 0; k < DEPTH; ++k) e[k] = sp[k];
#pragma unroll
        for (int k = 0; k < DEPTH; ++k) {
            const int c = __float_as_int(e[k].x);
            const float v = xrow[c];
            bool right = v > e[k].y;
            if (NANMAX) right = right || (v != v && a.col_nanmax[c]);
            leaf |= right << k;
        }
    } else {
        for (int k = 0; k < depth; ++k) {
            const float2 e = sp[k];
            const int c = __float_as_int(e.x);
            const float v = xrow[c];
            bool right = v > e.y;
            if (NANMAX) right = right || (v != v && a.col_nanmax[c]);
            leaf |= right << k;
        }
    }
    return leaf;
}

template <bool NANMAX>
__global__ void __launch_bounds__(1024, 1) cb_predict_wide_kernel(CbPredictWideArgs a) {
    extern __shared__ __align__(16) unsigned char sw[];
    const int XS = a.F | 1;                                   // odd row stride in floats
    float* xs_all = reinterpret_cast<float*>(sw);             // [groups][CB_PW_ROWS][XS]
    float2* s_split = reinterpret_cast<float2*>(xs_all + ((CB_PW_NG * CB_PW_ROWS * XS + 1) & ~1));   // [S] (column bits, border)
    int* s_tree = reinterpret_cast<int*>(s_split + a.S);      // [T][2]: depth | first split << 8, first leaf value (floats)
    float* s_part_all = reinterpret_cast<float*>(s_tree + 2 * a.T);       // [groups][slices][dims][CB_PW_ROWS]
    float* s_lv = s_part_all + CB_PW_NG * CB_PW_NSL * a.dims * CB_PW_ROWS;  // [total_leaf_floats] when staged
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / CB_PW_GW, gw = warp % CB_PW_GW, gtid = threadIdx.x - group * CB_PW_GW * 32;
    const int row = lane & (CB_PW_ROWS - 1), sub = lane / CB_PW_ROWS;
    const int slice = gw * CB_PW_SUB + sub;                   // this lane's trees: slice, slice + CB_PW_NSL, ...
    const int dims = min(a.dims, 8);
    for (int i = threadIdx.x; i < a.S; i += 1024)
        s_split[i] = make_float2(__int_as_float(a.split_col[i]), a.split_border[i]);
    for (int i = threadIdx.x; i < a.T; i += 1024) {
        s_tree[2 * i] = a.tree_depth[i] | (a.tree_split_off[i] << 8);
        s_tree[2 * i + 1] = (int)(a.tree_leaf_off[i] * a.dims);
    }
    if (a.stage_leaves)
        for (long long i = threadIdx.x; i < a.total_leaf_floats; i += 1024) s_lv[i] = __ldg(a.leaf_vals + i);
    __syncthreads();
    float* xs = xs_all + group * CB_PW_ROWS * XS;
    float* s_part = s_part_all + group * CB_PW_NSL * a.dims * CB_PW_ROWS;
    const long long ntiles = (a.n + CB_PW_ROWS - 1) / CB_PW_ROWS;
    for (long long tile = (long long)blockIdx.x * CB_PW_NG + group; tile < ntiles; tile += (long long)CB_PW_NG * gridDim.x) {
        const long long row0 = tile * CB_PW_ROWS;
        const int nrow = (int)min((long long)CB_PW_ROWS, a.n - row0);
        // stage the rows: a warp takes whole rows, lanes along the columns.  (The previous tile's readers of this buffer
        // passed the group barrier after their tree walk.)
        for (int r = gw; r < nrow; r += CB_PW_GW) {
            const float* src = a.X + (row0 + r) * a.ldx;
            float* dst = xs + r * XS;
            for (int c0 = lane; c0 < a.F; c0 += 32 * CB_PW_BATCH) {
                float v[CB_PW_BATCH];
#pragma unroll
                for (int q = 0; q < CB_PW_BATCH; ++q) v[q] = (c0 + 32 * q < a.F) ? __ldcs(src + c0 + 32 * q) : 0.0f;
#pragma unroll
                for (int q = 0; q < CB_PW_BATCH; ++q)
                    if (c0 + 32 * q < a.F) dst[c0 + 32 * q] = v[q];
            }
        }
        cb_pw_group_sync(group);
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
        const float* xrow = xs + (row < nrow ? row : 0) * XS;
        if (a.stage_leaves) {
            for (int tt = slice; tt < a.T; tt += CB_PW_NSL) {
                const int2 td = *reinterpret_cast<const int2*>(s_tree + 2 * tt);
                const int depth = td.x & 255;
                const float2* sp = s_split + (td.x >> 8);
                const int leaf = depth == 6 ? cb_pw_leaf<NANMAX, 6>(a, sp, xrow, depth) : cb_pw_leaf<NANMAX, 0>(a, sp, xrow, depth);
                const int lo = td.y + leaf * a.dims;
                for (int k = 0; k < dims; ++k) acc[k] += s_lv[lo + k];
            }
        } else {
            // leaf values through the read-only cache (the 64 values of a tree are two lines, shared by the 32 rows of the
            // warp); the values of a tree are added one tree later, so their latency hides under the next walk
            float pend[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pend[k] = 0.0f;
            for (int tt = slice; tt < a.T; tt += CB_PW_NSL) {
                const int2 td = *reinterpret_cast<const int2*>(s_tree + 2 * tt);
                const int depth = td.x & 255;
                const float2* sp = s_split + (td.x >> 8);
                const int leaf = depth == 6 ? cb_pw_leaf<NANMAX, 6>(a, sp, xrow, depth) : cb_pw_leaf<NANMAX, 0>(a, sp, xrow, depth);
                const int lo = td.y + leaf * a.dims;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k < dims) { acc[k] += pend[k]; pend[k] = __ldg(a.leaf_vals + lo + k); }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += pend[k];
        }
        for (int k = 0; k < dims; ++k) s_part[(slice * a.dims + k) * CB_PW_ROWS + row] = acc[k];
        cb_pw_group_sync(group);                              // partial sums complete; nobody reads the row buffer any more
        // eight threads per output: CB_PW_NSL / 8 partial sums each, then a fixed shuffle tree (the same order every time)
        for (int i = gtid; i < dims * CB_PW_ROWS * 8; i += CB_PW_GW * 32) {
            const int part = i & 7, l = (i >> 3) & (CB_PW_ROWS - 1), k = i / (8 * CB_PW_ROWS);
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < CB_PW_NSL / 8; ++w) t += s_part[((part * (CB_PW_NSL / 8) + w) * a.dims + k) * CB_PW_ROWS + l];
            t += __shfl_xor_sync(0xffffffffu, t, 1);
            t += __shfl_xor_sync(0xffffffffu, t, 2);
            t += __shfl_xor_sync(0xffffffffu, t, 4);
            if (part == 0 && l < nrow) a.out[(long long)k * a.n + row0 + l] = t * a.scale + (a.bias ? a.bias[k] : 0.0f);
        }
        // s_part is rewritten after the next tile's first group barrier, which these readers reach after this loop
    }
}

// ---- the same evaluation with the rows brought in by bulk copies (TMA, cp.async.bulk) -------------------------------
// One group of 32 warps; a tile is 16 rows; two row buffers.  Thread 0 issues one bulk copy per row (the whole row,
// F * 4 bytes, 16-byte aligned on both sides) against the buffer's mbarrier; all warps wait for the barrier's phase,
// walk the trees of the tile (64 (warp, half) slices) and, once every reader is past the block barrier, thread 0
// refills the buffer with the tile after next.  No thread spends instructions on the rows, and the copy of the next
// tile runs under the walk of the current one.  Row stride in shared memory: a multiple of 4 floats (alignment of the
// bulk copy) that is 4 modulo 8, so 16 rows fall into 8 banks (two-way conflicts at worst).
// Every wait on a barrier is bounded; on expiry the status word is set, the copies in flight get a second bounded wait,
// and the block returns.
#define CB_PW_TMA_TIMEOUT 0x61
#define CB_PWT_ROWS 16

__device__ __forceinline__ bool cb_pwt_wait(unsigned int bar, unsigned int parity, int limit) {
    for (int it = 0; it < limit; ++it) {
        unsigned int ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ void cb_pwt_issue(const CbPredictWideArgs& a, float* buf, int XS, unsigned int bar, long long tile) {
    const long long row0 = tile * CB_PWT_ROWS;
    const int nrow = (int)min((long long)CB_PWT_ROWS, a.n - row0);
    const unsigned int bytes = (unsigned int)a.F * 4u;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes * (unsigned int)nrow) : "memory");
    for (int r = 0; r < nrow; ++r) {
        const unsigned int dst = (unsigned int)__cvta_generic_to_shared(buf + r * XS);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(a.X + (row0 + r) * a.ldx), "r"(bytes), "r"(bar) : "memory");
    }
}

template <bool NANMAX>
__global__ void __launch_bounds__(1024, 1) cb_predict_wide_tma_kernel(CbPredictWideArgs a, int XS, int* status) {
    extern __shared__ __align__(16) unsigned char sw[];
    float* xs = reinterpret_cast<float*>(sw);                 // [2][CB_PWT_ROWS][XS]
    float2* s_split = reinterpret_cast<float2*>(xs + 2 * CB_PWT_ROWS * XS);      // [S]
    int* s_tree = reinterpret_cast<int*>(s_split + a.S);      // [T][2]
    float* s_part = reinterpret_cast<float*>(s_tree + 2 * a.T);                  // [2][64 slices][dims][CB_PWT_ROWS]
    float* s_lv = s_part + 2 * 64 * a.dims * CB_PWT_ROWS;     // [total_leaf_floats] when staged
    __shared__ __align__(8) unsigned long long s_bar[2];
    __shared__ int s_fail;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = lane & (CB_PWT_ROWS - 1), half = lane >> 4;
    const int slice = warp * 2 + half;                        // this lane's trees: slice, slice + 64, ...
    const int dims = min(a.dims, 8);
    const unsigned int bar0 = (unsigned int)__cvta_generic_to_shared(&s_bar[0]);
    const unsigned int bar1 = (unsigned int)__cvta_generic_to_shared(&s_bar[1]);
    const long long ntiles = (a.n + CB_PWT_ROWS - 1) / CB_PWT_ROWS;
    if (threadIdx.x == 0) {
        s_fail = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if ((long long)blockIdx.x < ntiles) cb_pwt_issue(a, xs, XS, bar0, blockIdx.x);
        if ((long long)blockIdx.x + gridDim.x < ntiles) cb_pwt_issue(a, xs + CB_PWT_ROWS * XS, XS, bar1, (long long)blockIdx.x + gridDim.x);
    }
    for (int i = threadIdx.x; i < a.S; i += 1024) s_split[i] = make_float2(__int_as_float(a.split_col[i]), a.split_border[i]);
    for (int i = threadIdx.x; i < a.T; i += 1024) {
        s_tree[2 * i] = a.tree_depth[i] | (a.tree_split_off[i] << 8);
        s_tree[2 * i + 1] = (int)(a.tree_leaf_off[i] * a.dims);
    }
    if (a.stage_leaves)
        for (long long i = threadIdx.x; i < a.total_leaf_floats; i += 1024) s_lv[i] = __ldg(a.leaf_vals + i);
    __syncthreads();
    unsigned int phase0 = 0u, phase1 = 0u;
    int b = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, b ^= 1) {
        const long long row0 = tile * CB_PWT_ROWS;
        const int nrow = (int)min((long long)CB_PWT_ROWS, a.n - row0);
        const unsigned int bar = b ? bar1 : bar0, parity = b ? phase1 : phase0;
        if (!cb_pwt_wait(bar, parity, 1 << 22)) {
            atomicExch(status, CB_PW_TMA_TIMEOUT);
            cb_pwt_wait(bar, parity, 1 << 22);                // a second bounded chance for the copies in flight to land
            s_fail = 1;
        }
        __syncthreads();
        if (s_fail) {
            cb_pwt_wait(b ? bar0 : bar1, b ? phase0 : phase1, 1 << 22);      // the other buffer's copies as well
            return;
        }
        if (b) phase1 ^= 1u; else phase0 ^= 1u;
        const float* xb = xs + b * CB_PWT_ROWS * XS;
        float* part = s_part + b * 64 * a.dims * CB_PWT_ROWS;
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
        const float* xrow = xb + (row < nrow ? row : 0) * XS;
        for (int tt = slice; tt < a.T; tt += 64) {
            const int2 td = *reinterpret_cast<const int2*>(s_tree + 2 * tt);
            const int depth = td.x & 255;
            const float2* sp = s_split + (td.x >> 8);
            const int leaf = depth == 6 ? cb_pw_leaf<NANMAX, 6>(a, sp, xrow, depth) : cb_pw_leaf<NANMAX, 0>(a, sp, xrow, depth);
            const int lo = td.y + leaf * a.dims;
            if (a.stage_leaves) {
                for (int k = 0; k < dims; ++k) acc[k] += s_lv[lo + k];
            } else {
                for (int k = 0; k < dims; ++k) acc[k] += __ldg(a.leaf_vals + lo + k);
            }
        }
        for (int k = 0; k < dims; ++k) part[(slice * a.dims + k) * CB_PWT_ROWS + row] = acc[k];
        __syncthreads();                                      // partial sums complete; nobody reads this row buffer any more
        if (threadIdx.x == 0 && tile + 2ll * gridDim.x < ntiles)
            cb_pwt_issue(a, xs + b * CB_PWT_ROWS * XS, XS, bar, tile + 2ll * gridDim.x);
        // eight threads per output: eight partial sums each, then a fixed shuffle tree (the same order every time)
        for (int i = threadIdx.x; i < dims * CB_PWT_ROWS * 8; i += 1024) {
            const int pp = i & 7, l = (i >> 3) & (CB_PWT_ROWS - 1), k = i / (8 * CB_PWT_ROWS);
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += part[((pp * 8 + w) * a.dims + k) * CB_PWT_ROWS + l];
            t += __shfl_xor_sync(0xffffffffu, t, 1);
            t += __shfl_xor_sync(0xffffffffu, t, 2);
            t += __shfl_xor_sync(0xffffffffu, t, 4);
            if (pp == 0 && l < nrow) a.out[(long long)k * a.n + row0 + l] = t * a.scale + (a.bias ? a.bias[k] : 0.0f);
        }
        // this buffer's partial sums are rewritten two tiles later, after the next tile's block barrier
    }
}

static size_t cb_predict_wide_tma_smem(int XS, int S, int T, int dims, long long leaf_floats) {
    return (size_t)2 * CB_PWT_ROWS * XS * 4 + (size_t)S * 8 + (size_t)T * 8 + (size_t)2 * 64 * dims * CB_PWT_ROWS * 4 +
           (size_t)leaf_floats * 4 + 16;
}

// Shared memory this kernel needs for F staged columns, S splits, `leaf_floats` staged leaf values (0 = not staged).
static size_t cb_predict_wide_smem(int F, int S, int T, int dims, long long leaf_floats) {
    return (size_t)((CB_PW_NG * CB_PW_ROWS * (F | 1) + 1) & ~1) * 4 + (size_t)S * 8 + (size_t)T * 8 + (size_t)CB_PW_NG * CB_PW_NSL * dims * CB_PW_ROWS * 4 + (size_t)leaf_floats * 4 + 16;
}

// 1 when the direct kernel can take this model (the row tile and the split table fit in shared memory).
CB_API int cb_predict_wide_fits(int F, int S, int T, int dims, long long total_leaf_floats) {
    return (dims >= 1 && dims <= 8 && S < (1 << 23) && total_leaf_floats < (1ll << 31) &&
            cb_predict_wide_smem(F, S, T, dims, 0) <= 224 * 1024) ? 1 : 0;
}

CB_API int cb_predict_oblivious_wide(const float* X, long long n, long long ldx, int F, const unsigned char* col_nanmax,
                                     const int* tree_depth, const int* tree_split_off, const int* split_col,
                                     const float* split_border, const long long* tree_leaf_off, const float* leaf_vals,
                                     int T, int S, int dims, long long total_leaf_floats, float scale, const float* bias,
                                     float* out, int* status, cudaStream_t st) {
    if (n <= 0) return 0;
    if (!cb_predict_wide_fits(F, S, T, dims, total_leaf_floats)) return (int)cudaErrorInvalidValue;
    const size_t lim = 224 * 1024;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // bulk-copy variant (CB200_PREDICT_WIDE_TMA=1; measured slower than the default on a 700-feature model: 7.9e8 against
    // 8.6e8 rows/s, its 16-byte aligned rows share shared-memory banks): whole rows must be 16-byte aligned pieces;
    // status = where a timed-out wait is reported
    bool tma = false;
    if (const char* e = getenv("CB200_PREDICT_WIDE_TMA")) tma = atoi(e) != 0;
    tma = tma && status != nullptr && (F & 3) == 0 && (ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0 && F >= 4;
    if (tma) {
        const int XS = F + ((4 - (F & 7)) & 7);               // multiple of 4, equal to 4 modulo 8
        if (cb_predict_wide_tma_smem(XS, S, T, dims, 0) <= lim) {
            const int stage_t = cb_predict_wide_tma_smem(XS, S, T, dims, total_leaf_floats) <= lim ? 1 : 0;
            const size_t smem_t = cb_predict_wide_tma_smem(XS, S, T, dims, stage_t ? total_leaf_floats : 0);
            static unsigned long long set_t = 0ull;
            if (cb_first_on_device(&set_t)) {
                cudaError_t e = cudaFuncSetAttribute(cb_predict_wide_tma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lim);
                if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_predict_wide_tma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lim);
                if (e != cudaSuccess) { cudaGetLastError(); set_t = 0ull; return (int)e; }
            }
            const long long ntiles_t = (n + CB_PWT_ROWS - 1) / CB_PWT_ROWS;
            const unsigned grid_t = (unsigned)(ntiles_t < sms ? ntiles_t : sms);
            CbPredictWideArgs at{X, n, ldx, F, col_nanmax, tree_depth, tree_split_off, split_col, split_border, tree_leaf_off,
                                 leaf_vals, T, S, dims, total_leaf_floats, stage_t, scale, bias, out};
            if (col_nanmax) cb_predict_wide_tma_kernel<true><<<grid_t, 1024, smem_t, st>>>(at, XS, status);
            else cb_predict_wide_tma_kernel<false><<<grid_t, 1024, smem_t, st>>>(at, XS, status);
            CB_LAUNCH_CHECK();
            return 0;
        }
    }
    const int stage = cb_predict_wide_smem(F, S, T, dims, total_leaf_floats) <= lim ? 1 : 0;
    const size_t smem = cb_predict_wide_smem(F, S, T, dims, stage ? total_leaf_floats : 0);
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_predict_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lim);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_predict_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lim);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    const long long ntiles = (n + CB_PW_ROWS - 1) / CB_PW_ROWS;
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);
    CbPredictWideArgs a{X, n, ldx, F, col_nanmax, tree_depth, tree_split_off, split_col, split_border, tree_leaf_off,
                        leaf_vals, T, S, dims, total_leaf_floats, stage, scale, bias, out};
    if (col_nanmax) cb_predict_wide_kernel<true><<<grid, 1024, smem, st>>>(a);
    else cb_predict_wide_kernel<false><<<grid, 1024, smem, st>>>(a);
    CB_LAUNCH_CHECK();
    return 0;
}
