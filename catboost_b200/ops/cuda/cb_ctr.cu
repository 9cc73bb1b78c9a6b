// K11 / K12  CTR engine on the device (catboost/cuda/ctrs/kernel/ctr_calcers.cu, catboost/cuda/ctrs/ctr_calcers.h:32-285,
// catboost/cuda/gpu_data/batch_binarized_ctr_calcer.cpp:53-96).
//
// Input: the documents of one projection sorted by (projection hash, position in the learn permutation) -- `sorted_h[p]`
// is the hash and `rows[p]` the document at sorted position p.  Equal hashes are contiguous and keep permutation order,
// so the ordered target statistic of a document is a segmented exclusive prefix sum over this order:
//
//   cb_ctr_scan      segmented exclusive scans of the count column and of up to CB_CTR_MAX_TB class indicators
//                    (class > target border), the dense segment number of every position, the distinct hashes and the
//                    per-segment totals (the model's CTR table).  Three launches: tile-local scan with one aggregate per
//                    tile, scan of the aggregates in one block, fix-up.
//   cb_ctr_minmax    smallest / largest CTR value of every requested CTR over all documents (for uniform borders)
//   cb_ctr_binarize  value -> border bucket -> one byte per (CTR, document), scattered back to document order
//
// The reference reads the float CTR values back to the host and binarises there; here the values never leave registers.
// All arithmetic on values is IEEE float32 (explicit round-to-nearest intrinsics: the file is compiled with fast-math),
// so the buckets equal those of the tensor implementation bit for bit.
#include "cb_common.cuh"

#define CB_CTR_MAX_TB 4
#define CB_CTR_C (1 + CB_CTR_MAX_TB)
#define CB_CTR_THREADS 512
#define CB_CTR_ITEMS 8
#define CB_CTR_TILE (CB_CTR_THREADS * CB_CTR_ITEMS)
#define CB_CTR_MAX_SPECS 16

// ---- segmented-scan element: sums since the last segment start, whether a start was seen, how many starts ---------------
struct CbSeg {
    int s[CB_CTR_C];
    int flag;      // a segment start lies inside the span
    int starts;    // number of segment starts inside the span
};

template <int C>
__device__ __forceinline__ CbSeg cb_seg_combine(const CbSeg& a, const CbSeg& b) {     // a before b
    CbSeg r;
#pragma unroll
    for (int c = 0; c < C; ++c) r.s[c] = b.flag ? b.s[c] : a.s[c] + b.s[c];
    r.flag = a.flag | b.flag;
    r.starts = a.starts + b.starts;
    return r;
}

template <int C>
__device__ __forceinline__ CbSeg cb_seg_shfl_up(const CbSeg& v, int delta) {
    CbSeg r;
#pragma unroll
    for (int c = 0; c < C; ++c) r.s[c] = __shfl_up_sync(0xffffffffu, v.s[c], delta);
    r.flag = __shfl_up_sync(0xffffffffu, v.flag, delta);
    r.starts = __shfl_up_sync(0xffffffffu, v.starts, delta);
    return r;
}

// Exclusive scan of one CbSeg per thread over the block; returns the combination of all earlier threads (identity for
// thread 0) and leaves the block total in *total (valid in every thread).
template <int C>
__device__ CbSeg cb_seg_block_exclusive(CbSeg mine, CbSeg* warp_tot /* [32] shared */, CbSeg* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    CbSeg inc = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const CbSeg up = cb_seg_shfl_up<C>(inc, d);
        if (lane >= d) inc = cb_seg_combine<C>(up, inc);
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    CbSeg before;                                    // all earlier warps
#pragma unroll
    for (int c = 0; c < C; ++c) before.s[c] = 0;
    before.flag = 0;
    before.starts = 0;
    CbSeg all = before;
    for (int w = 0; w < nwarp; ++w) {
        if (w == warp) before = all;
        all = cb_seg_combine<C>(all, warp_tot[w]);
    }
    *total = all;
    CbSeg ex = cb_seg_shfl_up<C>(inc, 1);            // earlier lanes of this warp
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < C; ++c) ex.s[c] = 0;
        ex.flag = 0;
        ex.starts = 0;
    }
    __syncthreads();
    return cb_seg_combine<C>(before, ex);
}

struct CbCtrScanArgs {
    const long long* sorted_h;    // [n]
    const long long* rows;        // [n]
    const unsigned char* cls;     // [n documents] target class
    long long n;
    int nb;                       // indicator columns in use (<= CB_CTR_MAX_TB)
    int tb[CB_CTR_MAX_TB];        // indicator c: cls > tb[c]
    int* excl;                    // [1 + nb][n]   exclusive in-segment prefix per sorted position (final after phase C)
    int* seg_id;                  // [n]           phase A: 1-based start count inside the tile; phase C: dense segment number
    unsigned char* open;          // [n]           no segment start at or before the position inside its tile
    CbSeg* tile_agg;              // [tiles]       aggregate of every tile, after phase B the exclusive prefix over tiles
    long long* uniq;              // [n]           hash of every segment (first U entries used)
    int* totals;                  // [1 + nb][n]   per-segment totals (first U entries of every row used)
    int* n_segments;              // [1]
};

template <int C>
__device__ __forceinline__ void cb_ctr_values(const CbCtrScanArgs& a, long long p, int* v) {
    v[0] = 1;
    if (C > 1) {
        const int k = a.cls[a.rows[p]];
#pragma unroll
        for (int c = 1; c < C; ++c) v[c] = (c - 1 < a.nb && k > a.tb[c - 1]) ? 1 : 0;
    }
}

// phase A: tile-local scan
template <int C>
__global__ void __launch_bounds__(CB_CTR_THREADS) cb_ctr_scan_tiles(CbCtrScanArgs a) {
    __shared__ CbSeg warp_tot[32];
    const long long tile0 = (long long)blockIdx.x * CB_CTR_TILE;
    const long long p0 = tile0 + (long long)threadIdx.x * CB_CTR_ITEMS;
    int loc[CB_CTR_ITEMS][C];
    int loc_starts[CB_CTR_ITEMS];
    unsigned seen_mask = 0;                     // bit k: a start at or before item k inside this thread
    CbSeg mine;
#pragma unroll
    for (int c = 0; c < C; ++c) mine.s[c] = 0;
    mine.flag = 0;
    mine.starts = 0;
    long long prev_h = 0;
    if (p0 > 0 && p0 < a.n) prev_h = a.sorted_h[p0 - 1];
#pragma unroll
    for (int k = 0; k < CB_CTR_ITEMS; ++k) {
        const long long p = p0 + k;
        if (p < a.n) {
            const long long h = a.sorted_h[p];
            const bool start = p == 0 || h != prev_h;
            prev_h = h;
            if (start) {
#pragma unroll
                for (int c = 0; c < C; ++c) mine.s[c] = 0;
                mine.flag = 1;
                mine.starts += 1;
            }
            int v[C];
            cb_ctr_values<C>(a, p, v);
#pragma unroll
            for (int c = 0; c < C; ++c) {
                loc[k][c] = mine.s[c];
                mine.s[c] += v[c];
            }
        }
        loc_starts[k] = mine.starts;
        if (mine.flag) seen_mask |= 1u << k;
    }
    CbSeg total;
    const CbSeg before = cb_seg_block_exclusive<C>(mine, warp_tot, &total);
#pragma unroll
    for (int k = 0; k < CB_CTR_ITEMS; ++k) {
        const long long p = p0 + k;
        if (p < a.n) {
            const bool seen = (seen_mask >> k) & 1u;
#pragma unroll
            for (int c = 0; c < C; ++c) a.excl[(long long)c * a.n + p] = loc[k][c] + (seen ? 0 : before.s[c]);
            a.open[p] = (!seen && !before.flag) ? 1 : 0;
            a.seg_id[p] = before.starts + loc_starts[k];
        }
    }
    if (threadIdx.x == 0) a.tile_agg[blockIdx.x] = total;
}

// phase B: exclusive scan of the tile aggregates (one block; every thread owns a contiguous run of tiles)
template <int C>
__global__ void __launch_bounds__(1024) cb_ctr_scan_aggregates(CbSeg* agg, int tiles, int* n_segments) {
    __shared__ CbSeg warp_tot[32];
    const int per = (tiles + blockDim.x - 1) / blockDim.x;
    const int t0 = threadIdx.x * per, t1 = min(tiles, t0 + per);
    CbSeg mine;
#pragma unroll
    for (int c = 0; c < C; ++c) mine.s[c] = 0;
    mine.flag = 0;
    mine.starts = 0;
    for (int t = t0; t < t1; ++t) mine = cb_seg_combine<C>(mine, agg[t]);
    CbSeg total;
    CbSeg run = cb_seg_block_exclusive<C>(mine, warp_tot, &total);
    for (int t = t0; t < t1; ++t) {
        const CbSeg own = agg[t];
        agg[t] = run;
        run = cb_seg_combine<C>(run, own);
    }
    if (threadIdx.x == 0) *n_segments = total.starts;
}

// phase C: carry of the earlier tiles, dense segment numbers, distinct hashes, per-segment totals
template <int C>
__global__ void __launch_bounds__(CB_CTR_THREADS) cb_ctr_scan_finish(CbCtrScanArgs a) {
    const long long p = (long long)blockIdx.x * CB_CTR_THREADS + threadIdx.x;
    if (p >= a.n) return;
    const CbSeg carry = a.tile_agg[p / CB_CTR_TILE];
    const bool open = a.open[p] != 0;
    const int sid = carry.starts + a.seg_id[p] - 1;
    a.seg_id[p] = sid;
    const long long h = a.sorted_h[p];
    const bool start = p == 0 || a.sorted_h[p - 1] != h;
    const bool last = p + 1 == a.n || a.sorted_h[p + 1] != h;
    int v[C];
    if (last) cb_ctr_values<C>(a, p, v);
#pragma unroll
    for (int c = 0; c < C; ++c) {
        int e = a.excl[(long long)c * a.n + p];
        if (open) {
            e += carry.s[c];
            a.excl[(long long)c * a.n + p] = e;
        }
        if (last) a.totals[(long long)c * a.n + sid] = e + v[c];
    }
    if (start) a.uniq[sid] = h;
}

template <int C>
static cudaError_t cb_ctr_scan_launch(const CbCtrScanArgs& a, cudaStream_t st) {
    const int tiles = (int)((a.n + CB_CTR_TILE - 1) / CB_CTR_TILE);
    cb_ctr_scan_tiles<C><<<tiles, CB_CTR_THREADS, 0, st>>>(a);
    cb_ctr_scan_aggregates<C><<<1, 1024, 0, st>>>(a.tile_agg, tiles, a.n_segments);
    cb_ctr_scan_finish<C><<<(unsigned)((a.n + CB_CTR_THREADS - 1) / CB_CTR_THREADS), CB_CTR_THREADS, 0, st>>>(a);
    return cudaGetLastError();
}

CB_API int cb_ctr_tile() { return CB_CTR_TILE; }
CB_API int cb_ctr_agg_bytes() { return (int)sizeof(CbSeg); }
CB_API int cb_ctr_max_tb() { return CB_CTR_MAX_TB; }
CB_API int cb_ctr_max_specs() { return CB_CTR_MAX_SPECS; }

// Returns 0, or a CUDA error code, or -1 for a bad argument.  Work buffers: `open` [n] bytes, `tile_agg`
// [ceil(n / cb_ctr_tile())] * cb_ctr_agg_bytes() bytes.
CB_API int cb_ctr_scan(const long long* sorted_h, const long long* rows, const unsigned char* cls, long long n, int nb,
                       const int* tb, int* excl, int* seg_id, unsigned char* open, void* tile_agg, long long* uniq,
                       int* totals, int* n_segments, cudaStream_t st) {
    if (n <= 0 || nb < 0 || nb > CB_CTR_MAX_TB || n >= (1ll << 31)) return -1;
    CbCtrScanArgs a;
    a.sorted_h = sorted_h; a.rows = rows; a.cls = cls; a.n = n; a.nb = nb;
    for (int k = 0; k < CB_CTR_MAX_TB; ++k) a.tb[k] = k < nb ? tb[k] : 0;
    a.excl = excl; a.seg_id = seg_id; a.open = open; a.tile_agg = (CbSeg*)tile_agg; a.uniq = uniq; a.totals = totals;
    a.n_segments = n_segments;
    cudaError_t e;
    switch (nb) {
        case 0: e = cb_ctr_scan_launch<1>(a, st); break;
        case 1: e = cb_ctr_scan_launch<2>(a, st); break;
        case 2: e = cb_ctr_scan_launch<3>(a, st); break;
        case 3: e = cb_ctr_scan_launch<4>(a, st); break;
        default: e = cb_ctr_scan_launch<CB_CTR_C>(a, st); break;       // nb == CB_CTR_MAX_TB: the buffers have 1 + nb rows
    }
    return e == cudaSuccess ? 0 : (int)e;
}

// ---- values, their range, their buckets -----------------------------------------------------------------------------------
struct CbCtrSpecs {
    int count;
    int kind[CB_CTR_MAX_SPECS];          // 0: target statistic (ordered), 1: whole-data frequency (Counter / FeatureFreq)
    int column[CB_CTR_MAX_SPECS];        // kind 0: which scanned column holds the numerator counts (1 + index of the border)
    float prior_num[CB_CTR_MAX_SPECS];
    float prior_denom[CB_CTR_MAX_SPECS]; // kind 0: added to the running count; kind 1: unused
    float denom[CB_CTR_MAX_SPECS];       // kind 1: the whole denominator
    int border_off[CB_CTR_MAX_SPECS];
    int border_cnt[CB_CTR_MAX_SPECS];
};

__device__ __forceinline__ float cb_ctr_value(const CbCtrSpecs& sp, int s, const int* excl, const int* totals, const int* seg_id,
                                              long long n, long long p) {
    if (sp.kind[s] == 0) {
        const float num = __fadd_rn((float)excl[(long long)sp.column[s] * n + p], sp.prior_num[s]);
        const float den = __fadd_rn((float)excl[p], sp.prior_denom[s]);
        return __fdiv_rn(num, den);
    }
    const float num = __fadd_rn((float)totals[seg_id[p]], sp.prior_num[s]);
    return __fdiv_rn(num, sp.denom[s]);
}

// mm: [specs][2] uint32 bit patterns of (min, max); CTR values are never negative, so unsigned order is float order.
// The caller initialises min to 0xFFFFFFFF and max to 0.
__global__ void __launch_bounds__(256) cb_ctr_minmax_kernel(CbCtrSpecs sp, const int* excl, const int* totals, const int* seg_id,
                                                            long long n, unsigned* mm) {
    unsigned lo[CB_CTR_MAX_SPECS], hi[CB_CTR_MAX_SPECS];
    for (int s = 0; s < sp.count; ++s) { lo[s] = 0xFFFFFFFFu; hi[s] = 0u; }
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (long long)gridDim.x * blockDim.x)
        for (int s = 0; s < sp.count; ++s) {
            const unsigned b = __float_as_uint(cb_ctr_value(sp, s, excl, totals, seg_id, n, p));
            lo[s] = min(lo[s], b);
            hi[s] = max(hi[s], b);
        }
    for (int s = 0; s < sp.count; ++s) {
        unsigned l = lo[s], h = hi[s];
        for (int d = 16; d > 0; d >>= 1) {
            l = min(l, __shfl_xor_sync(0xffffffffu, l, d));
            h = max(h, __shfl_xor_sync(0xffffffffu, h, d));
        }
        if ((threadIdx.x & 31) == 0) {
            atomicMin(&mm[2 * s], l);
            atomicMax(&mm[2 * s + 1], h);
        }
    }
}

// out: [specs][n_out] bytes in document order; only documents row_lo <= row < row_lo + n_out are written
__global__ void __launch_bounds__(256) cb_ctr_binarize_kernel(CbCtrSpecs sp, const int* excl, const int* totals, const int* seg_id,
                                                              const long long* rows, long long n, const float* borders,
                                                              int n_borders, long long row_lo, long long n_out,
                                                              unsigned char* out) {
    extern __shared__ float s_borders[];
    for (int k = threadIdx.x; k < n_borders; k += blockDim.x) s_borders[k] = borders[k];
    __syncthreads();
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < n; p += (long long)gridDim.x * blockDim.x) {
        const long long row = rows[p] - row_lo;
        if (row < 0 || row >= n_out) continue;
        for (int s = 0; s < sp.count; ++s) {
            const float v = cb_ctr_value(sp, s, excl, totals, seg_id, n, p);
            const float* b = s_borders + sp.border_off[s];
            int lo = 0, hi = sp.border_cnt[s];                 // number of borders strictly below v
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (b[mid] < v) lo = mid + 1; else hi = mid;
            }
            out[(long long)s * n_out + row] = (unsigned char)lo;
        }
    }
}

static int cb_ctr_fill_specs(CbCtrSpecs* sp, int count, const int* kind, const int* column, const float* prior_num,
                             const float* prior_denom, const float* denom, const int* border_off, const int* border_cnt) {
    if (count < 0 || count > CB_CTR_MAX_SPECS) return -1;
    sp->count = count;
    for (int s = 0; s < count; ++s) {
        sp->kind[s] = kind[s]; sp->column[s] = column[s]; sp->prior_num[s] = prior_num[s];
        sp->prior_denom[s] = prior_denom[s]; sp->denom[s] = denom[s];
        sp->border_off[s] = border_off ? border_off[s] : 0;
        sp->border_cnt[s] = border_cnt ? border_cnt[s] : 0;
    }
    return 0;
}

CB_API int cb_ctr_minmax(int count, const int* kind, const int* column, const float* prior_num, const float* prior_denom,
                         const float* denom, const int* excl, const int* totals, const int* seg_id, long long n,
                         unsigned* mm, cudaStream_t st) {
    CbCtrSpecs sp;
    if (cb_ctr_fill_specs(&sp, count, kind, column, prior_num, prior_denom, denom, nullptr, nullptr)) return -1;
    if (n <= 0 || count == 0) return 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long grid = (n + 255) / 256;
    if (grid > sms * 8) grid = sms * 8;
    cb_ctr_minmax_kernel<<<(unsigned)grid, 256, 0, st>>>(sp, excl, totals, seg_id, n, mm);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

CB_API int cb_ctr_binarize(int count, const int* kind, const int* column, const float* prior_num, const float* prior_denom,
                           const float* denom, const int* border_off, const int* border_cnt, const float* borders,
                           int n_borders, const int* excl, const int* totals, const int* seg_id, const long long* rows,
                           long long n, long long row_lo, long long n_out, unsigned char* out, cudaStream_t st) {
    CbCtrSpecs sp;
    if (cb_ctr_fill_specs(&sp, count, kind, column, prior_num, prior_denom, denom, border_off, border_cnt)) return -1;
    if (n <= 0 || count == 0 || n_out <= 0) return 0;
    if (n_borders < 0 || n_borders > 8192) return -1;
    for (int s = 0; s < count; ++s)
        if (sp.border_cnt[s] > 255 || sp.border_off[s] < 0 || sp.border_off[s] + sp.border_cnt[s] > n_borders) return -1;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long grid = (n + 255) / 256;
    if (grid > sms * 8) grid = sms * 8;
    cb_ctr_binarize_kernel<<<(unsigned)grid, 256, (size_t)n_borders * sizeof(float), st>>>(sp, excl, totals, seg_id, rows, n,
                                                                                         borders, n_borders, row_lo, n_out, out);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
