// Stand-alone sm_100a kernels of catboost_b200 and their C launchers (called from Python through ctypes
// with raw device pointers and a CUDA stream handle).  Every launcher only enqueues work; none of them
// synchronises or allocates.
#include "cb_common.cuh"
#include "cb_losses.cuh"
#include "cb_tree.cuh"
#include "cb_comm.cuh"
#include <new>

#define CB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

// ======================================================================================================
// K1  quantize: float32 rows -> packed one-byte bins.  bin = #borders strictly below the value, i.e. the
// document goes right of border k iff bin > k  (catboost/cuda/gpu_data/kernel/binarize.cu:37,
// catboost/libs/data/quantization.cpp).  NaN goes to bin 0 (nan_mode Min) or to the last bin (Max).
// Thread = (document, feature group); blockIdx.x runs over groups fastest so that the blocks reading the
// same rows are co-scheduled and the row-major matrix is fetched from DRAM once.
__global__ void __launch_bounds__(256) cb_quantize_kernel(const float* __restrict__ X, long long n, int F, long long ldx,
                                                          const float* __restrict__ borders,
                                                          const int* __restrict__ border_off,
                                                          const unsigned char* __restrict__ nan_is_max,
                                                          uint32_t* __restrict__ bins, long long npad,
                                                          long long doc_offset, int G) {
    const int g = blockIdx.x % G;
    const long long tile = blockIdx.x / G;
    const long long i = tile * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float* row = X + i * ldx;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int f = g * 4 + j;
        if (f < F) {
            const float v = row[f];
            const int b0 = border_off[f], b1 = border_off[f + 1];
            int bin;
            if (v != v) {
                bin = (nan_is_max && nan_is_max[f]) ? (b1 - b0) : 0;
            } else {
                int lo = b0, hi = b1;          // first border >= v  ->  count of borders < v
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (__ldg(borders + mid) < v) lo = mid + 1; else hi = mid;
                }
                bin = lo - b0;
            }
            word |= (uint32_t)bin << (8 * j);
        }
    }
    bins[(long long)g * npad + doc_offset + i] = word;
}

CB_API int cb_quantize(const float* X, long long n, int F, long long ldx, const float* borders, const int* border_off,
                       const unsigned char* nan_is_max, uint32_t* bins, long long npad, long long doc_offset,
                       cudaStream_t st) {
    if (n <= 0) return 0;
    const int G = (F + 3) / 4;
    const long long tiles = (n + 255) / 256;
    cb_quantize_kernel<<<(unsigned)(tiles * G), 256, 0, st>>>(X, n, F, ldx, borders, border_off, nan_is_max, bins, npad,
                                                               doc_offset, G);
    CB_LAUNCH_CHECK();
    return 0;
}

// Pack already-binned uint8 columns (feature-major [F][n]) into the group store; used for CTR features and
// for host-quantized pools.
__global__ void cb_pack_bins_kernel(const unsigned char* __restrict__ cols, long long n, long long ld, int F,
                                    int f_dst_begin, uint32_t* __restrict__ bins, long long npad, long long doc_offset) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    for (int f = 0; f < F; ++f) {
        const int fd = f_dst_begin + f;
        uint32_t* w = bins + (long long)(fd >> 2) * npad + doc_offset + i;
        const int sh = (fd & 3) * 8;
        *w = (*w & ~(255u << sh)) | ((uint32_t)cols[(long long)f * ld + i] << sh);
    }
}

CB_API int cb_pack_bins(const unsigned char* cols, long long n, long long ld, int F, int f_dst_begin, uint32_t* bins,
                        long long npad, long long doc_offset, cudaStream_t st) {
    if (n <= 0 || F <= 0) return 0;
    cb_pack_bins_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(cols, n, ld, F, f_dst_begin, bins, npad, doc_offset);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K3 + K5 + K9  derivatives, fused with the cursor update by the previous tree and the bootstrap weights.
struct CbGradArgs {
    int loss; float p0, p1;
    float* approx; const float* target; const float* weight;
    unsigned short* leaf; const float* cur_vals;
    long long n, npad;
    float* stats; int newton_stats;
    int boot_type; float boot_p;        // 0 none, 1 Bayesian(temperature), 2 Bernoulli(subsample), 3 Poisson(lambda)
    unsigned long long seed; const int* iter_ptr;
    double* scal;
    const float* ext_der; const float* ext_hess;   // CB_LOSS_EXTERNAL
    float* statmax;          // [2] running max |stat| of this iteration (float bits are ordered for x >= 0)
};

__device__ __forceinline__ float cb_bootstrap_weight(int type, float p, unsigned long long h) {
    switch (type) {
        default: return 1.0f;
        case 1: {   // Bayesian: (-log u)^temperature   (catboost/cuda/cuda_util/kernel/bootstrap.cu:7-66)
            const float u = cb_uniform01(h);
            const float e = -__logf(u + 1e-20f);
            return (p == 1.0f) ? e : __powf(e, p);
        }
        case 2: return cb_uniform01(h) < p ? 1.0f : 0.0f;
        case 3: {   // Poisson(lambda = p) by inversion, lambda is O(1)
            float u = cb_uniform01(h);
            float pk = __expf(-p), cdf = pk;
            int k = 0;
            while (u > cdf && k < 32) { ++k; pk *= p / k; cdf += pk; }
            return (float)k;
        }
    }
}

// Four documents per thread and step with 16-byte loads / stores; the loads of the next step are issued before the
// current one is processed (all arrays are padded to npad, a multiple of 256, so vectors never run past the end).
struct CbGradIn { float4 ap, tg, w, ed, eh; ushort4 lf; };
template <int LOSS>
__device__ __forceinline__ void cb_grad_load(const CbGradArgs& a, long long i0, CbGradIn& v) {
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    v.ap = *reinterpret_cast<const float4*>(a.approx + i0);
    if (a.cur_vals) v.lf = *reinterpret_cast<const ushort4*>(a.leaf + i0);
    if (a.weight) v.w = *reinterpret_cast<const float4*>(a.weight + i0);
    if (loss == CB_LOSS_EXTERNAL) {
        v.ed = *reinterpret_cast<const float4*>(a.ext_der + i0);
        if (a.ext_hess) v.eh = *reinterpret_cast<const float4*>(a.ext_hess + i0);
    } else {
        v.tg = *reinterpret_cast<const float4*>(a.target + i0);
    }
}

// LOSS >= 0 fixes the objective at compile time (the common ones get their own instantiation, which removes the
// dispatch and the unused inputs from the loop); LOSS = -1 reads it from the arguments.
template <int LOSS>
__global__ void __launch_bounds__(256, 4) cb_grad_kernel(CbGradArgs a) {
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    const int it = *a.iter_ptr;
    double s_loss = 0.0, s_w = 0.0, s_d2 = 0.0, s_n = 0.0;
    float m0 = 0.0f, m1 = 0.0f;
    const long long n4 = a.npad >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    CbGradIn nx;
    nx.w = make_float4(1.f, 1.f, 1.f, 1.f);
    nx.eh = make_float4(1.f, 1.f, 1.f, 1.f);
    nx.ed = nx.tg = nx.ap = make_float4(0.f, 0.f, 0.f, 0.f);
    nx.lf = make_ushort4(0, 0, 0, 0);
    if (q < n4) cb_grad_load<LOSS>(a, q << 2, nx);
    for (; q < n4; q += stride) {
        const long long i0 = q << 2;
        const CbGradIn v = nx;
        if (q + stride < n4) cb_grad_load<LOSS>(a, (q + stride) << 2, nx);
        float ap[4] = {v.ap.x, v.ap.y, v.ap.z, v.ap.w};
        const float tg[4] = {v.tg.x, v.tg.y, v.tg.z, v.tg.w};
        const float wt[4] = {v.w.x, v.w.y, v.w.z, v.w.w};
        const float ed[4] = {v.ed.x, v.ed.y, v.ed.z, v.ed.w};
        const float eh[4] = {v.eh.x, v.eh.y, v.eh.z, v.eh.w};
        const unsigned int lf[4] = {v.lf.x, v.lf.y, v.lf.z, v.lf.w};
        float o0[4], o1[4];
        float f_loss = 0.f, f_w = 0.f, f_d2 = 0.f, f_n = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long i = i0 + k;
            const bool live = i < a.n;
            if (a.cur_vals) ap[k] += a.cur_vals[lf[k]];
            const float w = wt[k];
            CbLossOut o;
            if (loss == CB_LOSS_EXTERNAL) { o.der = ed[k]; o.hess = eh[k]; o.value = 0.0f; }
            else o = cb_loss_eval(loss, a.p0, a.p1, ap[k], tg[k]);
            const float wb = a.boot_type ? cb_bootstrap_weight(a.boot_type, a.boot_p,
                                                                 cb_mix64(a.seed ^ cb_mix64(((unsigned long long)it << 40) ^ (unsigned long long)i)))
                                         : 1.0f;
            const float wd = w * o.der;
            const float st0 = live ? wb * wd : 0.0f;
            const float st1 = live ? wb * w * (a.newton_stats ? o.hess : 1.0f) : 0.0f;
            o0[k] = st0; o1[k] = st1;
            m0 = fmaxf(m0, fabsf(st0));
            m1 = fmaxf(m1, fabsf(st1));
            if (live) { f_loss += w * o.value; f_w += w; f_d2 += wd * wd; f_n += 1.0f; }
        }
        if (a.cur_vals) *reinterpret_cast<float4*>(a.approx + i0) = make_float4(ap[0], ap[1], ap[2], ap[3]);
        *reinterpret_cast<ushort4*>(a.leaf + i0) = make_ushort4(0, 0, 0, 0);
        *reinterpret_cast<float4*>(a.stats + i0) = make_float4(o0[0], o0[1], o0[2], o0[3]);
        *reinterpret_cast<float4*>(a.stats + a.npad + i0) = make_float4(o1[0], o1[1], o1[2], o1[3]);
        s_loss += (double)f_loss; s_w += (double)f_w; s_d2 += (double)f_d2; s_n += (double)f_n;
    }
    __shared__ double red[4][8];
    s_loss = cb_warp_sum_d(s_loss); s_w = cb_warp_sum_d(s_w); s_d2 = cb_warp_sum_d(s_d2); s_n = cb_warp_sum_d(s_n);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s_loss; red[1][warp] = s_w; red[2][warp] = s_d2; red[3][warp] = s_n; }
    __syncthreads();
    if (threadIdx.x < 4) {
        double t = 0.0;
        for (int k = 0; k < (blockDim.x >> 5); ++k) t += red[threadIdx.x][k];
        atomicAdd(a.scal + threadIdx.x, t);
    }
    if (a.statmax) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
            m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
        }
        if (lane == 0) {
            atomicMax(reinterpret_cast<int*>(a.statmax), __float_as_int(m0));
            atomicMax(reinterpret_cast<int*>(a.statmax) + 1, __float_as_int(m1));
        }
    }
}

CB_API int cb_grad_pointwise(int loss, float p0, float p1, float* approx, const float* target, const float* weight,
                             unsigned short* leaf, const float* cur_vals, long long n, long long npad, float* stats,
                             int newton_stats, int boot_type, float boot_p, unsigned long long seed,
                             const int* iter_ptr, double* scal, const float* ext_der, const float* ext_hess,
                             float* statmax, int grid, cudaStream_t st) {
    CbGradArgs a{loss, p0, p1, approx, target, weight, leaf, cur_vals, n, npad, stats, newton_stats,
                 boot_type, boot_p, seed, iter_ptr, scal, ext_der, ext_hess, statmax};
    if (loss == CB_LOSS_LOGLOSS) cb_grad_kernel<CB_LOSS_LOGLOSS><<<grid, 256, 0, st>>>(a);
    else if (loss == CB_LOSS_RMSE) cb_grad_kernel<CB_LOSS_RMSE><<<grid, 256, 0, st>>>(a);
    else cb_grad_kernel<-1><<<grid, 256, 0, st>>>(a);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// Host-side handles
CB_API CbData* cb_data_create(const uint32_t* bins, long long npad, long long n, int F, const int* feat_off,
                              const int* feat_nb, const unsigned char* feat_onehot, const float* feat_weight, int TB) {
    CbData* d = new (std::nothrow) CbData();
    if (!d) return nullptr;
    d->bins = bins; d->npad = npad; d->n = n; d->G = (F + 3) / 4; d->F = F;
    d->feat_off = feat_off; d->feat_nb = feat_nb; d->feat_onehot = feat_onehot; d->feat_weight = feat_weight; d->TB = TB;
    return d;
}
CB_API void cb_data_destroy(CbData* d) { delete d; }

CB_API CbComm* cb_comm_create(int rank, int nranks, long long timeout_ns, int* status, unsigned long long* epoch,
                              char* const* mbox, unsigned long long* const* mbox_flag, int mbox_bytes,
                              float* const* slot, unsigned long long* const* slot_flag, long long slot_floats) {
    if (nranks < 1 || nranks > CB_MAX_RANKS) return nullptr;
    CbComm* c = new (std::nothrow) CbComm();
    if (!c) return nullptr;
    c->rank = rank; c->nranks = nranks; c->timeout_ns = timeout_ns; c->status = status; c->epoch = epoch;
    c->mbox_bytes = mbox_bytes; c->slot_floats = slot_floats;
    for (int r = 0; r < CB_MAX_RANKS; ++r) {
        c->peer_mbox[r] = r < nranks ? mbox[r] : nullptr;
        c->peer_mbox_flag[r] = r < nranks ? mbox_flag[r] : nullptr;
        c->peer_slot[r] = r < nranks ? slot[r] : nullptr;
        c->peer_slot_flag[r] = r < nranks ? slot_flag[r] : nullptr;
    }
    return c;
}
CB_API void cb_comm_destroy(CbComm* c) { delete c; }

// ======================================================================================================
// K7 (leaf part)  stand-alone leaf update for the split of (current tree, level)
__global__ void __launch_bounds__(256) cb_update_leaf_kernel(CbData d, unsigned short* leaf, const CbSplit* splits,
                                                             const int* iter_ptr, int depth, int level) {
    const CbSplit sp = splits[(long long)(*iter_ptr) * depth + level];
    cb_update_leaf_range(d, leaf, sp, level, (long long)blockIdx.x * blockDim.x + threadIdx.x,
                         (long long)gridDim.x * blockDim.x);
}

CB_API int cb_update_leaf(const CbData* d, unsigned short* leaf, const CbSplit* splits, const int* iter_ptr, int depth,
                          int level, int grid, cudaStream_t st) {
    cb_update_leaf_kernel<<<grid, 256, 0, st>>>(*d, leaf, splits, iter_ptr, depth, level);
    CB_LAUNCH_CHECK();
    return 0;
}

// Non-symmetric trees: leaf holds a node id; nodes with a split send their documents to a child.
// node_split[node] = {feature, bin, flags, left_child}; right child = left_child + 1; feature < 0 = leaf.
__global__ void __launch_bounds__(256) cb_update_nodes_kernel(CbData d, unsigned short* leaf, const int4* node_split,
                                                              int n_nodes) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride) {
        const int node = leaf[i];
        if (node >= n_nodes) continue;
        const int4 sp = node_split[node];
        if (sp.x < 0) continue;
        const uint32_t w = d.bins[(long long)(sp.x >> 2) * d.npad + i];
        const unsigned int b = (w >> ((sp.x & 3) * 8)) & 255u;
        const bool right = (sp.z & 1) ? (b == (unsigned)sp.y) : (b > (unsigned)sp.y);
        leaf[i] = (unsigned short)(sp.w + (right ? 1 : 0));
    }
}

CB_API int cb_update_nodes(const CbData* d, unsigned short* leaf, const int* node_split, int n_nodes, int grid,
                           cudaStream_t st) {
    cb_update_nodes_kernel<<<grid, 256, 0, st>>>(*d, leaf, reinterpret_cast<const int4*>(node_split), n_nodes);
    CB_LAUNCH_CHECK();
    return 0;
}

// One node splits (leaf-wise growth): its documents move to left_child (+1 when the condition holds).  The split comes
// as kernel arguments, so the growth loop uploads nothing per split.
__global__ void __launch_bounds__(256) cb_update_one_node_kernel(CbData d, unsigned short* leaf, int node, int feature, int bin,
                                                                 int onehot, int left_child) {
    const uint32_t* col = d.bins + (long long)(feature >> 2) * d.npad;
    const int sh = (feature & 3) * 8;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride) {
        if (leaf[i] != (unsigned short)node) continue;
        const unsigned int b = (col[i] >> sh) & 255u;
        const bool right = onehot ? (b == (unsigned)bin) : (b > (unsigned)bin);
        leaf[i] = (unsigned short)(left_child + (right ? 1 : 0));
    }
}

CB_API int cb_update_one_node(const CbData* d, unsigned short* leaf, int node, int feature, int bin, int onehot, int left_child,
                              int grid, cudaStream_t st) {
    if (feature < 0 || feature >= d->F) return (int)cudaErrorInvalidValue;
    cb_update_one_node_kernel<<<grid, 256, 0, st>>>(*d, leaf, node, feature, bin, onehot, left_child);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K6a  stand-alone histogram kernel (non-fused path, NCCL baseline, CPU-oracle tests)
__global__ void __launch_bounds__(512) cb_hist_kernel(CbHistArgs a) {
    extern __shared__ __align__(16) float cb_sh[];
    cb_hist_phase(a, cb_sh, blockIdx.x, gridDim.x);
}

static int g_hist_smem_set = 0;

CB_API int cb_hist_smem_bytes(int slots_per_pass, int S, int B) { return slots_per_pass * S * 4 * B * 4; }

static int cb_hist_launch(const CbData* d, const unsigned short* leaf, const float* stats, int S, int level,
                          const unsigned int* small_mask, const short* slot_table, int nslots_table, int slots_per_pass,
                          int B, float* out, const float* statmax, int grid, int threads, cudaStream_t st);

CB_API int cb_hist(const CbData* d, const unsigned short* leaf, const float* stats, int S, int level,
                   const unsigned int* small_mask, const short* slot_table, int nslots_table, int slots_per_pass, int B,
                   float* out, int grid, int threads, cudaStream_t st) {
    return cb_hist_launch(d, leaf, stats, S, level, small_mask, slot_table, nslots_table, slots_per_pass, B, out, nullptr,
                          grid, threads, st);
}

// Same histogram with integer cells: statmax[s] = max |stats[s][i]| (device array of S floats).
CB_API int cb_hist_n(const CbData* d, const unsigned short* leaf, const float* stats, int S, int level,
                     const unsigned int* small_mask, const short* slot_table, int nslots_table, int slots_per_pass, int B,
                     float* out, const float* statmax, int grid, int threads, cudaStream_t st) {
    return cb_hist_launch(d, leaf, stats, S, level, small_mask, slot_table, nslots_table, slots_per_pass, B, out, statmax,
                          grid, threads, st);
}

static int cb_hist_launch(const CbData* d, const unsigned short* leaf, const float* stats, int S, int level,
                          const unsigned int* small_mask, const short* slot_table, int nslots_table, int slots_per_pass,
                          int B, float* out, const float* statmax, int grid, int threads, cudaStream_t st) {
    CbHistArgs a = CbHistArgs();
    a.d = *d; a.leaf = leaf; a.stats = stats; a.S = S; a.level = level; a.small_mask = small_mask;
    a.slots_per_pass = slots_per_pass; a.B = B; a.out = out; a.slot_table = slot_table; a.nslots_table = nslots_table;
    a.priv = nullptr; a.statmax = statmax; a.nK = 0; a.copies = 1; a.work = nullptr; a.narrow = 0; a.bundle = 0;
    const int smem = cb_hist_smem_bytes(slots_per_pass, S, B);
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set) || !g_hist_smem_set) {
        int dev = 0, optin = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, cb_hist_kernel);
        if (e == cudaSuccess) {
            g_hist_smem_set = optin - (int)fa.sharedSizeBytes;
            e = cudaFuncSetAttribute(cb_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g_hist_smem_set);
        }
        if (e != cudaSuccess) { g_hist_smem_set = 0; set = 0ull; cudaGetLastError(); return (int)e; }
    }
    if (smem > g_hist_smem_set) return (int)cudaErrorInvalidValue;
    cb_hist_kernel<<<grid, threads, smem, st>>>(a);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K6b  stand-alone scoring + selection kernels
static void cb_fill_score_args(CbScoreArgs& a, const CbData* d, const float* const* hsrc, int nsrc, const float* hprev,
                               float* hcur, int W, int col_base, int f_begin, int f_end, int level, int S,
                               const unsigned int* small_mask, float l2, int score_fn, float random_strength,
                               const double* scal, const int* iter_ptr, unsigned long long seed, float lr,
                               unsigned long long* best_key) {
    a.d = *d;
    for (int r = 0; r < CB_MAX_RANKS; ++r) a.hsrc[r] = r < nsrc ? hsrc[r] : nullptr;
    a.nsrc = nsrc; a.hprev = hprev; a.hcur = hcur; a.W = W; a.col_base = col_base; a.f_begin = f_begin; a.f_end = f_end;
    a.level = level; a.S = S; a.small_mask = small_mask; a.l2 = l2; a.score_fn = score_fn;
    a.random_strength = random_strength; a.scal = scal; a.iter_ptr = iter_ptr; a.seed = seed; a.learning_rate = lr;
    a.best_key = best_key;
}

__global__ void __launch_bounds__(256) cb_score_kernel(CbScoreArgs a) {
    extern __shared__ float score_sh[];            // CB_SCORE_WARP_FLOATS per warp
    cb_score_phase(a, blockIdx.x, gridDim.x, score_sh, (int)(blockDim.x >> 5) * CB_SCORE_WARP_FLOATS);
}

CB_API int cb_score(const CbData* d, const float* const* hsrc, int nsrc, const float* hprev, float* hcur, int W,
                    int col_base, int f_begin, int f_end, int level, int S, const unsigned int* small_mask, float l2,
                    int score_fn, float random_strength, const double* scal, const int* iter_ptr,
                    unsigned long long seed, float lr, unsigned long long* best_key, cudaStream_t st) {
    CbScoreArgs a = CbScoreArgs();
    cb_fill_score_args(a, d, hsrc, nsrc, hprev, hcur, W, col_base, f_begin, f_end, level, S, small_mask, l2, score_fn,
                       random_strength, scal, iter_ptr, seed, lr, best_key);
    const int nf = f_end - f_begin;
    if (nf <= 0) return 0;
    const int grid = (nf + 7) / 8;
    cb_score_kernel<<<grid, 256, 8 * CB_SCORE_WARP_FLOATS * sizeof(float), st>>>(a);
    CB_LAUNCH_CHECK();
    return 0;
}

__global__ void __launch_bounds__(256) cb_select_local_kernel(CbScoreArgs a, unsigned long long* msg) {
    cb_select_local(a, msg);
}

CB_API int cb_select_local_launch(const CbData* d, float* hcur, int W, int col_base, int level, int S,
                                  unsigned long long* best_key, unsigned long long* msg, cudaStream_t st) {
    CbScoreArgs a = CbScoreArgs();
    const float* none[1] = {nullptr};
    cb_fill_score_args(a, d, none, 0, nullptr, hcur, W, col_base, 0, 0, level, S, nullptr, 0.f, 0, 0.f, nullptr, nullptr,
                       0ull, 0.f, best_key);
    cb_select_local_kernel<<<1, 256, 0, st>>>(a, msg);
    CB_LAUNCH_CHECK();
    return 0;
}

struct CbMsgPtrs { const unsigned long long* p[CB_MAX_RANKS]; };

__global__ void __launch_bounds__(256) cb_select_final_kernel(CbData d, CbMsgPtrs m, int nmsg, int level, CbSplit* splits,
                                                              const int* iter_ptr, int depth, unsigned int* mask_out,
                                                              unsigned long long* best_key) {
    cb_select_final(d, m.p, nmsg, level, splits + (long long)(*iter_ptr) * depth + level, mask_out);
    if (threadIdx.x == 0) *best_key = 0ull;
}

CB_API int cb_select_final_launch(const CbData* d, const unsigned long long* msgs, int nmsg, long long msg_stride_bytes,
                                  int level, CbSplit* splits, const int* iter_ptr, int depth, unsigned int* mask_out,
                                  unsigned long long* best_key, cudaStream_t st) {
    CbMsgPtrs m;
    for (int r = 0; r < CB_MAX_RANKS; ++r)
        m.p[r] = r < nmsg ? reinterpret_cast<const unsigned long long*>(reinterpret_cast<const char*>(msgs) + r * msg_stride_bytes)
                          : nullptr;
    cb_select_final_kernel<<<1, 256, 0, st>>>(*d, m, nmsg, level, splits, iter_ptr, depth, mask_out, best_key);
    CB_LAUNCH_CHECK();
    return 0;
}

CB_API int cb_select_msg_bytes() { return CB_SELECT_MSG_BYTES; }

// ======================================================================================================
// Small all-reduce through the peer-mapped mailboxes (device functions in cb_comm.cuh).
__global__ void __launch_bounds__(256) cb_allreduce_sum_kernel(CbComm c, double* vals, int count) {
    cb_mailbox_allreduce_sum(c, vals, count);
}

CB_API int cb_allreduce_sum(const CbComm* c, double* vals, int count, cudaStream_t st) {
    if (count * 8 > c->mbox_bytes) return (int)cudaErrorInvalidValue;
    cb_allreduce_sum_kernel<<<1, 256, 0, st>>>(*c, vals, count);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K8  leaf estimation pass: per-leaf sums of (w*der, w*hess, w) at approx + delta[leaf], then the
// Newton / gradient step by the last block to finish (and across ranks through the mailbox).
// catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:127-206, pointwise_oracle.cpp:86-116.
struct CbLeafArgs {
    int loss; float p0, p1;
    const float* approx; const float* target; const float* weight; const unsigned short* leaf;
    const float* ext_der; const float* ext_hess;
    long long n; int L;
    float* delta;            // [L] running leaf values of this tree (unscaled)
    double* sums;            // [L][3], zero on entry, zeroed again on exit
    unsigned int* counter;   // zero on entry/exit
    int first, last, newton;
    float l2, lr;
    float* cur_vals;         // [L] lr * delta after the last pass (applied by the next derivative kernel)
    float* model_vals; float* model_wts; int Lstride; const int* iter_ptr;
    float* leaf_w;           // [L] per-leaf weight sums, written by the first pass of a tree
    CbComm c;
    // Fixed-point passes (optional): the first pass of a tree records vmax = {max |w der|, max |w hess|}; the later
    // passes scale to 24 bits against twice that bound and add a signed high and an unsigned low part with native
    // integer shared-memory atomics (fp32 shared atomics are compare-and-swap loops).  A value beyond the bound -- the
    // derivative moved further than expected between Newton steps -- goes to the double accumulator directly.
    float* vmax;
};

struct CbLeafIn { float4 a4, t4, w4, d4, h4; ushort4 lf4; };
template <int LOSS>
__device__ __forceinline__ void cb_leaf_load(const CbLeafArgs& a, long long i0, CbLeafIn& v) {
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    v.lf4 = *reinterpret_cast<const ushort4*>(a.leaf + i0);
    if (loss == CB_LOSS_EXTERNAL) {
        v.d4 = *reinterpret_cast<const float4*>(a.ext_der + i0);
        if (a.ext_hess) v.h4 = *reinterpret_cast<const float4*>(a.ext_hess + i0);
    } else {
        v.a4 = *reinterpret_cast<const float4*>(a.approx + i0);
        v.t4 = *reinterpret_cast<const float4*>(a.target + i0);
    }
    if (a.weight) v.w4 = *reinterpret_cast<const float4*>(a.weight + i0);
}

// Shared-memory accumulators are replicated per lane group: cell (leaf, stat) has `C` copies and lane `l` uses copy
// l & (C-1), so the lanes of a warp never collide on an address (shared fp32 atomics are compare-and-swap loops;
// without collisions every one succeeds on its first try).  C = 32 for up to 128 leaves.
// LOSS as in cb_grad_kernel.
template <int LOSS>
__device__ __forceinline__ void cb_leaf_pass_body(const CbLeafArgs& a, int C) {
    extern __shared__ float sl[];     // [L][3][C] floats (or [L][4][C] ints in a fixed-point pass), else unused
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    const int L = a.L;
    const bool use_sh = C > 0;
    const int cm = C - 1;
    const int lane_copy = threadIdx.x & cm;
    const bool quant = use_sh && a.vmax && !a.first && (a.n / gridDim.x) < (1ll << 19);
    int* si = reinterpret_cast<int*>(sl);
    float M0 = 0.f, M1 = 0.f, sc0 = 0.f, sc1 = 0.f;
    if (quant) {
        M0 = 2.0f * fmaxf(__ldcg(a.vmax), 1e-30f);
        M1 = 2.0f * fmaxf(__ldcg(a.vmax + 1), 1e-30f);
        sc0 = 8388607.0f / M0;
        sc1 = 8388607.0f / M1;
    }
    float mx0 = 0.f, mx1 = 0.f;
    if (use_sh) {
        for (int i = threadIdx.x; i < (quant ? 4 : 3) * L * C; i += blockDim.x) sl[i] = 0.0f;
        __syncthreads();
    }
    const long long n4 = (a.n + 3) >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // the loads of the next step are issued before the current step is processed
    long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    CbLeafIn nx;
    nx.a4 = nx.t4 = nx.d4 = make_float4(0.f, 0.f, 0.f, 0.f);
    nx.w4 = nx.h4 = make_float4(1.f, 1.f, 1.f, 1.f);
    nx.lf4 = make_ushort4(0, 0, 0, 0);
    if (q < n4) cb_leaf_load<LOSS>(a, q << 2, nx);
    for (; q < n4; q += stride) {
        const long long i0 = q << 2;
        const CbLeafIn v = nx;
        if (q + stride < n4) cb_leaf_load<LOSS>(a, (q + stride) << 2, nx);
        const unsigned int lf[4] = {v.lf4.x, v.lf4.y, v.lf4.z, v.lf4.w};
        const float ap[4] = {v.a4.x, v.a4.y, v.a4.z, v.a4.w}, tg[4] = {v.t4.x, v.t4.y, v.t4.z, v.t4.w};
        const float wt[4] = {v.w4.x, v.w4.y, v.w4.z, v.w4.w};
        const float ed[4] = {v.d4.x, v.d4.y, v.d4.z, v.d4.w}, eh[4] = {v.h4.x, v.h4.y, v.h4.z, v.h4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + k >= a.n) break;
            const int l = (int)lf[k];
            CbLossOut o;
            if (loss == CB_LOSS_EXTERNAL) { o.der = ed[k]; o.hess = eh[k]; }
            else o = cb_loss_eval(loss, a.p0, a.p1, ap[k] + (a.first ? 0.0f : a.delta[l]), tg[k]);
            const float w = wt[k];
            if (quant) {
                const float vd = w * o.der, vh = w * o.hess;
                if (fabsf(vd) <= M0 && fabsf(vh) <= M1) {
                    const int qd = __float2int_rn(vd * sc0), qh = __float2int_rn(vh * sc1);
                    int* cell = si + (size_t)(l * 4) * C + lane_copy;
                    atomicAdd(cell, qd >> 12);
                    atomicAdd(reinterpret_cast<unsigned int*>(cell + C), (unsigned int)qd & 4095u);
                    atomicAdd(cell + 2 * C, qh >> 12);
                    atomicAdd(reinterpret_cast<unsigned int*>(cell + 3 * C), (unsigned int)qh & 4095u);
                } else {
                    atomicAdd(&a.sums[3 * l], (double)vd);
                    atomicAdd(&a.sums[3 * l + 1], (double)vh);
                }
                continue;
            }
            if (a.vmax && a.first) { mx0 = fmaxf(mx0, fabsf(w * o.der)); mx1 = fmaxf(mx1, fabsf(w * o.hess)); }
            if (use_sh) {
                float* cell = sl + (size_t)(l * 3) * C + lane_copy;
                atomicAdd(cell, w * o.der);
                atomicAdd(cell + C, w * o.hess);
                if (a.first) atomicAdd(cell + 2 * C, w);
            } else {
                atomicAdd(&a.sums[3 * l], (double)(w * o.der));
                atomicAdd(&a.sums[3 * l + 1], (double)(w * o.hess));
                if (a.first) atomicAdd(&a.sums[3 * l + 2], (double)w);
            }
        }
    }
    if (a.vmax && a.first) {
        for (int off = 16; off > 0; off >>= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        if ((threadIdx.x & 31) == 0) {           // non-negative floats order like their bit patterns
            atomicMax(reinterpret_cast<int*>(a.vmax), __float_as_int(mx0));
            atomicMax(reinterpret_cast<int*>(a.vmax) + 1, __float_as_int(mx1));
        }
    }
    if (quant) {
        __syncthreads();
        const double inv0 = (double)M0 / 8388607.0, inv1 = (double)M1 / 8388607.0;
        for (int i = threadIdx.x; i < 2 * L; i += blockDim.x) {
            const int l = i >> 1, s2 = i & 1;
            const int* ph = si + (size_t)(l * 4 + 2 * s2) * C;
            long long hi = 0, lo = 0;
            for (int c = 0; c < C; ++c) { hi += ph[c]; lo += (unsigned int)ph[C + c]; }
            const long long q = hi * 4096 + lo;
            if (q != 0) atomicAdd(&a.sums[3 * l + s2], (double)q * (s2 ? inv1 : inv0));
        }
    } else if (use_sh) {
        __syncthreads();
        for (int i = threadIdx.x; i < 3 * L; i += blockDim.x) {
            float v = 0.0f;
            for (int c = 0; c < C; ++c) v += sl[(size_t)i * C + c];
            if (v != 0.0f) atomicAdd(&a.sums[i], (double)v);
        }
    }
    __shared__ bool s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (a.c.nranks > 1) {
        for (int base = 0; base < 3 * L; base += a.c.mbox_bytes / 8) {
            cb_mailbox_allreduce_sum(a.c, a.sums + base, min(3 * L - base, a.c.mbox_bytes / 8));
        }
    }
    const int it = *a.iter_ptr;
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const double sd = __ldcg(&a.sums[3 * l]), shs = __ldcg(&a.sums[3 * l + 1]);
        if (a.first) a.leaf_w[l] = (float)__ldcg(&a.sums[3 * l + 2]);
        const double sw = (double)a.leaf_w[l];
        const double den = (a.newton ? shs : sw) + (double)a.l2;
        const float step = (den > 0.0) ? (float)(sd / den) : 0.0f;
        const float v = (a.first ? 0.0f : a.delta[l]) + step;
        a.delta[l] = v;
        if (a.last) {
            a.cur_vals[l] = a.lr * v;
            if (a.model_vals) a.model_vals[(long long)it * a.Lstride + l] = a.lr * v;
            if (a.model_wts) a.model_wts[(long long)it * a.Lstride + l] = (float)sw;
        }
        a.sums[3 * l] = 0.0; a.sums[3 * l + 1] = 0.0; a.sums[3 * l + 2] = 0.0;
    }
    if (threadIdx.x == 0) {
        *a.counter = 0u;
        if (a.vmax && a.last) { a.vmax[0] = 0.0f; a.vmax[1] = 0.0f; }
    }
}

__global__ void __launch_bounds__(512) cb_leaf_pass_kernel(CbLeafArgs a, int C) { cb_leaf_pass_body<-1>(a, C); }
template <int LOSS>
__global__ void __launch_bounds__(512) cb_leaf_pass_kernel_t(CbLeafArgs a, int C) { cb_leaf_pass_body<LOSS>(a, C); }

static int cb_leaf_pass_launch(CbLeafArgs& a, const CbComm* comm, int grid, cudaStream_t st) {
    if (comm) a.c = *comm; else { a.c.nranks = 1; a.c.rank = 0; }
    const int planes = a.vmax ? 4 : 3;
    int C = 32;
    while (C > 0 && (size_t)planes * a.L * C * 4 > 96 * 1024) C >>= 1;
    const int smem = planes * a.L * C * 4;
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_leaf_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_leaf_pass_kernel_t<CB_LOSS_LOGLOSS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_leaf_pass_kernel_t<CB_LOSS_RMSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    if (a.loss == CB_LOSS_LOGLOSS) cb_leaf_pass_kernel_t<CB_LOSS_LOGLOSS><<<grid, 512, smem, st>>>(a, C);
    else if (a.loss == CB_LOSS_RMSE) cb_leaf_pass_kernel_t<CB_LOSS_RMSE><<<grid, 512, smem, st>>>(a, C);
    else cb_leaf_pass_kernel<<<grid, 512, smem, st>>>(a, C);
    CB_LAUNCH_CHECK();
    return 0;
}

// Same as cb_leaf_pass with the fixed-point passes switched on: vmax is a device buffer of two floats, zero before the
// first pass of the first tree; the kernel clears it again at the end of the last pass of every tree.
CB_API int cb_leaf_pass_q(int loss, float p0, float p1, const float* approx, const float* target, const float* weight,
                          const unsigned short* leaf, const float* ext_der, const float* ext_hess, long long n, int L,
                          float* delta, double* sums, unsigned int* counter, int first, int last, int newton, float l2,
                          float lr, float* cur_vals, float* model_vals, float* model_wts, int Lstride,
                          const int* iter_ptr, float* leaf_w, const CbComm* comm, float* vmax, int grid,
                          cudaStream_t st) {
    CbLeafArgs a{loss, p0, p1, approx, target, weight, leaf, ext_der, ext_hess, n, L, delta, sums, counter,
                 first, last, newton, l2, lr, cur_vals, model_vals, model_wts, Lstride, iter_ptr, leaf_w, CbComm(), vmax};
    return cb_leaf_pass_launch(a, comm, grid, st);
}

CB_API int cb_leaf_pass(int loss, float p0, float p1, const float* approx, const float* target, const float* weight,
                        const unsigned short* leaf, const float* ext_der, const float* ext_hess, long long n, int L,
                        float* delta, double* sums, unsigned int* counter, int first, int last, int newton, float l2,
                        float lr, float* cur_vals, float* model_vals, float* model_wts, int Lstride,
                        const int* iter_ptr, float* leaf_w, const CbComm* comm, int grid, cudaStream_t st) {
    CbLeafArgs a{loss, p0, p1, approx, target, weight, leaf, ext_der, ext_hess, n, L, delta, sums, counter,
                 first, last, newton, l2, lr, cur_vals, model_vals, model_wts, Lstride, iter_ptr, leaf_w, CbComm(),
                 nullptr};
    if (comm) a.c = *comm; else { a.c.nranks = 1; a.c.rank = 0; }
    int C = 32;
    while (C > 0 && (size_t)3 * L * C * 4 > 96 * 1024) C >>= 1;
    const int smem = 3 * L * C * 4;
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_leaf_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    cb_leaf_pass_kernel<<<grid, 512, smem, st>>>(a, C);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// End of a boosting iteration: record the learn loss and the per-iteration extras (evaluation-set metric
// sums), clear the accumulators, advance the counter.
__global__ void cb_iter_end_kernel(int* iter_ptr, double* scal, double* loss_hist, double* extra_src, double* extra_dst,
                                   int n_extra, float* statmax, int n_statmax) {
    const int it = *iter_ptr;
    if (statmax) for (int k = 0; k < n_statmax; ++k) statmax[k] = 0.0f;
    if (loss_hist) { loss_hist[2 * it] = scal[0]; loss_hist[2 * it + 1] = scal[1]; }
    scal[0] = scal[1] = scal[2] = scal[3] = 0.0;
    for (int k = 0; k < n_extra; ++k) { extra_dst[(long long)it * n_extra + k] = extra_src[k]; extra_src[k] = 0.0; }
    *iter_ptr = it + 1;
}
CB_API int cb_iter_end(int* iter_ptr, double* scal, double* loss_hist, double* extra_src, double* extra_dst, int n_extra,
                       float* statmax, int n_statmax, cudaStream_t st) {
    cb_iter_end_kernel<<<1, 1, 0, st>>>(iter_ptr, scal, loss_hist, extra_src, extra_dst, n_extra, statmax, n_statmax);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K9  apply one oblivious tree to a binned set (evaluation sets during training):
// leaf = sum_d bit_d << d, approx[dim][i] += vals[leaf*dims + dim]   (models/kernel/add_model_value.cu:70)
__global__ void __launch_bounds__(256) cb_apply_tree_bins_kernel(CbData d, float* approx, long long approx_stride,
                                                                 const CbSplit* splits, const int* iter_ptr, int depth,
                                                                 const float* vals, int dims) {
    __shared__ CbSplit sp[16];
    const CbSplit* base = splits + (iter_ptr ? (long long)(*iter_ptr) * depth : 0);
    if (threadIdx.x < depth) sp[threadIdx.x] = base[threadIdx.x];
    __syncthreads();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride) {
        int leaf = 0;
        for (int k = 0; k < depth; ++k) {
            const CbSplit s = sp[k];
            if (s.feature < 0) continue;
            const uint32_t w = d.bins[(long long)(s.feature >> 2) * d.npad + i];
            const unsigned int b = (w >> ((s.feature & 3) * 8)) & 255u;
            const unsigned int bit = (s.flags & 1) ? (b == (unsigned)s.bin) : (b > (unsigned)s.bin);
            leaf |= bit << k;
        }
        for (int k = 0; k < dims; ++k) approx[k * approx_stride + i] += vals[leaf * dims + k];
    }
}

CB_API int cb_apply_tree_bins(const CbData* d, float* approx, long long approx_stride, const CbSplit* splits,
                              const int* iter_ptr, int depth, const float* vals, int dims, int grid, cudaStream_t st) {
    if (depth > 16) return (int)cudaErrorInvalidValue;
    cb_apply_tree_bins_kernel<<<grid, 256, 0, st>>>(*d, approx, approx_stride, splits, iter_ptr, depth, vals, dims);
    CB_LAUNCH_CHECK();
    return 0;
}

// leaf index only (used by the multi-dimensional and ranking trainers that update cursors themselves)
__global__ void __launch_bounds__(256) cb_leaf_index_kernel(CbData d, unsigned short* leaf, const CbSplit* splits, int depth) {
    __shared__ CbSplit sp[16];
    if (threadIdx.x < depth) sp[threadIdx.x] = splits[threadIdx.x];
    __syncthreads();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.n; i += stride) {
        int leaf_i = 0;
        for (int k = 0; k < depth; ++k) {
            const CbSplit s = sp[k];
            if (s.feature < 0) continue;
            const uint32_t w = d.bins[(long long)(s.feature >> 2) * d.npad + i];
            const unsigned int b = (w >> ((s.feature & 3) * 8)) & 255u;
            leaf_i |= ((s.flags & 1) ? (b == (unsigned)s.bin) : (b > (unsigned)s.bin)) << k;
        }
        leaf[i] = (unsigned short)leaf_i;
    }
}
CB_API int cb_leaf_index(const CbData* d, unsigned short* leaf, const CbSplit* splits, int depth, int grid, cudaStream_t st) {
    if (depth > 16) return (int)cudaErrorInvalidValue;
    cb_leaf_index_kernel<<<grid, 256, 0, st>>>(*d, leaf, splits, depth);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K14  batch apply of an oblivious-tree ensemble to raw float rows (inference).  Quantisation is fused:
// a block stages the bins of 256 rows for the features the model uses (shared memory, one byte each),
// then walks all trees; leaf values are read through the read-only path.  libs/model/cuda/evaluator.cu:85-343.
struct CbPredictArgs {
    const float* X; long long n; long long ldx;
    const int* used_feat;        // [U] column of X for used feature u
    const float* borders;        // concatenated borders of the used features
    const int* border_off;       // [U+1]
    const unsigned char* nan_is_max;   // [U] or null
    int U;
    const int* tree_depth;       // [T]
    const int* tree_split_off;   // [T] first split of tree t in split_feat/split_bin
    const unsigned short* split_feat;   // used-feature index
    const unsigned char* split_bin;     // go right when bin > split_bin
    const long long* tree_leaf_off;     // [T] first leaf value (in units of dims)
    const float* leaf_vals;      // [sum leaves][dims]
    int T; int dims;
    float scale; const float* bias;   // [dims]
    float* out;                  // [dims][n]
    int max_borders;             // largest border count of a used feature
    int lv_floats;               // shared-memory buffer for the leaf values of a chunk of trees, in floats (0 = none)
};

// Four rows per thread: the split descriptors of a chunk of trees are staged in shared memory as one word
// (feature << 8 | bin) per split, so a tree level costs one broadcast read + per row one byte read, a compare and an or.
// The leaf values of the chunk are staged next to them: a row reads one leaf value per tree at a random place, which
// from global memory is one 32-byte sector per value; from shared memory it is a bank access.  NT threads per block
// (1024 when the bins of 4096 rows fit beside the leaf buffer, so that the staging is paid once per 4096 rows).
#define CB_PRED_CHUNK_SPLITS 3072
template <int CB_PRED_ROWS, int NT>
__global__ void __launch_bounds__(NT) cb_predict_kernel(CbPredictArgs a) {
    // shared memory: bins [U][USTR] (USTR = NT * rows per thread + 4: the pad keeps the byte writes of 32 features of
    // one row in 32 different banks), split descriptors [CB_PRED_CHUNK_SPLITS], borders of 32 features [max_borders][32],
    // leaf values of the current chunk of trees [lv_floats]
    extern __shared__ unsigned char sb[];
    constexpr int RB = NT * CB_PRED_ROWS;
    constexpr int USTR = RB + 4;
    constexpr int NW = NT / 32;
    unsigned int* desc = reinterpret_cast<unsigned int*>(sb + (((size_t)a.U * USTR + 15) & ~(size_t)15));
    float* s_bd = reinterpret_cast<float*>(desc + CB_PRED_CHUNK_SPLITS);
    float* s_lv = s_bd + (size_t)a.max_borders * 32;
    const long long row0 = (long long)blockIdx.x * RB;
    const int nrow = (int)min((long long)RB, a.n - row0);
    // quantise, 32 used features at a time: their borders go to shared memory transposed ([border][feature], so a
    // lane's binary search never meets another lane's bank); then a warp takes one row at a time, lane = feature, so
    // that the row's values are read as one contiguous piece when the model uses neighbouring columns.
    // Row lr of the block belongs to thread lr % NT, slot lr / NT.
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int mb = a.max_borders;
        for (int c0 = 0; c0 < a.U; c0 += 32) {
            __syncthreads();
            for (int i = threadIdx.x; i < mb * 32; i += NT) {
                const int j = i >> 5, u = c0 + (i & 31);
                float bv = __int_as_float(0x7f800000);                 // +inf: never below a value
                if (u < a.U) {
                    const int b0 = a.border_off[u];
                    if (j < a.border_off[u + 1] - b0) bv = a.borders[b0 + j];
                }
                s_bd[i] = bv;
            }
            __syncthreads();
            const int u = c0 + lane;
            if (u < a.U) {
                const int col = a.used_feat[u];
                const int nbd = a.border_off[u + 1] - a.border_off[u];
                const bool nmax = a.nan_is_max && a.nan_is_max[u];
                unsigned char* dst = sb + (size_t)u * USTR;
                // four rows per step: their loads are issued together, the searches run while later loads land
                for (int lr0 = warp; lr0 < nrow; lr0 += 4 * NW) {
                    float v[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int lr = lr0 + NW * q;
                        v[q] = lr < nrow ? a.X[(row0 + lr) * a.ldx + col] : 0.0f;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int lr = lr0 + NW * q;
                        if (lr >= nrow) break;
                        int pos = 0;               // borders < v, fixed power-of-two steps
#pragma unroll
                        for (int step = 128; step > 0; step >>= 1) {
                            const int idx = pos + step;
                            if (idx <= mb && s_bd[((idx - 1) << 5) + lane] < v[q]) pos = idx;
                        }
                        dst[(lr % NT) * CB_PRED_ROWS + (lr / NT)] = (unsigned char)((v[q] != v[q]) ? (nmax ? nbd : 0) : pos);
                    }
                }
            }
        }
    }
    float acc[CB_PRED_ROWS][8];
    const int dims = min(a.dims, 8);
#pragma unroll
    for (int r = 0; r < CB_PRED_ROWS; ++r)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[r][k] = 0.0f;
    int t = 0;
    while (t < a.T) {
        // trees [t, t_end): as many as fit into the descriptor buffer and, when there is one, the leaf-value buffer
        const int s_begin = a.tree_split_off[t];
        const long long l_begin = a.tree_leaf_off[t];
        int t_end = t, s_end = s_begin;
        bool staged = a.lv_floats > 0;
        while (t_end < a.T && a.tree_split_off[t_end] + a.tree_depth[t_end] - s_begin <= CB_PRED_CHUNK_SPLITS &&
               (!staged || (a.tree_leaf_off[t_end] + (1ll << a.tree_depth[t_end]) - l_begin) * a.dims <= a.lv_floats)) {
            s_end = a.tree_split_off[t_end] + a.tree_depth[t_end];
            ++t_end;
        }
        if (t_end == t && staged && a.tree_depth[t] <= CB_PRED_CHUNK_SPLITS) {
            // this tree alone has more leaf values than the buffer holds: it reads them from global memory
            staged = false;
            s_end = s_begin + a.tree_depth[t];
            t_end = t + 1;
        }
        if (t_end == t) return;                     // a single tree deeper than the buffer cannot happen (depth <= 16)
        __syncthreads();
        for (int i = threadIdx.x; i < s_end - s_begin; i += NT)
            desc[i] = ((unsigned int)a.split_feat[s_begin + i] << 8) | (unsigned int)a.split_bin[s_begin + i];
        if (staged) {
            const long long cnt = (a.tree_leaf_off[t_end - 1] + (1ll << a.tree_depth[t_end - 1]) - l_begin) * a.dims;
            const float* src = a.leaf_vals + l_begin * a.dims;
            for (long long i = threadIdx.x; i < cnt; i += NT) s_lv[i] = __ldg(src + i);
        }
        __syncthreads();
        for (int tt = t; tt < t_end; ++tt) {
            const int depth = a.tree_depth[tt];
            const unsigned int* dsc = desc + (a.tree_split_off[tt] - s_begin);
            int leaf[CB_PRED_ROWS];
            if (CB_PRED_ROWS == 4 && depth <= 8) {
                // the bins of the thread's four rows sit in one word: one per-byte compare decides all four rows
                unsigned int leaf4 = 0u;
                for (int k = 0; k < depth; ++k) {
                    const unsigned int d = dsc[k];
                    const unsigned int w = reinterpret_cast<const unsigned int*>(sb + (size_t)(d >> 8) * USTR)[threadIdx.x];
                    const unsigned int m = __vcmpgtu4(w, __byte_perm(d, 0, 0x0000));
                    leaf4 |= (m & 0x01010101u) << k;
                }
#pragma unroll
                for (int r = 0; r < CB_PRED_ROWS; ++r) leaf[r] = (int)((leaf4 >> (8 * r)) & 255u);
            } else {
#pragma unroll
                for (int r = 0; r < CB_PRED_ROWS; ++r) leaf[r] = 0;
                for (int k = 0; k < depth; ++k) {
                    const unsigned int d = dsc[k];
                    const unsigned char* col = sb + (size_t)(d >> 8) * USTR + threadIdx.x * CB_PRED_ROWS;
                    const unsigned int thr = d & 255u;
#pragma unroll
                    for (int r = 0; r < CB_PRED_ROWS; ++r) leaf[r] |= ((unsigned int)col[r] > thr) << k;
                }
            }
            if (staged) {
                const float* lv0 = s_lv + (a.tree_leaf_off[tt] - l_begin) * a.dims;
#pragma unroll
                for (int r = 0; r < CB_PRED_ROWS; ++r) {
                    const float* lv = lv0 + leaf[r] * a.dims;
                    for (int k = 0; k < dims; ++k) acc[r][k] += lv[k];
                }
            } else {
                const float* lv0 = a.leaf_vals + a.tree_leaf_off[tt] * a.dims;
#pragma unroll
                for (int r = 0; r < CB_PRED_ROWS; ++r) {
                    const float* lv = lv0 + (long long)leaf[r] * a.dims;
                    for (int k = 0; k < dims; ++k) acc[r][k] += __ldg(lv + k);
                }
            }
        }
        t = t_end;
    }
#pragma unroll
    for (int r = 0; r < CB_PRED_ROWS; ++r) {
        const int lr = r * NT + threadIdx.x;
        if (lr < nrow)
            for (int k = 0; k < dims; ++k)
                a.out[(long long)k * a.n + row0 + lr] = acc[r][k] * a.scale + (a.bias ? a.bias[k] : 0.0f);
    }
}

CB_API int cb_predict_oblivious(const float* X, long long n, long long ldx, const int* used_feat, const float* borders,
                                const int* border_off, const unsigned char* nan_is_max, int U, const int* tree_depth,
                                const int* tree_split_off, const unsigned short* split_feat,
                                const unsigned char* split_bin, const long long* tree_leaf_off, const float* leaf_vals,
                                int T, int dims, float scale, const float* bias, float* out, int max_borders,
                                long long total_leaf_floats, cudaStream_t st) {
    if (n <= 0) return 0;
    if (max_borders < 1) max_borders = 1;
    if (max_borders > 255) return (int)cudaErrorInvalidValue;
    const size_t CB_PRED_SMEM_MAX = 224 * 1024;
    const size_t fixed = CB_PRED_CHUNK_SPLITS * 4 + (size_t)max_borders * 32 * sizeof(float);
    auto bins_bytes = [&](int nt, int rows) { return (((size_t)U * ((size_t)nt * rows + 4) + 15) & ~(size_t)15); };
    // geometry: (a) 1024 threads x 4 rows with a 64 KB leaf buffer when the bins of 4096 rows leave room for it (narrow
    // models: the staging of descriptors and leaf values is paid once per 4096 rows); (b) 256 threads x 4 rows with
    // what is left of 72 KB for leaf values (three blocks per SM); (c) 256 threads x 1 row for wide models, leaf
    // values in whatever remains.  CB200_PREDICT_LV=0 keeps the leaf values in global memory.
    // Small models (all leaf values within 32 KB, about 100 trees of depth 6) keep them in global memory: they stay in
    // L1, and several small blocks per SM hide the quantisation latency better than one large block (100 trees on 4M x
    // 28: 0.74 ms against 1.12 ms; 1000 trees: 9.0 ms against 7.2 ms the other way round).
    bool lv_on = total_leaf_floats * 4 > 32 * 1024;
    if (const char* e = getenv("CB200_PREDICT_LV")) lv_on = atoi(e) != 0;
    int nt = 1024, rows = 4;
    size_t lv_bytes = 0, pred_smem = 0;
    if (lv_on && bins_bytes(1024, 4) + fixed + 32 * 1024 <= CB_PRED_SMEM_MAX && n >= 4096ll * 148) {
        lv_bytes = CB_PRED_SMEM_MAX - bins_bytes(1024, 4) - fixed;
        if (lv_bytes > 64 * 1024) lv_bytes = 64 * 1024;
        pred_smem = bins_bytes(1024, 4) + fixed + lv_bytes;
    } else {
        nt = 256;
        pred_smem = bins_bytes(256, 4) + fixed;
        if (pred_smem > CB_PRED_SMEM_MAX) {
            rows = 1;
            pred_smem = bins_bytes(256, 1) + fixed;
        }
        if (pred_smem > CB_PRED_SMEM_MAX) return (int)cudaErrorInvalidValue;
        if (lv_on) {
            const size_t target = rows == 4 ? 72 * 1024 : CB_PRED_SMEM_MAX;       // keep three narrow blocks per SM
            lv_bytes = pred_smem < target ? target - pred_smem : 0;
            if (lv_bytes > 64 * 1024) lv_bytes = 64 * 1024;
            if (lv_bytes < 8 * 1024) lv_bytes = 0;
            pred_smem += lv_bytes;
        }
    }
    if (dims > 8) return (int)cudaErrorInvalidValue;
    CbPredictArgs a{X, n, ldx, used_feat, borders, border_off, nan_is_max, U, tree_depth, tree_split_off, split_feat,
                    split_bin, tree_leaf_off, leaf_vals, T, dims, scale, bias, out, max_borders, (int)(lv_bytes / 4)};
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_predict_kernel<4, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CB_PRED_SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_predict_kernel<4, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CB_PRED_SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_predict_kernel<1, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CB_PRED_SMEM_MAX);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    const unsigned pred_grid = (unsigned)((n + (long long)nt * rows - 1) / ((long long)nt * rows));
    if (nt == 1024) cb_predict_kernel<4, 1024><<<pred_grid, 1024, pred_smem, st>>>(a);
    else if (rows == 4) cb_predict_kernel<4, 256><<<pred_grid, 256, pred_smem, st>>>(a);
    else cb_predict_kernel<1, 256><<<pred_grid, 256, pred_smem, st>>>(a);
    CB_LAUNCH_CHECK();
    return 0;
}

// ======================================================================================================
// K15  metric partial sums on device: out[0] += sum w*loss, out[1] += sum w   (same loss math as training).
// With `vals`/`leaf` the pending tree is added on the fly (approx + vals[leaf]), so the learn metric after the
// newest tree can be read without touching the cursor.
__global__ void __launch_bounds__(256) cb_metric_kernel(int loss, float p0, float p1, const float* approx,
                                                        const float* target, const float* weight, long long n,
                                                        const unsigned short* leaf, const float* vals, double* out) {
    double s = 0.0, sw = 0.0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float w = weight ? weight[i] : 1.0f;
        const float a = approx[i] + (vals ? vals[leaf[i]] : 0.0f);
        s += (double)(w * cb_loss_eval(loss, p0, p1, a, target[i]).value);
        sw += (double)w;
    }
    s = cb_warp_sum_d(s); sw = cb_warp_sum_d(sw);
    __shared__ double red[2][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s; red[1][warp] = sw; }
    __syncthreads();
    if (threadIdx.x < 2) {
        double t = 0.0;
        for (int k = 0; k < (blockDim.x >> 5); ++k) t += red[threadIdx.x][k];
        atomicAdd(out + threadIdx.x, t);
    }
}
CB_API int cb_metric_sum(int loss, float p0, float p1, const float* approx, const float* target, const float* weight,
                         long long n, const unsigned short* leaf, const float* vals, double* out, int grid,
                         cudaStream_t st) {
    cb_metric_kernel<<<grid, 256, 0, st>>>(loss, p0, p1, approx, target, weight, n, leaf, vals, out);
    CB_LAUNCH_CHECK();
    return 0;
}

CB_API int cb_device_info(int* sm_count, int* max_smem_optin) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    return 0;
}

// ======================================================================================================
// Allocation-free variant of cb_leaf_pass (declared and documented in cb_noalloc.h).  The scratch of the pass
// (per-leaf sums, block counter) is a fixed array in this library's device image instead of caller memory.
#include "cb_noalloc.h"
#include <cstdio>

struct CbNoallocScratch {
    double sums[CB_NOALLOC_MAX_LEAVES * 3];
    unsigned int counter;
};
static __device__ __align__(256) CbNoallocScratch cb_noalloc_scratch;

#define CB_NOALLOC_MAX_DEVICES 64
static CbNoallocScratch* g_noalloc_ptr[CB_NOALLOC_MAX_DEVICES];     // device address of the array, per device
static char g_noalloc_error[256] = "";

CB_API const char* cb_noalloc_last_error(void) { return g_noalloc_error; }

CB_API int cb_leaf_pass_noalloc(int loss, float p0, float p1, const float* approx, const float* target,
                                const float* weight, const unsigned short* leaf, const float* ext_der,
                                const float* ext_hess, long long n, int L, float* delta, int first, int last, int newton,
                                float l2, float lr, float* cur_vals, float* model_vals, float* model_wts, int Lstride,
                                const int* iter_ptr, float* leaf_w, int grid, cudaStream_t st) {
    if (L < 1 || L > CB_NOALLOC_MAX_LEAVES) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error),
                 "cb_leaf_pass_noalloc: %d leaves requested, the built-in scratch holds at most %d", L,
                 CB_NOALLOC_MAX_LEAVES);
        return CB_NOALLOC_TOO_LARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cb_leaf_pass_noalloc: cannot identify the current device (%s)",
                 cudaGetErrorString(e));
        cudaGetLastError();
        return CB_NOALLOC_SETUP_FAILED;
    }
    if (dev >= CB_NOALLOC_MAX_DEVICES) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error),
                 "cb_leaf_pass_noalloc: device ordinal %d is beyond the %d devices this entry point keeps an address for",
                 dev, CB_NOALLOC_MAX_DEVICES);
        return CB_NOALLOC_SETUP_FAILED;
    }
    if (g_noalloc_ptr[dev] == nullptr) {
        // Set-up, once per device, with that device current: the name of a __device__ array is only a host-side
        // stand-in; the address a kernel can use comes from the runtime.
        CbNoallocScratch* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, cb_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cb_leaf_pass_noalloc: cudaGetSymbolAddress failed (%s)",
                     cudaGetErrorString(e));
            cudaGetLastError();
            return e != cudaSuccess ? (int)e : CB_NOALLOC_SETUP_FAILED;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    CbNoallocScratch* scratch = g_noalloc_ptr[dev];
    // the array keeps the previous call's contents: clear what this call needs to start from zero
    e = cudaMemsetAsync(scratch->sums, 0, sizeof(double) * 3 * (size_t)L, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(&scratch->counter, 0, sizeof(unsigned int), st);
    if (e != cudaSuccess) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cb_leaf_pass_noalloc: clearing the scratch failed (%s)",
                 cudaGetErrorString(e));
        cudaGetLastError();
        return (int)e;
    }
    CbLeafArgs a{loss, p0, p1, approx, target, weight, leaf, ext_der, ext_hess, n, L, delta, scratch->sums,
                 &scratch->counter, first, last, newton, l2, lr, cur_vals, model_vals, model_wts, Lstride, iter_ptr,
                 leaf_w, CbComm()};
    a.c.nranks = 1; a.c.rank = 0;
    int C = 32;
    while (C > 0 && (size_t)3 * L * C * 4 > 96 * 1024) C >>= 1;
    const int smem = 3 * L * C * 4;
    e = cudaFuncSetAttribute(cb_leaf_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cb_leaf_pass_noalloc: cudaFuncSetAttribute failed (%s)",
                 cudaGetErrorString(e));
        cudaGetLastError();
        return (int)e;
    }
    cb_leaf_pass_kernel<<<grid, 512, smem, st>>>(a, C);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(g_noalloc_error, sizeof(g_noalloc_error), "cb_leaf_pass_noalloc: launch failed (%s)", cudaGetErrorString(e));
        return (int)e;
    }
    g_noalloc_error[0] = 0;
    return 0;
}
