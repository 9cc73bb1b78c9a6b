// MultiClass (softmax) on the device-resident trainer: derivatives, leaf estimation with the full K x K Hessian block
// per leaf, and the loss for logging.  The tree structure comes from the same fused level kernels as the
// one-dimensional losses, fed with K derivative columns + one weight column (S = K + 1 statistics).
//
// Behaviour reproduced from the reference (not its code): softmax derivatives and second derivatives
// (catboost/cuda/targets/kernel/multilogit.cu:10-211), one Newton step per leaf with the K x K Hessian block solved
// by Cholesky (catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:91-117,
// catboost/private/libs/algo/approx_calcer_multi.cpp), l2 on the diagonal.
#include "cb_common.cuh"
#include "cb_comm.cuh"

#define CB_MC_MAX_K 16
#define CB_MC_TRI(K) ((K) * ((K) + 1) / 2)

__device__ __forceinline__ float cb_mc_boot(int type, float p, unsigned long long h) {
    switch (type) {
        default: return 1.0f;
        case 1: {
            const float e = -__logf(cb_uniform01(h) + 1e-20f);
            return (p == 1.0f) ? e : __powf(e, p);
        }
        case 2: return cb_uniform01(h) < p ? 1.0f : 0.0f;
        case 3: {
            float u = cb_uniform01(h);
            float pk = __expf(-p), cdf = pk;
            int k = 0;
            while (u > cdf && k < 32) { ++k; pk *= p / k; cdf += pk; }
            return (float)k;
        }
    }
}

struct CbMcGradArgs {
    float* approx;                 // [K][npad], updated in place by the previous tree's leaf values
    const float* target;           // class index as float
    const float* weight;           // or null
    unsigned short* leaf;          // leaf of the previous tree on entry, zero on exit
    const float* cur_vals;         // [L][K] leaf values of the previous tree (lr applied), or null
    long long n, npad;
    int K;
    float* stats;                  // [K + 1][npad]: w * (1[y == k] - p_k), then the weight column
    int newton_stats;              // weight column = mean over k of w p_k (1 - p_k) instead of w
    int boot_type; float boot_p; unsigned long long seed;
    const int* iter_ptr;
    double* scal;                  // [0] += sum w * loss, [1] += sum w, [2] += sum |w der|^2, [3] += docs
    float* statmax;                // [K + 1] max |statistic| of this iteration (atomicMax on the bit patterns)
};

// CB_MC_V documents per thread and step (loads of all of them issued before the arithmetic, so twice the bytes are in
// flight per warp); every row of approx / stats is read and written with coalesced 4-byte accesses.  KM bounds the
// class count at compile time: the per-class arrays live in registers, and a kernel sized for 16 classes held 87 of
// them (two blocks per SM) when most models have a handful of classes.
#define CB_MC_V 2
template <int KM>
__global__ void __launch_bounds__(256, KM <= 8 ? 3 : 2) cb_mc_grad_kernel(CbMcGradArgs a) {
    const int K = a.K;
    const int it = *a.iter_ptr;
    double s_loss = 0.0, s_w = 0.0, s_d2 = 0.0, s_n = 0.0;
    float mx[KM + 1];
#pragma unroll
    for (int k = 0; k <= KM; ++k) mx[k] = 0.0f;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < a.npad; i0 += stride * CB_MC_V) {
        float ap[CB_MC_V][KM];
        int lf[CB_MC_V], y[CB_MC_V];
        float w[CB_MC_V];
        bool in[CB_MC_V], live[CB_MC_V];
#pragma unroll
        for (int v = 0; v < CB_MC_V; ++v) {
            const long long i = i0 + v * stride;
            in[v] = i < a.npad;
            live[v] = i < a.n;
            lf[v] = in[v] ? (int)a.leaf[i] : 0;
            y[v] = live[v] ? (int)a.target[i] : 0;
            w[v] = (a.weight && in[v]) ? a.weight[i] : 1.0f;
#pragma unroll
            for (int k = 0; k < KM; ++k)
                if (k < K) ap[v][k] = in[v] ? a.approx[(long long)k * a.npad + i] : 0.0f;
        }
#pragma unroll
        for (int v = 0; v < CB_MC_V; ++v) {
            if (!in[v]) continue;
            const long long i = i0 + v * stride;
            a.leaf[i] = 0;
            float m = -3.0e38f;
#pragma unroll
            for (int k = 0; k < KM; ++k) {
                if (k < K) {
                    float x = ap[v][k];
                    if (a.cur_vals) { x += a.cur_vals[lf[v] * K + k]; a.approx[(long long)k * a.npad + i] = x; }
                    ap[v][k] = x;
                    m = fmaxf(m, x);
                }
            }
            float Z = 0.0f;
#pragma unroll
            for (int k = 0; k < KM; ++k)
                if (k < K) { ap[v][k] = __expf(ap[v][k] - m); Z += ap[v][k]; }
            const float invZ = 1.0f / Z;
            const float wb = (a.boot_type && live[v])
                ? cb_mc_boot(a.boot_type, a.boot_p, cb_mix64(a.seed ^ cb_mix64(((unsigned long long)it << 40) ^ (unsigned long long)i)))
                : 1.0f;
            float hs = 0.0f, d2 = 0.0f, py = 1.0f;
#pragma unroll
            for (int k = 0; k < KM; ++k) {
                if (k < K) {
                    const float p = ap[v][k] * invZ;
                    if (k == y[v]) py = p;
                    const float d = w[v] * ((k == y[v] ? 1.0f : 0.0f) - p);
                    const float st = live[v] ? wb * d : 0.0f;
                    a.stats[(long long)k * a.npad + i] = st;
                    mx[k] = fmaxf(mx[k], fabsf(st));
                    hs += p * (1.0f - p);
                    d2 += d * d;
                }
            }
            const float wc = live[v] ? wb * w[v] * (a.newton_stats ? hs / (float)K : 1.0f) : 0.0f;
            a.stats[(long long)K * a.npad + i] = wc;
            mx[KM] = fmaxf(mx[KM], fabsf(wc));
            if (live[v]) {
                s_loss += (double)(-w[v] * __logf(fmaxf(py, 1e-38f))); s_w += (double)w[v]; s_d2 += (double)d2; s_n += 1.0;
            }
        }
    }
    __shared__ double red[4][8];
    s_loss = cb_warp_sum_d(s_loss); s_w = cb_warp_sum_d(s_w); s_d2 = cb_warp_sum_d(s_d2); s_n = cb_warp_sum_d(s_n);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s_loss; red[1][warp] = s_w; red[2][warp] = s_d2; red[3][warp] = s_n; }
    __syncthreads();
    if (threadIdx.x < 4) {
        double t = 0.0;
        for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += red[threadIdx.x][k];
        atomicAdd(a.scal + threadIdx.x, t);
    }
    if (a.statmax) {
#pragma unroll
        for (int k = 0; k <= KM; ++k) {
            if (k < K || k == KM) {
                float v = mx[k];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
                if (lane == 0) atomicMax(reinterpret_cast<int*>(a.statmax) + (k == KM ? K : k), __float_as_int(v));
            }
        }
    }
}

CB_API int cb_mc_max_classes(void) { return CB_MC_MAX_K; }

CB_API int cb_mc_grad(float* approx, const float* target, const float* weight, unsigned short* leaf, const float* cur_vals,
                      long long n, long long npad, int K, float* stats, int newton_stats, int boot_type, float boot_p,
                      unsigned long long seed, const int* iter_ptr, double* scal, float* statmax, int grid, cudaStream_t st) {
    if (K < 2 || K > CB_MC_MAX_K) return (int)cudaErrorInvalidValue;
    CbMcGradArgs a{approx, target, weight, leaf, cur_vals, n, npad, K, stats, newton_stats, boot_type, boot_p, seed, iter_ptr,
                   scal, statmax};
    // One wave of resident blocks: `grid` is the caller's SM count times a guess, the occupancy query knows the real
    // number of blocks per SM for this instantiation.
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    auto kern = K <= 4 ? cb_mc_grad_kernel<4> : K <= 8 ? cb_mc_grad_kernel<8> : cb_mc_grad_kernel<16>;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, 256, 0) == cudaSuccess && occ > 0 && sms > 0) grid = sms * occ;
    const long long need = (npad + 255) / 256;
    if (grid > need) grid = (int)need;
    if (grid < 1) grid = 1;
    kern<<<grid, 256, 0, st>>>(a);
    return (int)cudaGetLastError();
}

// ---- leaf estimation ---------------------------------------------------------------------------------------
// Per leaf: g[K] = sum w (1[y == k] - p_k), H = sum w (diag(p) - p p^T) as the upper triangle (Newton) or the weight
// sum (Gradient), and the weight sum (first pass).  Layout of one leaf's NS doubles: g[K], H tri [K (K + 1) / 2], w.
struct CbMcLeafArgs {
    const float* approx; const float* target; const float* weight; const unsigned short* leaf;
    long long n, npad; int K, L;
    const float* delta;      // [L][K] running (unscaled) leaf values, read when !first
    double* sums;            // [L][NS], zero on entry; the solve kernel zeroes it again
    int first, newton;
    int copies;              // replicas of a shared cell (power of two)
    float inv_wmax;          // 1 / largest document weight (1 without weights)
};

__device__ __forceinline__ int cb_mc_ns(int K) { return K + CB_MC_TRI(K) + 1; }

// Shared cells are int32 fixed point (15 bits + sign of value / largest weight per addend): fp32 shared atomics are
// compare-and-swap loops on this part and 21 of them per document (K = 5) on 64 x 21 hot cells took 2.2 ms per pass at
// 4M documents; native integer reductions do not retry, and integer sums do not depend on the order of the documents.
// A block adds at most 2^15 documents between two flushes to the global double sums, so a cell cannot overflow.
// `copies` replicas of every cell (lane & (copies - 1)) spread the lanes of a warp that meet in one leaf.
__global__ void __launch_bounds__(256) cb_mc_leaf_pass_kernel(CbMcLeafArgs a) {
    extern __shared__ int cells[];            // [L][NS][copies]
    const int K = a.K, L = a.L, NS = cb_mc_ns(K), C = a.copies;
    const int cshift = 31 - __clz(C);
    const int copy = threadIdx.x & (C - 1);
    const float qs = 32768.0f * a.inv_wmax;
    for (int i = threadIdx.x; i < L * NS * C; i += blockDim.x) cells[i] = 0;
    __syncthreads();
    const long long stride = (long long)gridDim.x * blockDim.x;
    int since = 0;
    for (long long base = (long long)blockIdx.x * blockDim.x; base < a.n; base += stride) {
        const long long i = base + threadIdx.x;
        if (i < a.n) {
            const int l = a.leaf[i];
            float p[CB_MC_MAX_K];
            float m = -3.0e38f;
#pragma unroll
            for (int k = 0; k < CB_MC_MAX_K; ++k) {
                if (k < K) {
                    float v = a.approx[(long long)k * a.npad + i];
                    if (!a.first) v += a.delta[l * K + k];
                    p[k] = v;
                    m = fmaxf(m, v);
                }
            }
            float Z = 0.0f;
#pragma unroll
            for (int k = 0; k < CB_MC_MAX_K; ++k)
                if (k < K) { p[k] = __expf(p[k] - m); Z += p[k]; }
            const float invZ = 1.0f / Z;
            const int y = (int)a.target[i];
            const float w = (a.weight ? a.weight[i] : 1.0f) * qs;
            int* c = cells + (((size_t)l * NS) << cshift) + copy;
            int t = K;
#pragma unroll
            for (int k = 0; k < CB_MC_MAX_K; ++k) {
                if (k < K) {
                    const float pk = p[k] * invZ;
                    atomicAdd(c + (k << cshift), __float2int_rn(w * ((k == y ? 1.0f : 0.0f) - pk)));
                    if (a.newton) {
#pragma unroll
                        for (int j = 0; j < CB_MC_MAX_K; ++j) {
                            if (j >= k && j < K) {
                                const float pj = p[j] * invZ;
                                atomicAdd(c + (t << cshift), __float2int_rn(w * ((j == k ? pk : 0.0f) - pk * pj)));
                                ++t;
                            }
                        }
                    }
                }
            }
            if (a.first) atomicAdd(c + ((NS - 1) << cshift), __float2int_rn(w));
        }
        since += blockDim.x;
        const bool last = base + stride >= a.n;
        if (last || since + (int)blockDim.x > 32768) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < L * NS; idx += blockDim.x) {
                long long v = 0;
                for (int cc = 0; cc < C; ++cc) { v += cells[(idx << cshift) + cc]; cells[(idx << cshift) + cc] = 0; }
                if (v != 0) atomicAdd(a.sums + idx, (double)v / (double)qs);
            }
            __syncthreads();
            since = 0;
        }
    }
}

struct CbMcSolveArgs {
    double* sums;            // [L][NS] complete sums of this rank; zero on exit
    double* combined;        // [L][NS] scratch (several ranks: the sum over the ranks)
    float* delta;            // [L][K] in / out
    float* leaf_w;           // [L] written on the first pass
    int K, L, first, last, newton;
    float l2, lr;
    float* cur_vals;         // [L][K] lr * delta after the last pass
    float* model_vals; float* model_wts; int Lstride; const int* iter_ptr;
    CbComm c;
};

// One block.  Several ranks: the sums are exchanged as tagged words through the peer mailboxes and added in rank order
// on every rank, so all ranks take bit-identical steps.  Then one thread per leaf solves (H + l2 I) d = g by Cholesky.
__global__ void __launch_bounds__(256) cb_mc_leaf_solve_kernel(CbMcSolveArgs a) {
    const int K = a.K, L = a.L, NS = cb_mc_ns(K);
    const int R = a.c.nranks, me = a.c.rank;
    const double* S = a.sums;
    if (R > 1) {
        __shared__ unsigned long long s_epoch;
        if (threadIdx.x == 0) { s_epoch = a.c.epoch[0] + 1; a.c.epoch[0] = s_epoch; }
        __syncthreads();
        const unsigned long long epoch = s_epoch;
        const unsigned int tag = cb_ll_tag(epoch);
        const int parity = (int)(epoch & 1ull);
        const int cnt = L * NS;
        for (long long idx = threadIdx.x; idx < (long long)cnt * R; idx += blockDim.x) {
            const int r = (int)(idx / cnt), i = (int)(idx - (long long)r * cnt);
            const unsigned long long bits = (unsigned long long)__double_as_longlong(a.sums[i]);
            unsigned long long* box = cb_ll_box(a.c, r, parity, me);
            cb_ll_store(box + 2 * i, (unsigned int)bits, tag);
            cb_ll_store(box + 2 * i + 1, (unsigned int)(bits >> 32), tag);
        }
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            double t = 0.0;
            for (int r = 0; r < R; ++r) {
                const unsigned long long* box = cb_ll_box(a.c, me, parity, r);
                const unsigned int lo = cb_ll_load(box + 2 * i, tag, a.c.timeout_ns, a.c.status, CB_TIMEOUT_MAILBOX, r);
                const unsigned int hi = cb_ll_load(box + 2 * i + 1, tag, a.c.timeout_ns, a.c.status, CB_TIMEOUT_MAILBOX, r);
                t += __longlong_as_double((long long)(((unsigned long long)hi << 32) | lo));
            }
            a.combined[i] = t;
        }
        __syncthreads();
        S = a.combined;
    }
    const int it = *a.iter_ptr;
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const double* s = S + (size_t)l * NS;
        if (a.first) a.leaf_w[l] = (float)s[NS - 1];
        const double sw = (double)a.leaf_w[l];
        double d[CB_MC_MAX_K];
        if (a.newton) {
            // Cholesky of A = H + l2 I (upper triangle, row-major packed), then two triangular solves
            double A[CB_MC_TRI(CB_MC_MAX_K)];
            int t = 0;
            for (int k = 0; k < K; ++k)
                for (int j = k; j < K; ++j, ++t) A[t] = s[K + t] + (j == k ? (double)a.l2 : 0.0);
            // packed index of (r, c), r <= c
            #define CB_MC_AT(r, c) A[(r) * K - (r) * ((r) - 1) / 2 + ((c) - (r))]
            bool ok = true;
            for (int k = 0; k < K && ok; ++k) {
                double diag = CB_MC_AT(k, k);
                for (int q = 0; q < k; ++q) diag -= CB_MC_AT(q, k) * CB_MC_AT(q, k);
                if (!(diag > 1e-300)) { ok = false; break; }
                diag = sqrt(diag);
                CB_MC_AT(k, k) = diag;
                for (int j = k + 1; j < K; ++j) {
                    double v = CB_MC_AT(k, j);
                    for (int q = 0; q < k; ++q) v -= CB_MC_AT(q, k) * CB_MC_AT(q, j);
                    CB_MC_AT(k, j) = v / diag;
                }
            }
            if (ok) {
                // U^T z = g, U d = z   (A = U^T U with U upper triangular in the packed array)
                for (int k = 0; k < K; ++k) {
                    double v = s[k];
                    for (int q = 0; q < k; ++q) v -= CB_MC_AT(q, k) * d[q];
                    d[k] = v / CB_MC_AT(k, k);
                }
                for (int k = K - 1; k >= 0; --k) {
                    double v = d[k];
                    for (int j = k + 1; j < K; ++j) v -= CB_MC_AT(k, j) * d[j];
                    d[k] = v / CB_MC_AT(k, k);
                }
            } else {
                for (int k = 0; k < K; ++k) d[k] = 0.0;
            }
            #undef CB_MC_AT
        } else {
            const double den = sw + (double)a.l2;
            for (int k = 0; k < K; ++k) d[k] = den > 0.0 ? s[k] / den : 0.0;
        }
        for (int k = 0; k < K; ++k) {
            const float v = (a.first ? 0.0f : a.delta[l * K + k]) + (float)d[k];
            a.delta[l * K + k] = v;
            if (a.last) {
                a.cur_vals[l * K + k] = a.lr * v;
                if (a.model_vals) a.model_vals[(long long)it * a.Lstride * K + (long long)l * K + k] = a.lr * v;
            }
        }
        if (a.last && a.model_wts) a.model_wts[(long long)it * a.Lstride + l] = (float)sw;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < L * NS; i += blockDim.x) a.sums[i] = 0.0;
}

CB_API int cb_mc_leaf_sums_doubles(int K, int L) { return L * (K + CB_MC_TRI(K) + 1); }
CB_API int cb_mc_leaf_msg_bytes(int K, int L) { return L * (K + CB_MC_TRI(K) + 1) * 16; }
CB_API int cb_mc_leaf_smem_bytes(int K, int L) { return L * (K + CB_MC_TRI(K) + 1) * 4; }

CB_API int cb_mc_leaf_step(const float* approx, const float* target, const float* weight, const unsigned short* leaf,
                           long long n, long long npad, int K, int L, float* delta, double* sums, double* combined,
                           float* leaf_w, int first, int last, int newton, float l2, float lr, float* cur_vals,
                           float* model_vals, float* model_wts, int Lstride, const int* iter_ptr, const CbComm* comm,
                           float wmax, int grid, cudaStream_t st) {
    if (K < 2 || K > CB_MC_MAX_K) return (int)cudaErrorInvalidValue;
    int smem = cb_mc_leaf_smem_bytes(K, L);
    if (smem > 96 * 1024) return -2;
    int copies = 1;
    while (copies < 4 && smem * 2 <= 48 * 1024) { copies *= 2; smem *= 2; }
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_mc_leaf_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    CbMcLeafArgs p{approx, target, weight, leaf, n, npad, K, L, delta, sums, first, newton, copies,
                   1.0f / (wmax > 0.0f ? wmax : 1.0f)};
    cb_mc_leaf_pass_kernel<<<grid, 256, smem, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    CbMcSolveArgs s{sums, combined, delta, leaf_w, K, L, first, last, newton, l2, lr, cur_vals, model_vals, model_wts, Lstride,
                    iter_ptr, CbComm()};
    if (comm) s.c = *comm; else { s.c.nranks = 1; s.c.rank = 0; }
    if (s.c.nranks > 1 && cb_mc_leaf_msg_bytes(K, L) > s.c.mbox_bytes) return -2;
    cb_mc_leaf_solve_kernel<<<1, 256, 0, st>>>(s);
    return (int)cudaGetLastError();
}

// ---- loss for logging ---------------------------------------------------------------------------------------
// out[0] += sum w * (-log p_y), out[1] += sum w, evaluated at approx (+ vals[leaf] when leaf is given).
__global__ void __launch_bounds__(256) cb_mc_metric_kernel(const float* approx, const float* target, const float* weight,
                                                           long long n, long long npad, int K, const unsigned short* leaf,
                                                           const float* vals, double* out) {
    double s_loss = 0.0, s_w = 0.0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int l = leaf ? leaf[i] : 0;
        const int y = (int)target[i];
        float m = -3.0e38f, ay = 0.0f;
        float ap[CB_MC_MAX_K];
#pragma unroll
        for (int k = 0; k < CB_MC_MAX_K; ++k) {
            if (k < K) {
                float v = approx[(long long)k * npad + i];
                if (leaf) v += vals[l * K + k];
                ap[k] = v;
                if (k == y) ay = v;
                m = fmaxf(m, v);
            }
        }
        float Z = 0.0f;
#pragma unroll
        for (int k = 0; k < CB_MC_MAX_K; ++k)
            if (k < K) Z += __expf(ap[k] - m);
        const float w = weight ? weight[i] : 1.0f;
        s_loss += (double)(w * (m + __logf(Z) - ay));
        s_w += (double)w;
    }
    __shared__ double red[2][8];
    s_loss = cb_warp_sum_d(s_loss); s_w = cb_warp_sum_d(s_w);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][warp] = s_loss; red[1][warp] = s_w; }
    __syncthreads();
    if (threadIdx.x < 2) {
        double t = 0.0;
        for (int k = 0; k < (int)(blockDim.x >> 5); ++k) t += red[threadIdx.x][k];
        atomicAdd(out + threadIdx.x, t);
    }
}

CB_API int cb_mc_metric(const float* approx, const float* target, const float* weight, long long n, long long npad, int K,
                        const unsigned short* leaf, const float* vals, double* out, int grid, cudaStream_t st) {
    if (K < 2 || K > CB_MC_MAX_K) return (int)cudaErrorInvalidValue;
    cb_mc_metric_kernel<<<grid, 256, 0, st>>>(approx, target, weight, n, npad, K, leaf, vals, out);
    return (int)cudaGetLastError();
}
