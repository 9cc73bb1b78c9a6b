// Derivatives of the query-wise and pair-wise ranking objectives (catboost/cuda/targets/kernel/query_rmse.cu:12-120,
// query_softmax.cu:9-150, pair_logit.cu:11-182).  Documents of a query are consecutive rows; offsets[q] .. offsets[q + 1].
//
//   QueryRMSE      der_i = w_i (t_i - a_i - shift_q),  shift_q = sum w (t - a) / sum w over the query;  hess_i = w_i
//   QuerySoftMax   p_i = w_i exp(beta a_i) / sum_q,  der_i = beta (w_i t_i - (sum_q w t) p_i),
//                  hess_i = max(beta^2 (sum_q w t) p_i (1 - p_i), 1e-16)
//   PairLogit      for a pair (winner, loser) with weight pw: p = sigmoid(a_loser - a_winner) is the probability of the
//                  wrong order; der_winner += pw p, der_loser -= pw p, both second derivatives += pw p (1 - p).
//                  From explicit pairs: one thread per pair, float atomics (the reference does the same).  From labels
//                  (every pair of a query whose labels differ): one warp per query, a lane owns a document and walks the
//                  query, so nothing is added atomically and the sums do not depend on a schedule.
//
// One warp per query in the query kernels: two or three passes over the query's rows with warp-shuffle reductions in
// between; queries are short (tens to hundreds of rows), so a pass is a few coalesced loads.
#include "cb_common.cuh"

#define CB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

__device__ __forceinline__ float cb_qw_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float cb_qw_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(256) cb_query_rmse_kernel(const float* approx, const float* target, const float* weight,
                                                            const long long* offsets, long long Q, float* der, float* hess) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long q = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < Q; q += warps) {
        const long long b = offsets[q], e = offsets[q + 1];
        float s = 0.0f, sw = 0.0f;
        for (long long i = b + lane; i < e; i += 32) {
            const float w = weight ? weight[i] : 1.0f;
            s += (target[i] - approx[i]) * w;
            sw += w;
        }
        s = cb_qw_sum(s);
        sw = cb_qw_sum(sw);
        const float shift = s / fmaxf(sw, 1e-30f);
        for (long long i = b + lane; i < e; i += 32) {
            const float w = weight ? weight[i] : 1.0f;
            der[i] = (target[i] - approx[i] - shift) * w;
            hess[i] = w;
        }
    }
}

__global__ void __launch_bounds__(256) cb_query_softmax_kernel(const float* approx, const float* target, const float* weight,
                                                               const long long* offsets, long long Q, float beta, float* der,
                                                               float* hess) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long q = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < Q; q += warps) {
        const long long b = offsets[q], e = offsets[q + 1];
        float m = -3.0e38f;
        for (long long i = b + lane; i < e; i += 32) m = fmaxf(m, approx[i] * beta);
        m = cb_qw_max(m);
        float z = 0.0f, swt = 0.0f;
        for (long long i = b + lane; i < e; i += 32) {
            const float w = weight ? weight[i] : 1.0f;
            z += __expf(approx[i] * beta - m) * w;
            swt += w * target[i];
        }
        z = fmaxf(cb_qw_sum(z), 1e-30f);
        swt = cb_qw_sum(swt);
        for (long long i = b + lane; i < e; i += 32) {
            const float w = weight ? weight[i] : 1.0f;
            const float p = __expf(approx[i] * beta - m) * w / z;
            der[i] = beta * (w * target[i] - swt * p);
            hess[i] = fmaxf(beta * beta * swt * p * (1.0f - p), 1e-16f);
        }
    }
}

__global__ void __launch_bounds__(256) cb_pair_logit_pairs_kernel(const float* approx, const long long* pairs, const float* pair_w,
                                                                  long long P, float* der, float* hess) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < P; k += stride) {
        const long long wi = pairs[2 * k], li = pairs[2 * k + 1];
        const float pw = pair_w ? pair_w[k] : 1.0f;
        const float p = 1.0f / (1.0f + __expf(approx[wi] - approx[li]));       // sigmoid(a_loser - a_winner)
        const float g = pw * p, h = pw * p * (1.0f - p);
        atomicAdd(der + wi, g);
        atomicAdd(der + li, -g);
        atomicAdd(hess + wi, h);
        atomicAdd(hess + li, h);
    }
}

__global__ void __launch_bounds__(256) cb_pair_logit_labels_kernel(const float* approx, const float* target, const long long* offsets,
                                                                   long long Q, float* der, float* hess) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long q = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < Q; q += warps) {
        const long long b = offsets[q], e = offsets[q + 1];
        for (long long i = b + lane; i < e; i += 32) {
            const float ai = approx[i], ti = target[i];
            float d = 0.0f, h = 0.0f;
            for (long long j = b; j < e; ++j) {                 // the whole warp reads the same row: one broadcast load
                const float aj = approx[j], tj = target[j];
                if (ti > tj) {                                  // i beats j: p = sigmoid(a_j - a_i)
                    const float p = 1.0f / (1.0f + __expf(ai - aj));
                    d += p;
                    h += p * (1.0f - p);
                } else if (tj > ti) {                           // j beats i: p = sigmoid(a_i - a_j)
                    const float p = 1.0f / (1.0f + __expf(aj - ai));
                    d -= p;
                    h += p * (1.0f - p);
                }
            }
            der[i] = d;
            hess[i] = fmaxf(h, 1e-16f);
        }
    }
}

// ---- PairLogit / PairAccuracy metrics -------------------------------------------------------------------------------
// out[0] += sum pw log(1 + exp(-(a_winner - a_loser))), out[1] += sum pw, out[2] += sum pw [a_winner > a_loser]
__device__ __forceinline__ void cb_qw_metric_flush(double l, double w, double c, double* out) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, o);
        w += __shfl_xor_sync(0xffffffffu, w, o);
        c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    if ((threadIdx.x & 31) == 0 && w != 0.0) { atomicAdd(out, l); atomicAdd(out + 1, w); atomicAdd(out + 2, c); }
}

__device__ __forceinline__ float cb_qw_softplus_neg(float d) {          // log(1 + exp(-d)), stable for both signs
    return d > 0.0f ? __logf(1.0f + __expf(-d)) : -d + __logf(1.0f + __expf(d));
}

__global__ void __launch_bounds__(256) cb_pair_metric_pairs_kernel(const float* approx, const long long* pairs, const float* pair_w,
                                                                   long long P, double* out) {
    double l = 0.0, w = 0.0, c = 0.0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < P; k += stride) {
        const float d = approx[pairs[2 * k]] - approx[pairs[2 * k + 1]];
        const float pw = pair_w ? pair_w[k] : 1.0f;
        l += (double)(pw * cb_qw_softplus_neg(d));
        w += (double)pw;
        c += d > 0.0f ? (double)pw : 0.0;
    }
    cb_qw_metric_flush(l, w, c, out);
}

__global__ void __launch_bounds__(256) cb_pair_metric_labels_kernel(const float* approx, const float* target, const long long* offsets,
                                                                    long long Q, double* out) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    double l = 0.0, w = 0.0, c = 0.0;
    for (long long q = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < Q; q += warps) {
        const long long b = offsets[q], e = offsets[q + 1];
        for (long long i = b + lane; i < e; i += 32) {
            const float ai = approx[i], ti = target[i];
            float fl = 0.0f, fw = 0.0f, fc = 0.0f;
            for (long long j = b; j < e; ++j) {
                if (ti > target[j]) {                         // i beats j
                    const float d = ai - approx[j];
                    fl += cb_qw_softplus_neg(d);
                    fw += 1.0f;
                    fc += d > 0.0f ? 1.0f : 0.0f;
                }
            }
            l += (double)fl; w += (double)fw; c += (double)fc;
        }
    }
    cb_qw_metric_flush(l, w, c, out);
}

static unsigned int cb_qw_grid(long long items, int per_block) {
    long long g = (items + per_block - 1) / per_block;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (unsigned int)g;
}

CB_API int cb_query_rmse_der(const float* approx, const float* target, const float* weight, const long long* offsets, long long Q,
                             float* der, float* hess, cudaStream_t st) {
    if (Q <= 0) return 0;
    cb_query_rmse_kernel<<<cb_qw_grid(Q, 8), 256, 0, st>>>(approx, target, weight, offsets, Q, der, hess);
    CB_LAUNCH_CHECK();
    return 0;
}

CB_API int cb_query_softmax_der(const float* approx, const float* target, const float* weight, const long long* offsets,
                                long long Q, float beta, float* der, float* hess, cudaStream_t st) {
    if (Q <= 0) return 0;
    cb_query_softmax_kernel<<<cb_qw_grid(Q, 8), 256, 0, st>>>(approx, target, weight, offsets, Q, beta, der, hess);
    CB_LAUNCH_CHECK();
    return 0;
}

// der and hess must be zero on entry.
CB_API int cb_pair_logit_pairs_der(const float* approx, const long long* pairs, const float* pair_w, long long P, float* der,
                                   float* hess, cudaStream_t st) {
    if (P <= 0) return 0;
    cb_pair_logit_pairs_kernel<<<cb_qw_grid(P, 256), 256, 0, st>>>(approx, pairs, pair_w, P, der, hess);
    CB_LAUNCH_CHECK();
    return 0;
}

CB_API int cb_pair_logit_labels_der(const float* approx, const float* target, const long long* offsets, long long Q, float* der,
                                    float* hess, cudaStream_t st) {
    if (Q <= 0) return 0;
    cb_pair_logit_labels_kernel<<<cb_qw_grid(Q, 8), 256, 0, st>>>(approx, target, offsets, Q, der, hess);
    CB_LAUNCH_CHECK();
    return 0;
}

// out: three doubles, zero on entry (loss sum, pair weight sum, weight of correctly ordered pairs).
CB_API int cb_pair_metric(const float* approx, const float* target, const long long* offsets, long long Q, const long long* pairs,
                          const float* pair_w, long long P, double* out, cudaStream_t st) {
    if (pairs) {
        if (P <= 0) return 0;
        cb_pair_metric_pairs_kernel<<<cb_qw_grid(P, 256), 256, 0, st>>>(approx, pairs, pair_w, P, out);
    } else {
        if (Q <= 0) return 0;
        cb_pair_metric_labels_kernel<<<cb_qw_grid(Q, 8), 256, 0, st>>>(approx, target, offsets, Q, out);
    }
    CB_LAUNCH_CHECK();
    return 0;
}
