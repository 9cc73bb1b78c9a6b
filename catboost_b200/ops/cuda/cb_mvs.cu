// Minimal-variance sampling (MVS) for the pointwise device trainer: importance sampling of the documents by the size
// of their gradient.  Behaviour follows catboost/cuda/cuda_util/kernel/mvs.cu:22-180 and
// catboost/private/libs/algo/mvs.cpp: documents are taken in blocks of 8192; inside a block every document gets the
// candidate c = sqrt(der^2 + lambda), the block's threshold mu solves  sum_i min(1, c_i / mu) = subsample * m, a document
// with c >= mu is kept with weight 1 and any other one is kept with probability c / mu and weight mu / c.  Blocks are
// independent, so nothing crosses ranks.
//
// One 1024-thread block per 8192 documents, 8 per thread in registers.  The threshold comes from 40 bisection steps on
// the monotone function mu -> sum min(1, c / mu) (a block-wide sum each), not from a sort: 40 block reductions cost
// about as much as one pass of a sort of 8192 keys and need no scratch memory.  The kernel multiplies both statistic
// rows (derivative and weight / second derivative) of the trainer in place and raises the running maxima the histogram
// quantisation scales by.
#include "cb_common.cuh"

#define CB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

#define CB_MVS_ITEMS 8
#define CB_MVS_THREADS 1024
#define CB_MVS_BLOCK (CB_MVS_ITEMS * CB_MVS_THREADS)

__device__ __forceinline__ float cb_mvs_block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < (CB_MVS_THREADS >> 5) ? red[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

__global__ void __launch_bounds__(CB_MVS_THREADS) cb_mvs_kernel(float* stats, long long npad, long long n, float rate,
                                                                float lambda, unsigned long long seed, const int* iter_ptr,
                                                                float* statmax, float* mu_out) {
    __shared__ float red[32];
    const long long base = (long long)blockIdx.x * CB_MVS_BLOCK;
    float d[CB_MVS_ITEMS], c[CB_MVS_ITEMS];
    float sum_abs = 0.0f, live = 0.0f;
#pragma unroll
    for (int k = 0; k < CB_MVS_ITEMS; ++k) {
        const long long i = base + (long long)k * CB_MVS_THREADS + threadIdx.x;
        const bool ok = i < n;
        d[k] = ok ? stats[i] : 0.0f;
        sum_abs += fabsf(d[k]);
        live += ok ? 1.0f : 0.0f;
    }
    const float m = cb_mvs_block_sum(live, red);
    if (m <= 0.0f) return;
    // lambda < 0: the square of the block's mean absolute derivative (the reference's default on the first iteration)
    float lam = lambda;
    if (lam < 0.0f) {
        const float mean = cb_mvs_block_sum(sum_abs, red) / m;
        lam = mean * mean;
    }
    float sum_c = 0.0f, max_c = 0.0f;
#pragma unroll
    for (int k = 0; k < CB_MVS_ITEMS; ++k) {
        const long long i = base + (long long)k * CB_MVS_THREADS + threadIdx.x;
        c[k] = i < n ? sqrtf(d[k] * d[k] + lam) : 0.0f;
        sum_c += c[k];
        max_c = fmaxf(max_c, c[k]);
    }
    const float total_c = cb_mvs_block_sum(sum_c, red);
    const float target = rate * m;
    // f(mu) = sum min(1, c / mu) falls from m (mu -> 0) to total_c / mu (mu >= max c): the root lies in (0, hi]
    float lo = 0.0f, hi = fmaxf(total_c / fmaxf(target, 1e-20f), 1e-30f);
    {
        // hi must satisfy f(hi) <= target also when hi < max c; grow it until it does (at most a few doublings)
        for (int g = 0; g < 64; ++g) {
            float f = 0.0f;
#pragma unroll
            for (int k = 0; k < CB_MVS_ITEMS; ++k) f += fminf(1.0f, c[k] / hi);
            f = cb_mvs_block_sum(f, red);
            if (f <= target) break;
            hi *= 2.0f;
        }
    }
    for (int it = 0; it < 40; ++it) {
        const float mid = 0.5f * (lo + hi);
        float f = 0.0f;
#pragma unroll
        for (int k = 0; k < CB_MVS_ITEMS; ++k) f += fminf(1.0f, c[k] / mid);
        f = cb_mvs_block_sum(f, red);
        if (f > target) lo = mid; else hi = mid;
    }
    const float mu = hi;
    if (mu_out && threadIdx.x == 0) mu_out[blockIdx.x] = mu;
    const int iter = *iter_ptr;
    float m0 = 0.0f, m1 = 0.0f;
    float* st1 = stats + npad;
#pragma unroll
    for (int k = 0; k < CB_MVS_ITEMS; ++k) {
        const long long i = base + (long long)k * CB_MVS_THREADS + threadIdx.x;
        if (i >= n) continue;
        float w = 1.0f;
        if (c[k] < mu) {
            const unsigned long long r = cb_mix64(seed ^ cb_mix64(((unsigned long long)iter << 40) ^ (unsigned long long)i ^ 0x6D76735F6B656570ull));
            const float u = (float)(r >> 40) * (1.0f / 16777216.0f);
            const float p = c[k] / mu;
            w = u < p ? 1.0f / p : 0.0f;
        }
        const float a0 = d[k] * w, a1 = st1[i] * w;
        stats[i] = a0;
        st1[i] = a1;
        m0 = fmaxf(m0, fabsf(a0));
        m1 = fmaxf(m1, fabsf(a1));
    }
    if (statmax) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
            m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
        }
        if ((threadIdx.x & 31) == 0) {
            atomicMax(reinterpret_cast<int*>(statmax), __float_as_int(m0));
            atomicMax(reinterpret_cast<int*>(statmax) + 1, __float_as_int(m1));
        }
    }
}

CB_API int cb_mvs_block_docs() { return CB_MVS_BLOCK; }

// stats: [2][npad] (derivative row, weight / second-derivative row), both multiplied by the sampling weight in place.
// lambda < 0 = per-block estimate.  mu_out (optional): the threshold of every block, [ceil(n / 8192)].
CB_API int cb_mvs_sample(float* stats, long long npad, long long n, float rate, float lambda, unsigned long long seed,
                         const int* iter_ptr, float* statmax, float* mu_out, cudaStream_t st) {
    if (n <= 0 || rate >= 1.0f) return 0;
    const unsigned int blocks = (unsigned int)((n + CB_MVS_BLOCK - 1) / CB_MVS_BLOCK);
    cb_mvs_kernel<<<blocks, CB_MVS_THREADS, 0, st>>>(stats, npad, n, rate, lambda, seed, iter_ptr, statmax, mu_out);
    CB_LAUNCH_CHECK();
    return 0;
}
