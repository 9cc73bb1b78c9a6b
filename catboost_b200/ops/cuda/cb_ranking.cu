// K4  YetiRank derivatives on the device (catboost/cuda/targets/kernel/yeti_rank_pointwise.cu:168,
// catboost/private/libs/algo/yetirank_helpers.cpp).  One block per query group:
//   for every permutation: key_i = approx_i + logit(u_i) (u uniform; the reference multiplies exp(approx) by u/(1-u)),
//   order the group by decreasing key (bitonic sort in shared memory), and for every pair of neighbours (k, k+1) with
//   different relevance add the PairLogit derivative of the pair with weight 0.15 * decay^k * |t_k - t_{k+1}|:
//   winner += w p, loser -= w p, both second derivatives += w p (1 - p), p = sigmoid(approx_loser - approx_winner).
// The result is the mean over the permutations, times the document weight.  Groups larger than CB_YETI_MAX_GROUP are
// left to the tensor implementation (the launcher reports them).
#include "cb_common.cuh"

#define CB_YETI_MAX_GROUP 2048
#define CB_YETI_THREADS 256

struct CbYetiArgs {
    const float* approx; const float* target; const float* weight;      // [n]
    const long long* offsets;                                            // [Q + 1]
    int Q;
    int permutations; float decay;
    unsigned long long seed;
    const float* noise;        // optional [permutations][n] uniforms in (0,1) (tests); null = counter-based generator
    long long n;
    float* der; float* hess;   // [n]
};

// MAXG = largest group the instantiation holds in shared memory.  Typical data has groups of tens to hundreds of
// documents: the small instantiation (256 documents, 128 threads, 5.5 KB) keeps sixteen blocks resident per SM, so
// the barriers of one group's sort overlap the work of the others; the large one covers groups up to 2048.
template <int MAXG, int THREADS>
__global__ void __launch_bounds__(THREADS) cb_yetirank_kernel(CbYetiArgs a) {
    __shared__ float s_key[MAXG];
    __shared__ unsigned short s_idx[MAXG];
    __shared__ float s_ap[MAXG];
    __shared__ float s_tg[MAXG];
    __shared__ float s_der[MAXG];
    __shared__ float s_hes[MAXG];
    for (int q = blockIdx.x; q < a.Q; q += gridDim.x) {
        const long long b = a.offsets[q], e = a.offsets[q + 1];
        const int L = (int)(e - b);
        if (L > MAXG) continue;                    // handled by the larger instantiation or by the caller
        int P2 = 1;
        while (P2 < L) P2 <<= 1;
        for (int i = threadIdx.x; i < L; i += blockDim.x) {
            s_ap[i] = a.approx[b + i];
            s_tg[i] = a.target[b + i];
            s_der[i] = 0.0f;
            s_hes[i] = 0.0f;
        }
        __syncthreads();
        if (L >= 2) {
            for (int perm = 0; perm < a.permutations; ++perm) {
                for (int i = threadIdx.x; i < P2; i += blockDim.x) {
                    float key = -3.0e38f;
                    if (i < L) {
                        float u = a.noise ? a.noise[(long long)perm * a.n + b + i]
                                          : cb_uniform01(cb_mix64(a.seed ^ cb_mix64(((unsigned long long)perm << 40) ^ (unsigned long long)(b + i))));
                        u = fminf(fmaxf(u, 1e-6f), 1.0f - 1e-6f);
                        key = s_ap[i] + __logf(u / (1.000001f - u));
                    }
                    s_key[i] = key;
                    s_idx[i] = (unsigned short)i;
                }
                __syncthreads();
                // bitonic sort, descending by key; ties by smaller index first (a stable order)
                for (int k = 2; k <= P2; k <<= 1) {
                    for (int j = k >> 1; j > 0; j >>= 1) {
                        for (int i = threadIdx.x; i < P2; i += blockDim.x) {
                            const int ixj = i ^ j;
                            if (ixj > i) {
                                const float ki = s_key[i], kj = s_key[ixj];
                                const unsigned short ii = s_idx[i], ij = s_idx[ixj];
                                const bool i_first = (ki > kj) || (ki == kj && ii < ij);     // i should precede ixj
                                const bool up = (i & k) == 0;
                                if (up ? !i_first : i_first) {
                                    s_key[i] = kj; s_key[ixj] = ki;
                                    s_idx[i] = ij; s_idx[ixj] = ii;
                                }
                            }
                        }
                        __syncthreads();
                    }
                }
                for (int k = threadIdx.x; k + 1 < L; k += blockDim.x) {
                    const int i1 = s_idx[k], i2 = s_idx[k + 1];
                    const float t1 = s_tg[i1], t2 = s_tg[i2];
                    const float wgt = 0.15f * __powf(a.decay, (float)k) * fabsf(t1 - t2);
                    if (wgt > 0.0f) {
                        const int win = t1 > t2 ? i1 : i2, los = t1 > t2 ? i2 : i1;
                        const float p = 1.0f / (1.0f + __expf(s_ap[win] - s_ap[los]));
                        const float g = wgt * p, h = wgt * p * (1.0f - p);
                        atomicAdd(&s_der[win], g);
                        atomicAdd(&s_der[los], -g);
                        atomicAdd(&s_hes[win], h);
                        atomicAdd(&s_hes[los], h);
                    }
                }
                __syncthreads();
            }
        }
        const float inv = 1.0f / (float)a.permutations;
        for (int i = threadIdx.x; i < L; i += blockDim.x) {
            const float w = a.weight ? a.weight[b + i] : 1.0f;
            a.der[b + i] = s_der[i] * inv * w;
            a.hess[b + i] = fmaxf(s_hes[i] * inv * w, 1e-16f);
        }
        __syncthreads();
    }
}

// Returns 0, or a CUDA error code.  Groups longer than cb_yetirank_max_group() are skipped (their der / hess entries are
// left untouched): the caller computes those with the tensor implementation.  max_group = size of the largest group
// (known to the caller from the offsets; it picks the instantiation).
CB_API int cb_yetirank_max_group() { return CB_YETI_MAX_GROUP; }

CB_API int cb_yetirank(const float* approx, const float* target, const float* weight, const long long* offsets, int Q,
                       long long n, int permutations, float decay, unsigned long long seed, const float* noise,
                       float* der, float* hess, int max_group, cudaStream_t st) {
    if (Q <= 0) return 0;
    CbYetiArgs a{approx, target, weight, offsets, Q, permutations, decay, seed, noise, n, der, hess};
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (max_group <= 256) {
        int grid = sms * 16;
        if (grid > Q) grid = Q;
        cb_yetirank_kernel<256, 128><<<grid, 128, 0, st>>>(a);
    } else {
        int grid = sms * 4;
        if (grid > Q) grid = Q;
        cb_yetirank_kernel<CB_YETI_MAX_GROUP, CB_YETI_THREADS><<<grid, CB_YETI_THREADS, 0, st>>>(a);
    }
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
