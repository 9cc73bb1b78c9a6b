// K4  YetiRank derivatives on the device (catboost/cuda/targets/kernel/yeti_rank_pointwise.cu:168,
// catboost/private/libs/algo/yetirank_helpers.cpp).  One block per query group:
//   for every permutation: key_i = approx_i + logit(u_i) (u uniform; the reference multiplies exp(approx) by u/(1-u)),
//   order the group by decreasing key (bitonic sort in shared memory), and for every pair of neighbours (k, k+1) with
//   different relevance add the PairLogit derivative of the pair with weight 0.15 * decay^k * |t_k - t_{k+1}|:
//   winner += w p, loser -= w p, both second derivatives += w p (1 - p), p = sigmoid(approx_loser - approx_winner).
// The result is the mean over the permutations, times the document weight.  Groups of up to 256 documents go to the
// warp-per-permutation kernel further down, longer ones to this block-wide kernel; groups larger than
// CB_YETI_MAX_GROUP are left to the tensor implementation (the launcher reports them).
#include "cb_common.cuh"
#include <cstdlib>

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
    int min_group;             // groups of at most this many documents are skipped (another kernel took them)
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
        if (L > MAXG || L <= a.min_group) continue;          // handled by another kernel or by the caller
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

// ---- groups of up to 256 documents: one warp per permutation ---------------------------------------------------------
// The permutations of a group are independent, so every warp of the block takes permutations of its own: keys and
// document indices live in registers (element e = r * 32 + lane), the bitonic network exchanges them with shuffles
// (strides below 32) or between a lane's own registers (strides of 32 and more), and no block barrier is needed inside a
// permutation -- the block-wide version spends 28 barriers per permutation on a 128-document group.  Pair terms are
// added to shared int32 cells in fixed point (scale chosen from the group's label range so that the cell cannot
// overflow): integer reductions do not retry under contention and their sum does not depend on the order of the warps.
// Measured on 2M documents in queries of 5..200, 10 permutations: 1.75 ms for the block-wide kernel, 1.07 ms for this one
// (now bound by the instructions of the sorting network: about 11 per compare-exchange of a (key, index) pair).
#define CB_YETI_WARP_GROUP 256

template <int R>
__device__ __forceinline__ void cb_yeti_warp_sort(float (&key)[R], int (&idx)[R], int lane) {
#pragma unroll
    for (int k = 2; k <= 32 * R; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j >= 32) {
                const int rj = j >> 5;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int rp = r ^ rj;
                    if (rp > r) {
                        const bool up = (((r << 5) | lane) & k) == 0;
                        const bool first = key[r] > key[rp] || (key[r] == key[rp] && idx[r] < idx[rp]);
                        if (up ? !first : first) {
                            const float tk = key[r]; key[r] = key[rp]; key[rp] = tk;
                            const int ti = idx[r]; idx[r] = idx[rp]; idx[rp] = ti;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float ok = __shfl_xor_sync(0xffffffffu, key[r], j);
                    const int oi = __shfl_xor_sync(0xffffffffu, idx[r], j);
                    const bool lower = (lane & j) == 0;
                    const bool up = (((r << 5) | lane) & k) == 0;
                    const bool mine_first = key[r] > ok || (key[r] == ok && idx[r] < oi);
                    const bool keep = lower ? (up ? mine_first : !mine_first) : (up ? !mine_first : mine_first);
                    if (!keep) { key[r] = ok; idx[r] = oi; }
                }
            }
        }
    }
}

template <int R>
__device__ __forceinline__ void cb_yeti_warp_perm(const CbYetiArgs& a, int perm, long long b, int L, const float* s_ap,
                                                  const float* s_tg, int* s_der, int* s_hes, float qscale, int lane) {
    float key[R];
    int idx[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = r * 32 + lane;
        float k = -3.0e38f;
        if (i < L) {
            float u = a.noise ? a.noise[(long long)perm * a.n + b + i]
                              : cb_uniform01(cb_mix64(a.seed ^ cb_mix64(((unsigned long long)perm << 40) ^ (unsigned long long)(b + i))));
            u = fminf(fmaxf(u, 1e-6f), 1.0f - 1e-6f);
            k = s_ap[i] + __logf(u / (1.000001f - u));
        }
        key[r] = k;
        idx[r] = i;
    }
    cb_yeti_warp_sort<R>(key, idx, lane);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int e = r * 32 + lane;
        const int same = __shfl_down_sync(0xffffffffu, idx[r], 1);
        const int wrap = (r + 1 < R) ? __shfl_sync(0xffffffffu, idx[(r + 1 < R) ? r + 1 : r], 0) : 0;
        const int i2 = lane < 31 ? same : wrap;
        if (e + 1 < L) {
            const int i1 = idx[r];
            const float t1 = s_tg[i1], t2 = s_tg[i2];
            const float wgt = 0.15f * __powf(a.decay, (float)e) * fabsf(t1 - t2);
            if (wgt > 0.0f) {
                const int win = t1 > t2 ? i1 : i2, los = t1 > t2 ? i2 : i1;
                const float p = 1.0f / (1.0f + __expf(s_ap[win] - s_ap[los]));
                const int g = __float2int_rn(wgt * p * qscale), h = __float2int_rn(wgt * p * (1.0f - p) * qscale);
                atomicAdd(&s_der[win], g);
                atomicAdd(&s_der[los], -g);
                atomicAdd(&s_hes[win], h);
                atomicAdd(&s_hes[los], h);
            }
        }
    }
}

__global__ void __launch_bounds__(512) cb_yetirank_warp_kernel(CbYetiArgs a) {
    __shared__ float s_ap[CB_YETI_WARP_GROUP];
    __shared__ float s_tg[CB_YETI_WARP_GROUP];
    __shared__ int s_der[CB_YETI_WARP_GROUP];
    __shared__ int s_hes[CB_YETI_WARP_GROUP];
    __shared__ float s_lo[16], s_hi[16];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int q = blockIdx.x; q < a.Q; q += gridDim.x) {
        const long long b = a.offsets[q], e = a.offsets[q + 1];
        const int L = (int)(e - b);
        if (L > CB_YETI_WARP_GROUP) continue;      // left to the block-wide kernel
        float lo = 3.0e38f, hi = -3.0e38f;
        for (int i = threadIdx.x; i < L; i += blockDim.x) {
            const float t = a.target[b + i];
            s_ap[i] = a.approx[b + i];
            s_tg[i] = t;
            s_der[i] = 0;
            s_hes[i] = 0;
            lo = fminf(lo, t);
            hi = fmaxf(hi, t);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
        __syncthreads();
        for (int w = 0; w < nwarps; ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
        // a document sits in at most two neighbour pairs per permutation, each worth at most 0.15 * (label range)
        const float bound = 0.3f * fmaxf(hi - lo, 1e-30f) * (float)a.permutations;
        const float qscale = 1073741824.0f / bound;
        if (L >= 2) {
            for (int perm = warp; perm < a.permutations; perm += nwarps) {
                if (L <= 64) cb_yeti_warp_perm<2>(a, perm, b, L, s_ap, s_tg, s_der, s_hes, qscale, lane);
                else if (L <= 128) cb_yeti_warp_perm<4>(a, perm, b, L, s_ap, s_tg, s_der, s_hes, qscale, lane);
                else cb_yeti_warp_perm<8>(a, perm, b, L, s_ap, s_tg, s_der, s_hes, qscale, lane);
            }
        }
        __syncthreads();
        const float inv = 1.0f / ((float)a.permutations * qscale);
        for (int i = threadIdx.x; i < L; i += blockDim.x) {
            const float w = a.weight ? a.weight[b + i] : 1.0f;
            a.der[b + i] = (float)s_der[i] * inv * w;
            a.hess[b + i] = fmaxf((float)s_hes[i] * inv * w, 1e-16f);
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
    CbYetiArgs a{approx, target, weight, offsets, Q, permutations, decay, seed, noise, n, der, hess, 0};
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    bool warp_kernel = true;
    if (const char* e = getenv("CB200_YETI_WARP")) warp_kernel = atoi(e) != 0;
    if (warp_kernel) {
        // one warp per permutation for the groups of up to 256 documents; the block-wide kernel takes the longer ones
        int nw = permutations < 1 ? 1 : (permutations > 16 ? 16 : permutations);
        int occ = 1;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cb_yetirank_warp_kernel, nw * 32, 0) != cudaSuccess || occ < 1) {
            cudaGetLastError();
            occ = 1;
        }
        int grid = sms * occ;                      // exactly the resident blocks: a second wave would double the time
        if (grid > Q) grid = Q;
        cb_yetirank_warp_kernel<<<grid, nw * 32, 0, st>>>(a);
        if (max_group > CB_YETI_WARP_GROUP) {
            a.min_group = CB_YETI_WARP_GROUP;
            int grid2 = sms * 4;
            if (grid2 > Q) grid2 = Q;
            cb_yetirank_kernel<CB_YETI_MAX_GROUP, CB_YETI_THREADS><<<grid2, CB_YETI_THREADS, 0, st>>>(a);
        }
    } else if (max_group <= 256) {
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
