// Leaf values of one oblivious tree in ONE cooperative launch: all Newton / gradient steps of the leaf estimation
// (catboost/cuda/methods/leaves_estimation/*, catboost/private/libs/algo/approx_calcer.cpp) run back to back inside
// the kernel, separated by ONE grid barrier per step, instead of one launch (and one host round trip) per step.
//
// A step: every block streams its documents (approx, target, leaf -- the same ones in every step, so from the second
// step on they mostly come out of L2), evaluates the objective at approx + delta[leaf], accumulates per-leaf sums in
// lane-replicated shared-memory cells and adds them into the global double accumulators of the step (three rotating
// copies).  After the grid barrier the sums of this rank are complete.  With several ranks block 0 then sends them to
// every rank as tagged words (cb_comm.cuh) and EVERY block polls the R messages in its own arena and adds them in rank
// order; with one rank every block reads the accumulators directly.  Either way each block takes the Newton step
// itself, in shared memory, with bit-identical arithmetic, so no second barrier and no single-block serial section
// is needed.
//
// Step-length control (leaf_estimation_backtracking, catboost/cuda/methods/leaves_estimation/descent_helpers.cpp:127-206,
// step_estimator.cpp): every pass also sums the loss at the point it evaluates.  A pass whose point does not satisfy
// the condition (AnyImprovement: the loss did not get worse; Armijo: sufficient decrease, C = 1e-5) is not accepted:
// the next pass evaluates base + (step / 2) * direction instead.  As in the reference a rejected try uses up one of
// the leaf_estimation_iterations; unlike the reference the move taken after the last pass is not verified (the
// reference spends an extra pass on that).
//
// Cells: the first step uses fp32 cells (shared fp32 atomics are compare-and-swap loops, but the scale of the values
// is not known yet) and records max |w der|, max |w hess|; later steps use fixed point with native integer atomics:
// one int32 cell per (leaf, statistic, replica), scaled so that twice the recorded bound times the number of documents
// a replica can receive stays below 2^31 (about 21 bits per value with 32 replicas at 10M documents -- finer than what
// an fp32 running sum keeps).  A value beyond the bound goes to the double accumulator directly.
#include "cb_common.cuh"
#include "cb_losses.cuh"
#include "cb_comm.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

enum CbBacktrack : int { CB_BT_NONE = 0, CB_BT_ANY_IMPROVEMENT = 1, CB_BT_ARMIJO = 2 };

struct CbLeafNewtonArgs {
    int loss; float p0, p1;
    const float* approx; const float* target; const float* weight; const unsigned short* leaf;
    long long n; int L;
    float* delta;            // [L] running leaf values of this tree (unscaled); written by block 0
    double* sums;            // [3][3L + 4] zero on entry, zero on exit: per leaf (der, hess, weight), then the loss sum
    unsigned int* counter;   // zero on entry / exit
    float* vmax;             // [2] zero on entry, zero on exit
    int steps, newton;
    float l2, lr;
    float* cur_vals;         // [L] lr * delta after the last step
    float* model_vals; float* model_wts; int Lstride; const int* iter_ptr;
    float* leaf_w;           // [L] per-leaf weight sums
    int backtrack;           // CbBacktrack
    CbComm c;
};

struct CbLeafDocs { float4 a4, t4, w4; ushort4 lf4; };

__device__ __forceinline__ void cb_leaf_docs_load(const CbLeafNewtonArgs& a, long long i0, CbLeafDocs& v) {
    v.lf4 = *reinterpret_cast<const ushort4*>(a.leaf + i0);
    v.a4 = __ldcg(reinterpret_cast<const float4*>(a.approx + i0));
    v.t4 = __ldcg(reinterpret_cast<const float4*>(a.target + i0));
    if (a.weight) v.w4 = __ldcg(reinterpret_cast<const float4*>(a.weight + i0));
}

__device__ __forceinline__ double cb_ll_load_double(const unsigned long long* box, int i, unsigned int tag,
                                                    const CbComm& c, int src) {
    const unsigned int lo = cb_ll_load(box + 2 * i, tag, c.timeout_ns, c.status, CB_TIMEOUT_MAILBOX, src);
    const unsigned int hi = cb_ll_load(box + 2 * i + 1, tag, c.timeout_ns, c.status, CB_TIMEOUT_MAILBOX, src);
    return __longlong_as_double((long long)(((unsigned long long)hi << 32) | lo));
}

// C = replicas of every cell (lane l uses replica l & (C-1)), a power of two <= 32.  BT = step-length control compiled in.
template <int LOSS, bool BT>
__global__ void __launch_bounds__(512, 2) cb_leaf_newton_kernel(CbLeafNewtonArgs a, int C) {
    extern __shared__ float sl[];                 // cells: [L][4][C]; then delta, leaf weights, base point, direction: [L] each
    cg::grid_group grid = cg::this_grid();
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    const int L = a.L;
    const int lane_copy = threadIdx.x & (C - 1);
    int* si = reinterpret_cast<int*>(sl);
    float* sdelta = sl + (size_t)4 * L * C;
    float* sleafw = sdelta + L;
    float* sbase = sleafw + L;
    float* sdir = sbase + L;
    __shared__ double s_red[16];
    __shared__ double s_value;
    const int R = a.c.nranks, me = a.c.rank;
    const bool solo = R <= 1;
    const unsigned long long epoch0 = solo ? 0ull : *a.c.epoch;      // every block reads it before the first barrier
    const int SS = 3 * L + 4;                                        // doubles per copy of the accumulators
    const long long n4 = (a.n + 3) >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const bool can_quant = (a.n / gridDim.x) < (1ll << 22);
    // documents one replica of a cell can receive: those of the threads that share the replica index
    const long long per_thread = ((n4 + stride - 1) / stride) * 4;
    const float qcap = fminf(8388607.0f, floorf(2147483647.0f / (float)(per_thread * (blockDim.x / C) + 1)) - 1.0f);
    double f_base = 0.0, dirgrad = 0.0;           // loss and gradient . direction at the last accepted point
    float cur_step = 1.0f;
    for (int step = 0; step < a.steps; ++step) {
        const bool first = step == 0, last = step == a.steps - 1;
        const bool quant = !first && can_quant;
        float M0 = 0.f, M1 = 0.f, sc0 = 0.f, sc1 = 0.f;
        if (quant) {
            M0 = 2.0f * fmaxf(__ldcg(a.vmax), 1e-30f);
            M1 = 2.0f * fmaxf(__ldcg(a.vmax + 1), 1e-30f);
            sc0 = qcap / M0;
            sc1 = qcap / M1;
        }
        double* S = a.sums + (size_t)(step % 3) * SS;
        for (int i = threadIdx.x; i < 4 * L * C; i += blockDim.x) sl[i] = 0.0f;
        if (first)
            for (int i = threadIdx.x; i < L; i += blockDim.x) { sdelta[i] = 0.0f; sbase[i] = 0.0f; sdir[i] = 0.0f; }
        __syncthreads();
        float mx0 = 0.f, mx1 = 0.f, vsum = 0.f;
        long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
        CbLeafDocs nx;
        nx.a4 = nx.t4 = make_float4(0.f, 0.f, 0.f, 0.f);
        nx.w4 = make_float4(1.f, 1.f, 1.f, 1.f);
        nx.lf4 = make_ushort4(0, 0, 0, 0);
        if (q < n4) cb_leaf_docs_load(a, q << 2, nx);
        for (; q < n4; q += stride) {
            const long long i0 = q << 2;
            const CbLeafDocs v = nx;
            if (q + stride < n4) cb_leaf_docs_load(a, (q + stride) << 2, nx);
            const unsigned int lf[4] = {v.lf4.x, v.lf4.y, v.lf4.z, v.lf4.w};
            const float ap[4] = {v.a4.x, v.a4.y, v.a4.z, v.a4.w}, tg[4] = {v.t4.x, v.t4.y, v.t4.z, v.t4.w};
            const float wt[4] = {v.w4.x, v.w4.y, v.w4.z, v.w4.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (i0 + k >= a.n) break;
                const int l = (int)lf[k];
                const CbLossOut o = cb_loss_eval(loss, a.p0, a.p1, ap[k] + sdelta[l], tg[k]);
                const float w = wt[k];
                const float vd = w * o.der, vh = w * o.hess;
                if (BT) vsum += w * o.value;
                if (quant) {
                    if (fmaxf(fabsf(vd) * sc0, fabsf(vh) * sc1) <= qcap) {
                        int* cell = si + (size_t)(l * 4) * C + lane_copy;
                        atomicAdd(cell, __float2int_rn(vd * sc0));
                        atomicAdd(cell + C, __float2int_rn(vh * sc1));
                    } else {
                        atomicAdd(&S[3 * l], (double)vd);
                        atomicAdd(&S[3 * l + 1], (double)vh);
                    }
                } else {
                    float* cell = sl + (size_t)(l * 4) * C + lane_copy;
                    atomicAdd(cell, vd);
                    atomicAdd(cell + C, vh);
                    if (first) {
                        atomicAdd(cell + 2 * C, w);
                        mx0 = fmaxf(mx0, fabsf(vd));
                        mx1 = fmaxf(mx1, fabsf(vh));
                    }
                }
            }
        }
        if (first) {
            for (int off = 16; off > 0; off >>= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            if ((threadIdx.x & 31) == 0) {         // non-negative floats order like their bit patterns
                atomicMax(reinterpret_cast<int*>(a.vmax), __float_as_int(mx0));
                atomicMax(reinterpret_cast<int*>(a.vmax) + 1, __float_as_int(mx1));
            }
        }
        if (BT) {
            double dv = cb_warp_sum_d((double)vsum);
            if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = dv;
        }
        __syncthreads();
        if (BT && threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w];
            if (t != 0.0) atomicAdd(&S[3 * L], t);
        }
        if (quant) {
            const double inv0 = (double)M0 / (double)qcap, inv1 = (double)M1 / (double)qcap;
            for (int i = threadIdx.x; i < 2 * L; i += blockDim.x) {
                const int l = i >> 1, s2 = i & 1;
                const int* ph = si + (size_t)(l * 4 + s2) * C;
                long long qq = 0;
                for (int c = 0; c < C; ++c) qq += ph[c];
                if (qq != 0) atomicAdd(&S[3 * l + s2], (double)qq * (s2 ? inv1 : inv0));
            }
        } else {
            for (int i = threadIdx.x; i < 3 * L; i += blockDim.x) {
                const int l = i / 3, s3 = i - 3 * l;
                if (s3 == 2 && !first) continue;
                float vs = 0.0f;
                for (int c = 0; c < C; ++c) vs += sl[(size_t)(l * 4 + s3) * C + c];
                if (vs != 0.0f) atomicAdd(&S[i], (double)vs);
            }
        }
        __threadfence();
        grid.sync();
        // ---- the sums of this rank are complete -------------------------------------------------------------
        const unsigned long long epoch = epoch0 + (unsigned long long)step + 1ull;
        const unsigned int tag = cb_ll_tag(epoch);
        const int parity = (int)(epoch & 1ull);
        if (!solo && blockIdx.x == 0) {
            // one tagged copy of (der, hess[, weight]) per leaf and of the loss sum to every rank, this one included
            const int cnt = 3 * L + 1;
            for (int idx = threadIdx.x; idx < cnt * R; idx += blockDim.x) {
                const int r = idx / cnt, i = idx - r * cnt;
                if (i < 3 * L && (i % 3) == 2 && !first) continue;
                const unsigned long long bits = (unsigned long long)__double_as_longlong(__ldcg(&S[i]));
                unsigned long long* box = cb_ll_box(a.c, r, parity, me);
                cb_ll_store(box + 2 * i, (unsigned int)bits, tag);
                cb_ll_store(box + 2 * i + 1, (unsigned int)(bits >> 32), tag);
            }
        }
        if (threadIdx.x == 0) {
            double v = 0.0;
            if (BT) {
                if (solo) v = __ldcg(&S[3 * L]);
                else for (int r = 0; r < R; ++r) v += cb_ll_load_double(cb_ll_box(a.c, me, parity, r), 3 * L, tag, a.c, r);
            }
            s_value = v;
        }
        __syncthreads();
        bool accept = true;
        if (BT && !first) {
            const double v = s_value;
            accept = (a.backtrack == CB_BT_ARMIJO) ? (v <= f_base - 1e-5 * (double)cur_step * dirgrad) : (v <= f_base);
            if (!(v == v)) accept = false;
        }
        const int it = *a.iter_ptr;
        double dg = 0.0;
        for (int l = threadIdx.x; l < L; l += blockDim.x) {
            float nd;
            if (accept) {
                double sd = 0.0, shs = 0.0, sw = 0.0;
                if (solo) {
                    sd = __ldcg(&S[3 * l]); shs = __ldcg(&S[3 * l + 1]);
                    if (first) sw = __ldcg(&S[3 * l + 2]);
                } else {
                    for (int r = 0; r < R; ++r) {
                        const unsigned long long* box = cb_ll_box(a.c, me, parity, r);
                        sd += cb_ll_load_double(box, 3 * l, tag, a.c, r);
                        shs += cb_ll_load_double(box, 3 * l + 1, tag, a.c, r);
                        if (first) sw += cb_ll_load_double(box, 3 * l + 2, tag, a.c, r);
                    }
                }
                if (first) sleafw[l] = (float)sw;
                const double den = (a.newton ? shs : (double)sleafw[l]) + (double)a.l2;
                const float dir = (den > 0.0) ? (float)(sd / den) : 0.0f;
                if (BT) { sbase[l] = sdelta[l]; sdir[l] = dir; dg += sd * (double)dir; }
                nd = sdelta[l] + dir;
            } else {
                nd = sbase[l] + 0.5f * cur_step * sdir[l];
            }
            sdelta[l] = nd;
            if (blockIdx.x == 0) {
                a.delta[l] = nd;
                if (first) a.leaf_w[l] = sleafw[l];
                if (last) {
                    a.cur_vals[l] = a.lr * nd;
                    if (a.model_vals) a.model_vals[(long long)it * a.Lstride + l] = a.lr * nd;
                    if (a.model_wts) a.model_wts[(long long)it * a.Lstride + l] = sleafw[l];
                }
            }
        }
        if (BT) {
            if (accept) {
                // gradient . direction at the new base point, added up in a fixed order (every block gets the same bits)
                dg = cb_warp_sum_d(dg);
                __syncthreads();
                if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = dg;
                __syncthreads();
                double t = 0.0;
                for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_red[w];
                dirgrad = t;
                f_base = s_value;
                cur_step = 1.0f;
            } else {
                cur_step *= 0.5f;
            }
        }
        if (blockIdx.x == 0) {
            double* Z = a.sums + (size_t)((step + 2) % 3) * SS;
            for (int i = threadIdx.x; i < SS; i += blockDim.x) Z[i] = 0.0;
            __threadfence();
        }
        __syncthreads();
        if (last) {
            // the block that finishes last clears what the final steps left behind
            __shared__ bool s_last_block;
            __threadfence();
            if (threadIdx.x == 0) s_last_block = (atomicAdd(a.counter, 1u) == gridDim.x - 1);
            __syncthreads();
            if (s_last_block) {
                for (int i = threadIdx.x; i < 3 * SS; i += blockDim.x) a.sums[i] = 0.0;
                if (threadIdx.x == 0) {
                    *a.counter = 0u; a.vmax[0] = 0.0f; a.vmax[1] = 0.0f;
                    if (!solo) *a.c.epoch = epoch0 + (unsigned long long)a.steps;
                }
            }
        }
    }
}

// Launcher.  `grid` must not exceed the number of co-resident blocks (cb_leaf_newton_max_grid).  Returns a CUDA error
// code (0 = ok), or -2 when the tree has too many leaves for the shared-memory cells or for one mailbox message (use
// the per-step kernel).
template <int LOSS, bool BT>
static int cb_leaf_newton_launch_t(CbLeafNewtonArgs& a, int C, int smem, int grid, cudaStream_t st) {
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_leaf_newton_kernel<LOSS, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             100 * 1024);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    void* args[] = {&a, &C};
    return (int)cudaLaunchCooperativeKernel((void*)cb_leaf_newton_kernel<LOSS, BT>, dim3(grid), dim3(512), args,
                                            (size_t)smem, st);
}

static int cb_leaf_newton_cells(int L, int* smem) {
    int C = 32;
    while (C > 1 && (size_t)(4 * L * C + 4 * L) * 4 > 96 * 1024) C >>= 1;
    *smem = (4 * L * C + 4 * L) * 4;
    return (size_t)*smem <= 96 * 1024 ? C : 0;
}

// Doubles the caller must provide (zeroed) as `sums`: three rotating copies of (3 per leaf + the loss sum, padded).
CB_API int cb_leaf_newton_sums_doubles(int L) { return 3 * (3 * L + 4); }
// Bytes one mailbox message of this kernel takes (tagged words): the arena's mailbox slots must be at least this big.
CB_API int cb_leaf_newton_msg_bytes(int L) { return (3 * L + 1) * 16; }

CB_API int cb_leaf_newton_max_grid(int L) {
    int smem = 0;
    const int C = cb_leaf_newton_cells(L, &smem);
    if (C == 0) return 0;
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(cb_leaf_newton_kernel<-1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cb_leaf_newton_kernel<-1, true>, 512, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (occ > 2) occ = 2;
    return occ * sms;
}

CB_API int cb_leaf_newton(int loss, float p0, float p1, const float* approx, const float* target, const float* weight,
                          const unsigned short* leaf, long long n, int L, float* delta, double* sums,
                          unsigned int* counter, float* vmax,
                          int steps, int newton, float l2, float lr, float* cur_vals, float* model_vals,
                          float* model_wts, int Lstride, const int* iter_ptr, float* leaf_w, const CbComm* comm,
                          int backtrack, int grid, cudaStream_t st) {
    CbLeafNewtonArgs a{loss, p0, p1, approx, target, weight, leaf, n, L, delta, sums, counter, vmax, steps, newton, l2, lr,
                       cur_vals, model_vals, model_wts, Lstride, iter_ptr, leaf_w, backtrack, CbComm()};
    if (comm) a.c = *comm; else { a.c.nranks = 1; a.c.rank = 0; }
    int smem = 0;
    const int C = cb_leaf_newton_cells(L, &smem);
    if (C == 0 || loss == CB_LOSS_EXTERNAL) return -2;
    if (a.c.nranks > 1 && cb_leaf_newton_msg_bytes(L) > a.c.mbox_bytes) return -2;
    const bool bt = backtrack != CB_BT_NONE && steps > 1;
    if (loss == CB_LOSS_LOGLOSS)
        return bt ? cb_leaf_newton_launch_t<CB_LOSS_LOGLOSS, true>(a, C, smem, grid, st)
                  : cb_leaf_newton_launch_t<CB_LOSS_LOGLOSS, false>(a, C, smem, grid, st);
    if (loss == CB_LOSS_RMSE)
        return bt ? cb_leaf_newton_launch_t<CB_LOSS_RMSE, true>(a, C, smem, grid, st)
                  : cb_leaf_newton_launch_t<CB_LOSS_RMSE, false>(a, C, smem, grid, st);
    return bt ? cb_leaf_newton_launch_t<-1, true>(a, C, smem, grid, st) : cb_leaf_newton_launch_t<-1, false>(a, C, smem, grid, st);
}
