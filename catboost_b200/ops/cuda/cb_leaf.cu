// Leaf values of one oblivious tree in ONE cooperative launch: all Newton / gradient steps of the leaf estimation
// (catboost/cuda/methods/leaves_estimation/*, catboost/private/libs/algo/approx_calcer.cpp) run back to back inside
// the kernel, separated by grid barriers, instead of one launch per step.
//
// A step: every block streams its documents (approx, target, leaf -- the same ones in every step, so from the second
// step on they mostly come out of L2), evaluates the objective's derivatives at approx + delta[leaf], accumulates
// per-leaf sums in lane-replicated shared-memory cells, adds them into the global double accumulators; after a grid
// barrier block 0 all-reduces the sums over the ranks through the peer mailboxes, takes the step and publishes the new
// delta; a second grid barrier releases the other blocks into the next step.
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

struct CbLeafNewtonArgs {
    int loss; float p0, p1;
    const float* approx; const float* target; const float* weight; const unsigned short* leaf;
    long long n; int L;
    float* delta;            // [L] running leaf values of this tree (unscaled); written by block 0
    double* sums;            // [3][L][3] zero on entry, zero on exit (one rank rotates through the three copies)
    unsigned int* counter;   // zero on entry / exit
    float* vmax;             // [2] zero on entry, zero on exit
    int steps, newton;
    float l2, lr;
    float* cur_vals;         // [L] lr * delta after the last step
    float* model_vals; float* model_wts; int Lstride; const int* iter_ptr;
    float* leaf_w;           // [L] per-leaf weight sums
    CbComm c;
};

struct CbLeafDocs { float4 a4, t4, w4; ushort4 lf4; };

__device__ __forceinline__ void cb_leaf_docs_load(const CbLeafNewtonArgs& a, long long i0, CbLeafDocs& v) {
    v.lf4 = *reinterpret_cast<const ushort4*>(a.leaf + i0);
    v.a4 = __ldcg(reinterpret_cast<const float4*>(a.approx + i0));
    v.t4 = __ldcg(reinterpret_cast<const float4*>(a.target + i0));
    if (a.weight) v.w4 = __ldcg(reinterpret_cast<const float4*>(a.weight + i0));
}

// C = replicas of every cell (lane l uses replica l & (C-1)), a power of two <= 32.
template <int LOSS>
__global__ void __launch_bounds__(512, 2) cb_leaf_newton_kernel(CbLeafNewtonArgs a, int C) {
    extern __shared__ float sl[];                 // cells: [L][4][C]; then delta copy: [L]
    cg::grid_group grid = cg::this_grid();
    const int loss = LOSS >= 0 ? LOSS : a.loss;
    const int L = a.L;
    const int lane_copy = threadIdx.x & (C - 1);
    int* si = reinterpret_cast<int*>(sl);
    float* sdelta = sl + (size_t)4 * L * C;
    float* sleafw = sdelta + L;
    // One rank: every block takes the Newton step itself from the complete sums, so a step needs a single grid barrier.
    // The sums rotate through three copies; block 0 clears the copy of step s + 2 after the barrier of step s, when
    // nobody can still be reading it and nobody can already be adding to it.
    const bool solo = a.c.nranks <= 1;
    const long long n4 = (a.n + 3) >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const bool can_quant = (a.n / gridDim.x) < (1ll << 22);
    // documents one replica of a cell can receive: those of the threads that share the replica index
    const long long per_thread = ((n4 + stride - 1) / stride) * 4;
    const float qcap = fminf(8388607.0f, floorf(2147483647.0f / (float)(per_thread * (blockDim.x / C) + 1)) - 1.0f);
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
        double* S = a.sums + (solo ? (size_t)(step % 3) * 3 * L : 0);
        for (int i = threadIdx.x; i < 4 * L * C; i += blockDim.x) sl[i] = 0.0f;
        if (!solo || first)
            for (int i = threadIdx.x; i < L; i += blockDim.x) sdelta[i] = first ? 0.0f : __ldcg(a.delta + i);
        __syncthreads();
        float mx0 = 0.f, mx1 = 0.f;
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
        __syncthreads();
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
                float vsum = 0.0f;
                for (int c = 0; c < C; ++c) vsum += sl[(size_t)(l * 4 + s3) * C + c];
                if (vsum != 0.0f) atomicAdd(&S[i], (double)vsum);
            }
        }
        __threadfence();
        grid.sync();
        if (solo) {
            const int it = *a.iter_ptr;
            for (int l = threadIdx.x; l < L; l += blockDim.x) {
                const double sd = __ldcg(&S[3 * l]), shs = __ldcg(&S[3 * l + 1]);
                if (first) sleafw[l] = (float)__ldcg(&S[3 * l + 2]);
                const double sw = (double)sleafw[l];
                const double den = (a.newton ? shs : sw) + (double)a.l2;
                const float stp = (den > 0.0) ? (float)(sd / den) : 0.0f;
                const float v = sdelta[l] + stp;
                sdelta[l] = v;
                if (blockIdx.x == 0) {
                    a.delta[l] = v;
                    if (first) a.leaf_w[l] = sleafw[l];
                    if (last) {
                        a.cur_vals[l] = a.lr * v;
                        if (a.model_vals) a.model_vals[(long long)it * a.Lstride + l] = a.lr * v;
                        if (a.model_wts) a.model_wts[(long long)it * a.Lstride + l] = (float)sw;
                    }
                }
            }
            if (blockIdx.x == 0) {
                double* Z = a.sums + (size_t)((step + 2) % 3) * 3 * L;
                for (int i = threadIdx.x; i < 3 * L; i += blockDim.x) Z[i] = 0.0;
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
                    for (int i = threadIdx.x; i < 9 * L; i += blockDim.x) a.sums[i] = 0.0;
                    if (threadIdx.x == 0) { *a.counter = 0u; a.vmax[0] = 0.0f; a.vmax[1] = 0.0f; }
                }
            }
            continue;
        }
        if (blockIdx.x == 0) {
            if (a.c.nranks > 1) {
                for (int base = 0; base < 3 * L; base += a.c.mbox_bytes / 8)
                    cb_mailbox_allreduce_sum(a.c, a.sums + base, min(3 * L - base, a.c.mbox_bytes / 8));
            }
            const int it = *a.iter_ptr;
            for (int l = threadIdx.x; l < L; l += blockDim.x) {
                const double sd = __ldcg(&a.sums[3 * l]), shs = __ldcg(&a.sums[3 * l + 1]);
                if (first) a.leaf_w[l] = (float)__ldcg(&a.sums[3 * l + 2]);
                const double sw = (double)a.leaf_w[l];
                const double den = (a.newton ? shs : sw) + (double)a.l2;
                const float stp = (den > 0.0) ? (float)(sd / den) : 0.0f;
                const float v = (first ? 0.0f : sdelta[l]) + stp;
                a.delta[l] = v;
                if (last) {
                    a.cur_vals[l] = a.lr * v;
                    if (a.model_vals) a.model_vals[(long long)it * a.Lstride + l] = a.lr * v;
                    if (a.model_wts) a.model_wts[(long long)it * a.Lstride + l] = (float)sw;
                }
                a.sums[3 * l] = 0.0; a.sums[3 * l + 1] = 0.0; a.sums[3 * l + 2] = 0.0;
            }
            if (last && threadIdx.x == 0) { a.vmax[0] = 0.0f; a.vmax[1] = 0.0f; }
            __threadfence();
        }
        if (!last) grid.sync();
    }
}

// Launcher.  `grid` must not exceed the number of co-resident blocks (cb_leaf_newton_max_grid).  Returns a CUDA error
// code (0 = ok), or -2 when the tree has too many leaves for the shared-memory cells (use the per-step kernel).
template <int LOSS>
static int cb_leaf_newton_launch_t(CbLeafNewtonArgs& a, int C, int smem, int grid, cudaStream_t st) {
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_leaf_newton_kernel<LOSS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             100 * 1024);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    void* args[] = {&a, &C};
    return (int)cudaLaunchCooperativeKernel((void*)cb_leaf_newton_kernel<LOSS>, dim3(grid), dim3(512), args,
                                            (size_t)smem, st);
}

static int cb_leaf_newton_cells(int L, int* smem) {
    int C = 32;
    while (C > 1 && (size_t)(4 * L * C + 2 * L) * 4 > 96 * 1024) C >>= 1;
    *smem = (4 * L * C + 2 * L) * 4;
    return (size_t)*smem <= 96 * 1024 ? C : 0;
}

CB_API int cb_leaf_newton_max_grid(int L) {
    int smem = 0;
    const int C = cb_leaf_newton_cells(L, &smem);
    if (C == 0) return 0;
    int dev = 0, sms = 0, occ = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaFuncSetAttribute(cb_leaf_newton_kernel<-1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cb_leaf_newton_kernel<-1>, 512, smem) != cudaSuccess) {
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
                          int grid, cudaStream_t st) {
    CbLeafNewtonArgs a{loss, p0, p1, approx, target, weight, leaf, n, L, delta, sums, counter, vmax, steps, newton, l2, lr,
                       cur_vals, model_vals, model_wts, Lstride, iter_ptr, leaf_w, CbComm()};
    if (comm) a.c = *comm; else { a.c.nranks = 1; a.c.rank = 0; }
    int smem = 0;
    const int C = cb_leaf_newton_cells(L, &smem);
    if (C == 0 || loss == CB_LOSS_EXTERNAL) return -2;
    if (loss == CB_LOSS_LOGLOSS) return cb_leaf_newton_launch_t<CB_LOSS_LOGLOSS>(a, C, smem, grid, st);
    if (loss == CB_LOSS_RMSE) return cb_leaf_newton_launch_t<CB_LOSS_RMSE>(a, C, smem, grid, st);
    return cb_leaf_newton_launch_t<-1>(a, C, smem, grid, st);
}
