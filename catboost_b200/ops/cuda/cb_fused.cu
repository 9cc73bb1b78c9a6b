// K6 fused level kernel: ONE cooperative launch per tree level does
//   (0) the leaf-index update for the split chosen at the previous level (inside the histogram pass when the
//       bundled path runs: the pass has the bin words of its documents in registers anyway),
//   (A) streaming histogram accumulation of the local rows (shared-memory integer atomics, one slot per parent
//       leaf: only the lighter child is accumulated, the sibling is parent - child),
//   (B) the reduce-scatter: every rank sums its chunk tiles and stores the feature slice that rank r owns straight
//       into rank r's slot buffer over NVLink as tagged 8-byte words (value + level tag),
//   (C) on the owner: the score phase polls the words it needs until they carry this level's tag (bounded), sums the
//       per-source slots in rank order (deterministic), sibling subtraction, bin prefix scan, split scoring, packed
//       64-bit atomicMax argmax -- no fence, flag or grid barrier stands between (B) and (C),
//   (D) an exchange of the per-rank best (key + lighter-child mask) as tagged words through the peer mailboxes and
//       the final argmax, which every rank evaluates identically.
// No NCCL call, no host round trip and no separate scoring kernel per level.  This replaces the reference's
// four-step path: histogram kernel -> GatherHistogramsByLeaves -> host-orchestrated ReduceScatter built from
// cudaMemcpyAsync + add kernel -> FindOptimalSplit -> device-to-host read + host argmin
// (catboost/cuda/methods/histograms_helper.cpp:58-91, cuda_lib/cuda_buffer_helpers/reduce_scatter.h:449-540,
// catboost/cuda/methods/histograms_helper.h:322-331).
//
// Only plain peer stores / loads touch remote memory: no bulk-copy engine, no switch-side reduction.
#include "cb_common.cuh"
#include <cstdlib>
#include "cb_tree.cuh"
#include "cb_comm.cuh"
#include <cooperative_groups.h>
#include <new>
#include <vector>
#include <algorithm>

namespace cg = cooperative_groups;

struct CbFusedArgs {
    CbHistArgs h;            // h.priv = per-block private tiles; h.out is unused by the fused kernel
    CbScoreArgs s;           // s.hsrc[r] = local slot r; s.W = owned width; s.col_base = first owned column
    CbComm c;
    unsigned short* leaf;
    CbSplit* splits; int depth;
    unsigned int* mask_out;          // lighter-child mask for the next level
    unsigned long long* msg_local;   // CB_SELECT_MSG_BYTES scratch in local memory
    unsigned long long* msg_stage;   // [nranks][msg_stage_stride] words: the peers' messages, unpacked from the mailbox
    int msg_stage_stride;
    int fuse_leaf;                   // 1: the histogram pass of this launch also applies the previous level's split
    int own_col[CB_MAX_RANKS + 1];   // rank r owns histogram columns [own_col[r], own_col[r+1]) (multiples of 4)
    int Wmax;                        // row stride (floats) of every slot buffer = max owned width
    int smem_floats;                 // dynamic shared memory of this launch, in floats
    unsigned long long* phase_ts;    // optional globaltimer stamps (phase profiling): [depth][8] by block 0,
                                     // then [4096][2] per-block histogram end + SM id, then [depth][4] inside the score phase
};

// Sum of the per-chunk private tiles of this rank, written to the owner's slot.  A unit of work is one 16-byte column
// group of one (slot, statistic) row.  At the shallow levels there are few units and many chunks (a bundle of all
// groups is cut into as many chunks as there are blocks), so the chunks of a unit are dealt to KS lanes of a warp
// (KS a power of two <= 32, as many as the grid has spare threads for) and combined with shuffles.
static __device__ void cb_reduce_chunks(const CbFusedArgs& a, int cta, int ncta, unsigned int ll_tag) {
    const CbHistArgs& h = a.h;
    const int G = h.d.G, S = h.S, B = h.B, TB = h.d.TB;
    const int nK = cb_hist_chunks(G, ncta, h.d.n, h.nK);
    const int nslots = cb_hist_nslots(h);
    const size_t slot_stride = (size_t)S * 4 * B;
    const size_t item_stride = (size_t)nslots * slot_stride;
    const int rows = nslots * S;
    const int C4 = TB >> 2;
    const int R = a.c.nranks, me = a.c.rank;
    const long long total = (long long)rows * C4;
    const long long gthreads = (long long)ncta * blockDim.x;
    int KS = 1;
    while (KS < 32 && total * (KS * 2) <= gthreads && KS * 2 <= nK) KS <<= 1;
    const int CW = 32 / KS;                      // units per warp
    const int lane = threadIdx.x & 31;
    const int cl = lane & (CW - 1), ks = lane / CW;
    const long long gwarp = ((long long)cta * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = gthreads >> 5;
    for (long long base = gwarp * CW; base < total; base += nwarps * CW) {
        const long long u = base + cl;
        const bool valid = u < total;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int row = 0, col = 0;
        if (valid) {
            row = (int)(u / C4);
            col = (int)(u % C4) << 2;
            const int f = cb_find_feature(h.d.feat_off, h.d.F, col);
            const int bin = col - h.d.feat_off[f];
            const int slot = row / S, st = row - slot * S;
            const float* src = h.priv + ((size_t)slot * S + st) * 4 * B + (size_t)(f & 3) * B + bin
                               + (size_t)(f >> 2) * item_stride;
            const size_t kstride = (size_t)G * item_stride;
            const int nKg = h.gchunks ? h.gchunks[f >> 2] : nK;       // chunks of this group's bundle
#pragma unroll 4
            for (int k = ks; k < nKg; k += KS) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)k * kstride));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        for (int off = CW; off < 32; off <<= 1) {
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
        }
        if (valid && ks == 0) {
            if (R > 1) {
                // tagged words: {value, level tag} pairs, two per 16-byte store (each 8-byte half is atomic on its own)
                int r = 0;
                while (r + 1 < R && col >= a.own_col[r + 1]) ++r;
                unsigned long long* dst = reinterpret_cast<unsigned long long*>(a.c.peer_slot[r] + (size_t)me * a.c.slot_floats)
                                          + (size_t)row * a.Wmax + (col - a.own_col[r]);
                const unsigned long long t = (unsigned long long)ll_tag << 32;
                const unsigned long long w0 = t | __float_as_uint(acc.x), w1 = t | __float_as_uint(acc.y);
                const unsigned long long w2 = t | __float_as_uint(acc.z), w3 = t | __float_as_uint(acc.w);
                asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(w0), "l"(w1) : "memory");
                asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(w2), "l"(w3) : "memory");
            } else {
                float* dst = const_cast<float*>(a.s.hsrc[0]) + (size_t)row * a.Wmax + col;
                *reinterpret_cast<float4*>(dst) = acc;
            }
        }
    }
}

__global__ void __launch_bounds__(1024, 1) cb_level_fused_kernel(CbFusedArgs a) {
    extern __shared__ __align__(16) float cb_sh[];
    cg::grid_group grid = cg::this_grid();
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int level = a.h.level;
    const int it = *a.s.iter_ptr;
    CbSplit* sp_arr = a.splits + (long long)it * a.depth;
    unsigned long long* ts = (a.phase_ts && cta == 0 && threadIdx.x == 0) ? a.phase_ts + level * 8 : nullptr;
    if (ts) ts[0] = cb_globaltimer();
    const int R = a.c.nranks, me = a.c.rank;
    // every block reads the level counter before the first grid barrier; block 0 advances it at the very end
    const unsigned long long hist_epoch = (R > 1) ? a.c.epoch[1] + 1 : 0ull;
    const unsigned int ll_tag = (R > 1) ? cb_ll_tag(hist_epoch) : 0u;

    // (0) leaf update with the split of the previous level: its own pass, unless the histogram pass does it
    if (level > 0 && !a.fuse_leaf) {
        cb_update_leaf_range(a.h.d, a.leaf, sp_arr[level - 1], level - 1,
                             (long long)cta * blockDim.x + threadIdx.x, (long long)ncta * blockDim.x);
        __threadfence();
        grid.sync();
    }

    // the score noise scale only depends on the iteration: one thread per block works it out now, off the critical path
    __shared__ float s_noise_std;
    if (threadIdx.x == 0) s_noise_std = cb_noise_std(a.s);
    if (ts) ts[1] = cb_globaltimer();
    // (A) local histograms: every block dumps its shared-memory tile into its private region (no atomics)
    cb_hist_phase(a.h, cb_sh, cta, ncta);
    if (ts) ts[2] = cb_globaltimer();
    if (a.phase_ts && threadIdx.x == 0 && level == a.depth - 2) {
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        a.phase_ts[a.depth * 8 + cta * 2] = cb_globaltimer();
        a.phase_ts[a.depth * 8 + cta * 2 + 1] = smid;
    }
    __threadfence();
    grid.sync();
    if (ts) ts[3] = cb_globaltimer();

    // (B) chunk reduction fused with the reduce-scatter: each 16-byte column group is summed over the chunks of
    // this rank and stored straight into the slot of the rank that owns the column (peer store over NVLink when
    // that is another GPU; every source keeps its own slot, so the owner later adds them in rank order).
    cb_reduce_chunks(a, cta, ncta, ll_tag);
    if (R <= 1) {
        __threadfence();
        grid.sync();
    }
    // several ranks: (C) needs no barrier here, the words announce themselves and the score phase polls exactly those
    // it reads (a.s.ll_epoch is set by the host)

    if (ts) ts[4] = cb_globaltimer();
    cb_score_phase(a.s, cta, ncta, cb_sh, a.smem_floats, ts ? a.phase_ts + a.depth * 8 + 8192 + level * 4 : nullptr,
                   s_noise_std);
    __threadfence();
    grid.sync();
    if (ts) ts[5] = cb_globaltimer();

    // (D) selection: one block
    if (cta == 0) {
        cb_select_local(a.s, a.msg_local);
        __threadfence();
        __syncthreads();
        const unsigned long long* msgs[CB_MAX_RANKS];
        if (R > 1) {
            // key (two words) + mask words, each as a tagged word into every rank's mailbox; then unpack the R messages
            // that arrived here into the staging rows
            __shared__ unsigned long long s_epoch;
            if (threadIdx.x == 0) { s_epoch = a.c.epoch[0] + 1; a.c.epoch[0] = s_epoch; }
            __syncthreads();
            const unsigned long long epoch = s_epoch;
            const unsigned int tag = cb_ll_tag(epoch);
            const int parity = (int)(epoch & 1ull);
            const int nw = 2 + (((1 << level) + 31) >> 5);
            const unsigned int* src = reinterpret_cast<const unsigned int*>(a.msg_local);
            for (int idx = threadIdx.x; idx < nw * R; idx += blockDim.x) {
                const int r = idx / nw, i = idx - r * nw;
                cb_ll_store(cb_ll_box(a.c, r, parity, me) + i, src[i], tag);
            }
            for (int idx = threadIdx.x; idx < nw * R; idx += blockDim.x) {
                const int r = idx / nw, i = idx - r * nw;
                reinterpret_cast<unsigned int*>(a.msg_stage + (size_t)r * a.msg_stage_stride)[i] =
                    cb_ll_load(cb_ll_box(a.c, me, parity, r) + i, tag, a.c.timeout_ns, a.c.status, CB_TIMEOUT_MAILBOX, r);
            }
            __threadfence();
            __syncthreads();
            for (int r = 0; r < R; ++r) msgs[r] = a.msg_stage + (size_t)r * a.msg_stage_stride;
        } else {
            msgs[0] = a.msg_local;
        }
        cb_select_final(a.h.d, msgs, R, level, sp_arr + level, a.mask_out);
        if (threadIdx.x == 0) {
            *a.s.best_key = 0ull;
            if (R > 1) a.c.epoch[1] = hist_epoch;
            if (ts) ts[6] = cb_globaltimer();
        }
        if (a.h.work) {
            for (int i = threadIdx.x; i <= a.h.d.G; i += blockDim.x) a.h.work[i] = 0u;
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------
#define CB_MAX_LEVELS 16
struct CbFusedPlan {
    CbFusedArgs a;
    int threads;
    int max_smem;      // dynamic shared memory one block may use
    int sm_smem;       // shared memory of one SM available to two resident blocks (after their static + reserved parts)
    int sm_count;
    int max_bundle;    // widest feature-group bundle of the single-cell histogram path (0 = off)
    int fuse_leaf_update;   // 1: let the bundled histogram pass apply the previous level's split (default)
    int max_copies;    // most replicas of a histogram cell (2 for dense columns; more when one bin dominates a column,
                       // where most lanes of a warp would otherwise add to the same cell)
    std::vector<int> group_bins;     // padded bins of the widest feature of every group (empty: all groups take B)
    // per level: bundle table and work list of the bundled path, on the device (made by cb_fused_geometry)
    CbBundle* d_btab[CB_MAX_LEVELS];
    int2* d_items[CB_MAX_LEVELS];
    int* d_gchunks[CB_MAX_LEVELS];     // document chunks of every feature group (those of its bundle)
    int n_btab[CB_MAX_LEVELS], n_items[CB_MAX_LEVELS];
    int single_pass_bundle[CB_MAX_LEVELS];     // 1: one bundle holds every group in one pass (leaf update can be fused)
};


CB_API CbFusedPlan* cb_fused_create(const CbData* d, const CbComm* comm, unsigned short* leaf, const float* stats, int S,
                                    int B, float* partial, float* const* local_slots, float* hbuf0, float* hbuf1,
                                    const int* own_col, int Wmax, unsigned int* mask0, unsigned int* mask1,
                                    CbSplit* splits, int depth, float l2, int score_fn, float random_strength,
                                    const double* scal, const int* iter_ptr, unsigned long long seed, float lr,
                                    unsigned long long* best_key, unsigned long long* msg_local,
                                    unsigned long long* msg_stage, int msg_stage_stride, int threads) {
    CbFusedPlan* p = new (std::nothrow) CbFusedPlan();
    if (!p) return nullptr;
    CbFusedArgs& a = p->a;
    a.h.d = *d; a.h.leaf = leaf; a.h.stats = stats; a.h.S = S; a.h.B = B; a.h.out = nullptr; a.h.priv = partial; a.h.statmax = nullptr; a.phase_ts = nullptr; a.h.nK = 0; a.h.copies = 1; a.h.work = nullptr; a.h.narrow = 0; a.h.bundle = 0;
    a.h.slot_table = nullptr; a.h.nslots_table = 0; a.h.level = 0; a.h.small_mask = mask0; a.h.slots_per_pass = 1;
    a.s.d = *d;
    if (comm) a.c = *comm; else { a.c = CbComm(); a.c.nranks = 1; a.c.rank = 0; }
    const int R = a.c.nranks;
    for (int r = 0; r < CB_MAX_RANKS; ++r) a.s.hsrc[r] = r < R ? local_slots[r] : nullptr;
    a.s.nsrc = R;
    a.s.hprev = hbuf0; a.s.hcur = hbuf1;   // swapped per level at launch
    for (int r = 0; r <= CB_MAX_RANKS; ++r) a.own_col[r] = r <= R ? own_col[r] : own_col[R];
    a.Wmax = Wmax;
    a.s.W = Wmax;
    a.s.col_base = own_col[a.c.rank];
    // owned feature range from the owned columns
    int fb = 0, fe = 0;
    // feat_off is device memory; the caller passes feature ranges through own_col only, so the
    // feature range is resolved by cb_fused_set_features().
    a.s.f_begin = fb; a.s.f_end = fe;
    a.s.level = 0; a.s.S = S; a.s.small_mask = mask0; a.s.l2 = l2; a.s.score_fn = score_fn;
    a.s.random_strength = random_strength; a.s.scal = scal; a.s.iter_ptr = iter_ptr; a.s.seed = seed;
    a.s.learning_rate = lr; a.s.best_key = best_key;
    a.leaf = leaf; a.splits = splits; a.depth = depth; a.mask_out = mask1; a.msg_local = msg_local;
    a.msg_stage = msg_stage; a.msg_stage_stride = msg_stage_stride; a.fuse_leaf = 0;
    a.h.domw = nullptr; a.h.btab = nullptr; a.h.bitems = nullptr; a.h.nbitems = 0; a.h.gchunks = nullptr;
    a.h.prev_splits = nullptr; a.h.prev_iter = iter_ptr; a.h.prev_depth = depth; a.h.leaf_rw = leaf;
    a.s.ll_epoch = R > 1 ? a.c.epoch + 1 : nullptr; a.s.ll_timeout_ns = a.c.timeout_ns; a.s.ll_status = a.c.status;
    p->threads = threads;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&p->max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    // dynamic shared memory available to this kernel = opt-in maximum minus its static shared memory
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, cb_level_fused_kernel) != cudaSuccess) { cudaGetLastError(); delete p; return nullptr; }
    p->max_smem -= (int)fa.sharedSizeBytes;
    cudaDeviceGetAttribute(&p->sm_smem, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    p->sm_smem -= 2 * (int)fa.sharedSizeBytes;
    p->max_bundle = 0;
    for (int l = 0; l < CB_MAX_LEVELS; ++l) { p->d_btab[l] = nullptr; p->d_items[l] = nullptr; p->d_gchunks[l] = nullptr; p->n_btab[l] = p->n_items[l] = 0; p->single_pass_bundle[l] = 0; }
    p->max_copies = 2;
    p->fuse_leaf_update = 1;
    if (cudaFuncSetAttribute(cb_level_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, p->max_smem) != cudaSuccess) {
        cudaGetLastError();
        delete p;
        return nullptr;
    }
    return p;
}

// domw: one packed word per feature group (the dominant bin of each of its four features, 255 = none), or null
CB_API void cb_fused_set_dominant(CbFusedPlan* p, const unsigned int* domw) { p->a.h.domw = domw; }
CB_API void cb_fused_set_fuse_leaf(CbFusedPlan* p, int on) { p->fuse_leaf_update = on ? 1 : 0; }
CB_API void cb_fused_set_phase_ts(CbFusedPlan* p, unsigned long long* ts) { p->a.phase_ts = ts; }
CB_API void cb_fused_set_work(CbFusedPlan* p, unsigned int* work) { p->a.h.work = work; }
CB_API void cb_fused_set_narrow(CbFusedPlan* p, int narrow, int max_bundle) {
    p->a.h.narrow = narrow;
    p->max_bundle = max_bundle > 8 ? 8 : max_bundle;
}

CB_API void cb_fused_set_features(CbFusedPlan* p, int f_begin, int f_end) {
    p->a.s.f_begin = f_begin;
    p->a.s.f_end = f_end;
}

CB_API void cb_fused_destroy(CbFusedPlan* p) {
    if (!p) return;
    for (int l = 0; l < CB_MAX_LEVELS; ++l) {
        if (p->d_btab[l]) cudaFree(p->d_btab[l]);
        if (p->d_items[l]) cudaFree(p->d_items[l]);
        if (p->d_gchunks[l]) cudaFree(p->d_gchunks[l]);
    }
    delete p;
}

// Padded number of bins (multiple of 4) of the widest feature of every feature group, host memory.  With it the
// bundled path sizes the tile of a bundle by its own widest feature instead of the widest feature of the data set.
CB_API void cb_fused_set_group_bins(CbFusedPlan* p, const int* group_bins, int G) {
    p->group_bins.assign(group_bins, group_bins + G);
}

// Launch geometry of one level.  Returns the cooperative grid size (0 on error) and, through the pointers, the
// slots per pass, dynamic shared memory, block size, document chunks per group and cell replicas.
CB_API void cb_fused_set_max_copies(CbFusedPlan* p, int max_copies) {
    p->max_copies = max_copies >= 8 ? 8 : (max_copies >= 4 ? 4 : (max_copies >= 2 ? 2 : 1));
}

CB_API int cb_fused_geometry(CbFusedPlan* p, int level, int* slots_per_pass, int* smem_bytes, int* threads, int* chunks,
                             int* copies, int* bundle) {
    const int nslots = level == 0 ? 1 : (1 << (level - 1));
    const bool narrow = p->a.h.statmax && p->a.h.S == 2 && p->a.h.narrow;
    const int G = p->a.h.d.G;
    const long long n = p->a.h.d.n;
    int thr = p->threads, spp = nslots, C = 1, gpc = 0, smem = 0;
    std::vector<CbBundle> bundles;
    if (narrow && p->max_bundle > 0) {
        // Bundled single-cell path: a block accumulates the groups of one bundle at once.  Tile of a bundle =
        // slots * groups * 8 * B * C ints with B the padded bins of its widest feature, ring = warps * 64 * (3 + groups)
        // words.  Consecutive groups of similar width (within a factor of two) form a run; a run is cut into the fewest
        // bundles whose tiles hold every slot, evened out (7 groups as 4 + 3 rather than 5 + 2); when not even one group
        // holds all slots the group takes several passes over the slots.  Then the cells are replicated while room is left.
        // One 1024-thread block per SM: measured a few percent faster than two 512-thread blocks at every level (one
        // tile instead of two leaves room for wider bundles and replicas) and it balances better.
        const bool skip = p->a.h.domw != nullptr;       // dominant-bin skipping: 256 bytes of slot totals per slot
        const int budget = p->max_smem;
        thr = 1024;
        auto gb = [&](int g) { return p->group_bins.empty() ? p->a.h.B : p->group_bins[g]; };
        auto need = [&](int slots, int gc, int Bb, int Cc) {
            return slots * gc * 8 * Bb * 4 * Cc + (thr / 32) * 64 * (3 + gc) * 4 + 16 + (skip ? slots * 256 : 0);
        };
        int max_copies = p->max_copies;
        if (const char* e = getenv("CB200_MAX_COPIES")) { const int v = atoi(e); if (v == 1 || v == 2 || v == 4 || v == 8) max_copies = v; }
        int g = 0;
        while (g < G) {
            int lo_b = gb(g), hi_b = gb(g), run = 1;
            while (g + run < G) {
                const int b2 = gb(g + run);
                const int lo2 = b2 < lo_b ? b2 : lo_b, hi2 = b2 > hi_b ? b2 : hi_b;
                if (hi2 > 2 * lo2) break;
                lo_b = lo2; hi_b = hi2; ++run;
            }
            int fitg = 0;
            while (fitg < run && fitg < p->max_bundle && need(nslots, fitg + 1, hi_b, 1) <= budget) ++fitg;
            if (fitg < 1) {
                for (int q = 0; q < run; ++q) {
                    const int Bb = gb(g + q);
                    int s1 = (budget - need(0, 1, Bb, 1)) / (8 * Bb * 4 + (skip ? 256 : 0));
                    if (s1 < 1) return 0;
                    const int np = (nslots + s1 - 1) / s1;
                    s1 = (nslots + np - 1) / np;
                    bundles.push_back(CbBundle{g + q, 1, Bb, 1, s1, np, 1});
                }
            } else {
                const int nbr = (run + fitg - 1) / fitg;
                int at = g;
                for (int q = 0; q < nbr; ++q) {
                    const int cnt = (run - (at - g) + (nbr - q) - 1) / (nbr - q);
                    int Bb = 4;
                    for (int k = 0; k < cnt; ++k) Bb = gb(at + k) > Bb ? gb(at + k) : Bb;
                    bundles.push_back(CbBundle{at, cnt, Bb, 1, nslots, 1, 1});
                    at += cnt;
                }
            }
            g += run;
        }
        // Replicas: columns of few bins put many lanes of a warp on the same cell whatever the data look like (32 lanes
        // over 16 bins), so their bundles take up to 8 replicas; measured on 4.5M x 52 columns (13 floats, 39 CTR columns
        // of 16 bins), depth 8: 7.4 ms per tree against 9.8 ms with 2 replicas.
        int narrow_copies = 8;
        if (const char* e = getenv("CB200_NARROW_COPIES")) { const int v = atoi(e); if (v == 1 || v == 2 || v == 4 || v == 8) narrow_copies = v; }
        for (CbBundle& b : bundles) {
            const int mc = b.B <= 32 ? (narrow_copies > max_copies ? narrow_copies : max_copies) : max_copies;
            while (b.C < mc && need(b.spp, b.gcnt, b.B, 2 * b.C) <= budget) b.C *= 2;
            const int nb_ = need(b.spp, b.gcnt, b.B, b.C);
            if (nb_ > smem) smem = nb_;
        }
        spp = bundles[0].spp; C = bundles[0].C; gpc = bundles[0].gcnt;
    } else {
        const bool narrow_cells = p->a.h.statmax && p->a.h.narrow;      // one int32 per cell, any number of statistics
        const int per_slot = p->a.h.S * 4 * p->a.h.B * 4 * ((p->a.h.statmax && !narrow_cells) ? 2 : 1);
        const bool ring = p->a.h.statmax && p->a.h.S == 2;      // per-warp compaction rings (16 bytes x 64 entries)
        int ring_bytes = ring ? (thr / 32) * 64 * 16 + 16 : 0;
        int budget = p->max_smem - ring_bytes;
        if (spp * per_slot > budget / 2) {
            // one 1024-thread block per SM when the tile needs more than half of the shared memory
            thr = 1024;
            ring_bytes = ring ? (thr / 32) * 64 * 16 + 16 : 0;
            budget = p->max_smem - ring_bytes;
        }
        if (spp * per_slot > budget) spp = budget / per_slot;
        if (spp < 1) return 0;
        // replicate the cells while two blocks per SM still fit (fewer bank / address collisions per atomic)
        if (ring && thr == p->threads) {
            while (C < 8 && 2 * (spp * per_slot * (C * 2) + ring_bytes) <= p->max_smem) C *= 2;
        }
        smem = spp * per_slot * C + ring_bytes;
    }
    // the score phase reuses the tile as scratch: CB_SCORE_WARP_FLOATS floats per scoring warp, at least 8 warps' worth
    // (a small tile -- few bins, one slot -- would otherwise leave it without a single warp)
    {
        const int want = (thr / 32 < 8 ? thr / 32 : 8) * CB_SCORE_WARP_FLOATS * 4;
        if (smem < want) smem = want;
    }
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cb_level_fused_kernel, thr, smem) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (occ < 1) return 0;
    if (occ > 4) occ = 4;
    const int grid = occ * p->sm_count;
    // document chunks per work unit (group or bundle): at least what the grid offers and what the 2^19-documents-per-
    // tile cap needs; among a few candidates take the one that fills the last round of blocks best
    const int by_docs = (int)((n + (1 << 19) - 1) >> 19);
    int best = 1;
    if (bundles.empty()) {
        const int units = G;
        const int by_grid = grid >= units ? grid / units : 1;
        const int lo = by_grid > by_docs ? by_grid : by_docs;
        best = lo;
        double best_eff = 0.0;
        for (int k = lo; k < lo + 8; ++k) {
            const long long items = (long long)units * k;
            const long long rounds = (items + grid - 1) / grid;
            const double eff = (double)items / (double)(rounds * grid);
            if (eff > best_eff + 0.02) { best_eff = eff; best = k; }
        }
    } else {
        if (level >= CB_MAX_LEVELS) return 0;
        // Every bundle is cut into its own number of document chunks so that all work items take about the same time
        // and their number is a whole multiple of the grid.  Cost of an item per document it streams: a fixed part (leaf
        // index, two statistics, compaction) worth 2.8 groups plus one unit per group of the bundle (measured on 4.5M
        // x 52 columns, depth 8: a one-group item took 0.49 of the time of a five-group item over the same documents).
        const int nbun = (int)bundles.size();
        std::vector<double> cost(nbun);
        std::vector<int> nk(nbun);
        double W = 0.0;
        long long min_items = 0;
        for (int i = 0; i < nbun; ++i) {
            cost[i] = 2.8 + bundles[i].gcnt;
            W += cost[i] * bundles[i].npass;
            min_items += (long long)bundles[i].npass * by_docs;
        }
        // bundles of different shapes: the cost model is rough (bin collisions depend on the data), so the work is cut
        // into two rounds of items handed out by a counter, which bounds the imbalance by half an item's time (measured
        // on the same data: 7.2 ms per tree with one round, 7.1 with two, 7.8 with four -- every item zeroes and dumps a tile)
        bool mixed = false;
        for (int i = 1; i < nbun; ++i)
            if (bundles[i].B != bundles[0].B || bundles[i].npass != bundles[0].npass || bundles[i].C != bundles[0].C) mixed = true;
        int rounds = (mixed && p->a.h.work) ? 2 : 1;
        if (const char* e = getenv("CB200_ITEM_ROUNDS")) { const int v = atoi(e); if (v >= 1 && v <= 16) rounds = v; }
        long long T = (long long)grid * rounds;
        while (T < min_items) T += grid;
        long long used = 0;
        for (int i = 0; i < nbun; ++i) {
            int k = (int)((double)T * cost[i] / W);
            if (k < by_docs) k = by_docs;
            if (k < 1) k = 1;
            nk[i] = k;
            used += (long long)k * bundles[i].npass;
        }
        for (;;) {
            int pick = -1;
            double worst = 0.0;
            for (int i = 0; i < nbun; ++i) {
                if (used + bundles[i].npass > T) continue;
                const double t = cost[i] / nk[i];
                if (t > worst) { worst = t; pick = i; }
            }
            if (pick < 0) break;
            ++nk[pick];
            used += bundles[pick].npass;
        }
        // work list: chunk-major, so that blocks running side by side stream the same documents (their leaf indices and
        // statistics then come from L2); the wider bundles of a chunk first
        std::vector<int> order(nbun);
        for (int i = 0; i < nbun; ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return cost[x] / nk[x] > cost[y] / nk[y]; });
        std::vector<int2> items;
        std::vector<int> gchunks(G, 1);
        for (int i = 0; i < nbun; ++i) {
            bundles[i].nK = nk[i];
            if (nk[i] > best) best = nk[i];
            for (int q = 0; q < bundles[i].gcnt; ++q) gchunks[bundles[i].g0 + q] = nk[i];
        }
        items.reserve((size_t)used);
        for (int k = 0; k < best; ++k)
            for (int bi : order)
                if (k < nk[bi])
                    for (int ps = 0; ps < bundles[bi].npass; ++ps) items.push_back(make_int2(bi | (ps << 16), k));
        if (p->d_btab[level]) { cudaFree(p->d_btab[level]); p->d_btab[level] = nullptr; }
        if (p->d_items[level]) { cudaFree(p->d_items[level]); p->d_items[level] = nullptr; }
        if (p->d_gchunks[level]) { cudaFree(p->d_gchunks[level]); p->d_gchunks[level] = nullptr; }
        if (cudaMalloc(&p->d_btab[level], bundles.size() * sizeof(CbBundle)) != cudaSuccess ||
            cudaMalloc(&p->d_items[level], items.size() * sizeof(int2)) != cudaSuccess ||
            cudaMalloc(&p->d_gchunks[level], (size_t)G * sizeof(int)) != cudaSuccess) { cudaGetLastError(); return 0; }
        cudaMemcpy(p->d_btab[level], bundles.data(), bundles.size() * sizeof(CbBundle), cudaMemcpyHostToDevice);
        cudaMemcpy(p->d_items[level], items.data(), items.size() * sizeof(int2), cudaMemcpyHostToDevice);
        cudaMemcpy(p->d_gchunks[level], gchunks.data(), (size_t)G * sizeof(int), cudaMemcpyHostToDevice);
        p->n_btab[level] = nbun;
        p->n_items[level] = (int)items.size();
        p->single_pass_bundle[level] = (nbun == 1 && bundles[0].npass == 1 && bundles[0].gcnt >= G) ? 1 : 0;
    }
    *slots_per_pass = spp;
    *smem_bytes = smem;
    *threads = thr;
    *chunks = best;
    *copies = C;
    *bundle = gpc;
    return grid;
}

CB_API void cb_fused_set_priv(CbFusedPlan* p, float* priv, const float* statmax) { p->a.h.priv = priv; p->a.h.statmax = statmax; }

CB_API int cb_fused_launch(CbFusedPlan* p, int level, float* hprev, float* hcur, const unsigned int* mask_in,
                           unsigned int* mask_out, int grid, int slots_per_pass, int smem_bytes, int threads,
                           int chunks, int copies, int bundle, cudaStream_t st) {
    CbFusedArgs a = p->a;
    a.h.nK = chunks; a.h.copies = copies; a.h.bundle = bundle;
    a.h.level = level; a.h.small_mask = mask_in; a.h.slots_per_pass = slots_per_pass;
    a.s.level = level; a.s.small_mask = mask_in; a.s.hprev = hprev; a.s.hcur = hcur;
    a.mask_out = mask_out;
    a.smem_floats = smem_bytes / 4;
    // the bundled histogram pass can apply the previous level's split itself (see CbHistArgs::prev_split)
    // ... when one bundle holds every feature group: then the split feature's bin word is already in registers and each
    // document is streamed by exactly one block.  With several bundles each of them would have to fetch that word as
    // well, which costs more than the separate pass (measured at 10.5M x 28, level 5, 4 bundles: +86 us against 18 us).
    const bool table = bundle > 0 && level < CB_MAX_LEVELS && p->d_btab[level] != nullptr;
    a.h.btab = table ? p->d_btab[level] : nullptr;
    a.h.bitems = table ? p->d_items[level] : nullptr;
    a.h.nbitems = table ? p->n_items[level] : 0;
    a.h.gchunks = table ? p->d_gchunks[level] : nullptr;
    const bool whole = table ? p->single_pass_bundle[level] != 0 : bundle >= a.h.d.G;
    a.fuse_leaf = (level > 0 && whole && a.h.statmax && a.h.S == 2 && a.h.narrow && p->fuse_leaf_update) ? 1 : 0;
    a.h.prev_splits = a.fuse_leaf ? a.splits : nullptr;
    void* args[] = {&a};
    cudaError_t e = cudaLaunchCooperativeKernel((void*)cb_level_fused_kernel, dim3(grid), dim3(threads), args,
                                                (size_t)smem_bytes, st);
    return (int)e;
}
