// Nearest-neighbour candidates for embedding features: distance GEMM on the 5th-generation tensor cores fused with the
// top-k selection, so the [queries x cloud] distance matrix never exists in memory.
//
// What it computes (the estimator it serves: catboost/private/libs/embedding_features/knn.cpp, class votes of the k
// nearest learn documents): for every query row q and every cloud row e, s(q, e) = |e|^2 - 2 q.e, which orders the cloud
// rows exactly like the Euclidean distance does; the CB_KNN_CAND smallest s per query come back with their indices.
// Inputs are bf16 (fp32 accumulation), so the order is approximate among near ties: the caller re-ranks the candidates
// with fp32 distances and keeps k <= CB_KNN_CAND / 2 of them.
//
// Structure of a CTA (384 threads, one tile of 128 queries, a range of 256-row cloud tiles):
//   warp 0   producer: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) loads the query tile once -- all K chunks stay
//            in shared memory up to 256 dimensions, above that they travel with the cloud chunks -- and streams the
//            cloud tiles through a ring of [256 rows x 64 bf16] boxes that takes all the shared memory left;
//   warp 1   one elected lane issues tcgen05.mma (M = 128, N = 256, K = 16, operands from shared memory through matrix
//            descriptors, accumulator in TMEM), tcgen05.commit releases the ring stage / publishes the accumulator;
//   warp 2   allocates and frees all 512 TMEM columns: two accumulators, so tile i + 1 is multiplied while tile i is read;
//   warps 4-11 epilogue: thread = query row = TMEM lane, two warps per lane quarter (128 columns of the tile each);
//            tcgen05.ld brings 64 columns at a time into registers, the TMEM buffer is handed back after the second read,
//            s = |e|^2 - 2 acc (|e|^2 from shared memory), the minimum of every 32 scores by a tree of minima, and a
//            sorted insertion into the thread's candidate list only for groups that hold something below its worst entry.
// Every mbarrier wait is bounded; when one runs out the CTA records CB_KNN_TIMEOUT in *status, every role leaves its
// loop, the CTA idles long enough for copies and MMAs in flight to land, frees its TMEM and returns.
#include "cb_common.cuh"
#include <cuda.h>
#include <cuda_bf16.h>

#define CB_KNN_CAND 16
#define CB_KNN_TM 128                 // queries per CTA (MMA M)
#define CB_KNN_TN 256                 // cloud rows per tile (MMA N): at N = 128 an MMA reads 8 KB of operands per 64 clocks,
                                      // all a SM's shared memory can deliver; at N = 256 it is 12 KB per 128 clocks
#define CB_KNN_KC 64                  // bf16 per K chunk = one 128-byte swizzled row
#define CB_KNN_MAX_STAGES 12           // the ring takes what is left of the 227 KB, up to this many stages
#define CB_KNN_FIXED_BYTES 37888       // barriers (256) | norms (4096) | abort flag | insertion scratch (32768), 1024-aligned
#define CB_KNN_SMEM_BYTES 232448       // all the shared memory a CTA may have
#define CB_KNN_BAD_LAYOUT 0x62
#define CB_KNN_MAX_KCHUNKS 4          // query tile resident in shared memory: up to 256 dimensions
#define CB_KNN_A_BYTES (CB_KNN_TM * CB_KNN_KC * 2)   // one K chunk of the query tile: 16 KB
#define CB_KNN_B_BYTES (CB_KNN_TN * CB_KNN_KC * 2)   // one K chunk of a cloud tile: 32 KB
#define CB_KNN_TIMEOUT 0x61
#define CB_KNN_WAIT_LIMIT (1 << 22)
#define CB_KNN_THREADS 384             // 4 role warps + 8 epilogue warps

__device__ __forceinline__ unsigned int cbk_smem_u32(const void* p) { return (unsigned int)__cvta_generic_to_shared(p); }

// three-input minimum (one instruction on sm_100)
__device__ __forceinline__ float cbk_min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ bool cbk_wait(unsigned int bar, unsigned int parity) {
    for (int it = 0; it < CB_KNN_WAIT_LIMIT; ++it) {
        unsigned int ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) with the 128-byte swizzle: groups
// of 8 rows lie 1024 bytes apart (stride byte offset), the leading byte offset is not used by swizzled K-major layouts
// (1 by convention), descriptor version 1, layout type 2 = SWIZZLE_128B.  Addresses and offsets are in 16-byte units.
__device__ __forceinline__ unsigned long long cbk_desc(unsigned int smem_addr) {
    return (unsigned long long)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D = fp32 (bits 4-5 = 1), A = B = bf16 (bits 7-9 and 10-12 = 1), both K-major, N / 8 at bit 17,
// M / 16 at bit 24.
#define CB_KNN_IDESC ((1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(CB_KNN_TN >> 3) << 17) | ((unsigned)(CB_KNN_TM >> 4) << 24))

struct CbKnnArgs {
    const float* e2;          // [ne] squared norms of the (bf16-rounded) cloud rows
    int nq, ne, kchunks;
    int stream_a;             // more K chunks than fit resident: the query chunk travels with every cloud chunk
    int smem_bytes;           // dynamic shared memory of the launch
    int tiles_per_split;      // cloud tiles handled by one blockIdx.y
    int* out_idx;             // [nq][2 * splits][candidates per list]
    float* out_val;
    int* status;
};

template <int CAND>
__global__ void __launch_bounds__(CB_KNN_THREADS, 1) cb_knn_tc_kernel(const __grid_constant__ CUtensorMap tmq,
                                                           const __grid_constant__ CUtensorMap tme, CbKnnArgs a) {
    extern __shared__ unsigned char cbk_raw[];
    unsigned char* smem = cbk_raw + ((1024u - (cbk_smem_u32(cbk_raw) & 1023u)) & 1023u);
    // barriers | norms of the epilogue warps | abort flag | insertion scratch || [kchunks] query chunks | ring.  A copy in
    // flight is the only thing that hides the L2 latency from the tensor pipe (with 4 stages of 16 KB it was busy a third
    // of the time), so the ring gets every byte the CTA can have.
    const bool stream = a.stream_a != 0;
    const int stage_bytes = stream ? CB_KNN_A_BYTES + CB_KNN_B_BYTES : CB_KNN_B_BYTES;
    const int kch = a.kchunks;
    const int pad = (int)(smem - cbk_raw);
    int nst = (a.smem_bytes - pad - CB_KNN_FIXED_BYTES - (stream ? 0 : kch * CB_KNN_A_BYTES)) / stage_bytes;
    if (nst > CB_KNN_MAX_STAGES) nst = CB_KNN_MAX_STAGES;
    if (nst < 2) {                                                          // uniform: nobody has touched a barrier yet
        if (threadIdx.x == 0) atomicExch(a.status, CB_KNN_BAD_LAYOUT);
        return;
    }
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem);
    // bars: full[MAX_STAGES] | empty[MAX_STAGES] | a_full | tmem_full[2] | tmem_empty[2] | tmem base
    const unsigned int bar_full = cbk_smem_u32(bars), bar_empty = cbk_smem_u32(bars + CB_KNN_MAX_STAGES);
    const unsigned int bar_a = cbk_smem_u32(bars + 2 * CB_KNN_MAX_STAGES);
    const unsigned int bar_tfull = cbk_smem_u32(bars + 2 * CB_KNN_MAX_STAGES + 1);
    const unsigned int bar_tempty = cbk_smem_u32(bars + 2 * CB_KNN_MAX_STAGES + 3);
    unsigned int* tmem_slot = reinterpret_cast<unsigned int*>(bars + 2 * CB_KNN_MAX_STAGES + 5);
    float (*s_e2)[128] = reinterpret_cast<float (*)[128]>(smem + 256);        // [8][128]
    int& s_abort = *reinterpret_cast<int*>(smem + 256 + 4096);
    float* scratch = reinterpret_cast<float*>(smem + 5120);                    // 8 epilogue warps x 1024 floats
    unsigned char* sA = smem + CB_KNN_FIXED_BYTES;                            // resident query chunks (not when streaming)
    unsigned char* ring = stream ? sA : sA + kch * CB_KNN_A_BYTES;
    unsigned char* sB = ring + (stream ? CB_KNN_A_BYTES : 0);              // cloud chunk of stage 0

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles_all = (a.ne + CB_KNN_TN - 1) / CB_KNN_TN;
    const int t0 = blockIdx.y * a.tiles_per_split;
    const int t1 = min(ntiles_all, t0 + a.tiles_per_split);
    const int ntiles = max(0, t1 - t0);
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < CB_KNN_MAX_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_full + 8 * s) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_empty + 8 * s) : "memory");
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
        for (int b = 0; b < 2; ++b) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_tfull + 8 * b) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 8;" ::"r"(bar_tempty + 8 * b) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(cbk_smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned int tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- producer ----------------------------------------------------------------------------------------
        if (lane == 0 && ntiles > 0) {
            if (!stream) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(kch * CB_KNN_A_BYTES) : "memory");
                for (int kc = 0; kc < kch; ++kc)
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(cbk_smem_u32(sA + kc * CB_KNN_A_BYTES)), "l"(&tmq), "r"(kc * CB_KNN_KC),
                                   "r"((int)(blockIdx.x * CB_KNN_TM)), "r"(bar_a) : "memory");
            }
            int it = 0;
            bool ok = true;
            for (int t = 0; t < ntiles && ok; ++t) {
                for (int kc = 0; kc < kch; ++kc, ++it) {
                    const int s = it % nst;
                    const unsigned int ph = (unsigned)(it / nst) & 1u;
                    if (*(volatile int*)&s_abort || !cbk_wait(bar_empty + 8 * s, ph ^ 1u)) { ok = false; break; }
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_full + 8 * s), "r"(stage_bytes) : "memory");
                    if (stream)
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                     ::"r"(cbk_smem_u32(ring + s * stage_bytes)), "l"(&tmq), "r"(kc * CB_KNN_KC),
                                       "r"((int)(blockIdx.x * CB_KNN_TM)), "r"(bar_full + 8 * s) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(cbk_smem_u32(sB + s * stage_bytes)), "l"(&tme), "r"(kc * CB_KNN_KC),
                                   "r"((t0 + t) * CB_KNN_TN), "r"(bar_full + 8 * s) : "memory");
                }
            }
            if (!ok) { atomicExch(a.status, CB_KNN_TIMEOUT); *(volatile int*)&s_abort = 1; }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------------
        if (lane == 0 && ntiles > 0) {
            bool ok = stream ? true : cbk_wait(bar_a, 0u);
            int it = 0;
            for (int t = 0; t < ntiles && ok; ++t) {
                const int buf = t & 1;
                const unsigned int tph = (unsigned)(t >> 1) & 1u;
                if (*(volatile int*)&s_abort || !cbk_wait(bar_tempty + 8 * buf, tph ^ 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned int dcol = tmem_base + (unsigned)buf * CB_KNN_TN;
                for (int kc = 0; kc < kch; ++kc, ++it) {
                    const int s = it % nst;
                    const unsigned int ph = (unsigned)(it / nst) & 1u;
                    if (!cbk_wait(bar_full + 8 * s, ph)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long da = cbk_desc(cbk_smem_u32(stream ? ring + s * stage_bytes : sA + kc * CB_KNN_A_BYTES));
                    const unsigned long long db = cbk_desc(cbk_smem_u32(sB + s * stage_bytes));
#pragma unroll
                    for (int k = 0; k < CB_KNN_KC / 16; ++k) {
                        const unsigned int acc = (kc | k) ? 1u : 0u;
                        // 16 bf16 = 32 bytes = 2 descriptor units further along the swizzled row
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                     ::"r"(dcol), "l"(da + 2ull * k), "l"(db + 2ull * k), "r"(CB_KNN_IDESC), "r"(acc) : "memory");
                    }
                    // the stage may be refilled once these MMAs have read it
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_empty + 8 * s) : "memory");
                }
                if (ok)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_tfull + 8 * buf) : "memory");
            }
            if (!ok) { atomicExch(a.status, CB_KNN_TIMEOUT); *(volatile int*)&s_abort = 1; }
        }
    } else if (warp >= 4) {
        // ---- epilogue: 8 warps, warp quarter = TMEM lanes (a warp may only read lanes 32 (warp % 4) ...), warp half =
        // columns 0-127 or 128-255 of the tile; a query row therefore has two candidate lists, merged by the caller ------
        const int ew = warp - 4, wq = ew & 3, half = ew >> 2;
        const int row = blockIdx.x * CB_KNN_TM + wq * 32 + lane;
        float val[CAND];
        int idx[CAND];
#pragma unroll
        for (int c = 0; c < CAND; ++c) { val[c] = 3.0e38f; idx[c] = -1; }
        bool ok = true;
        // |e|^2 of the warp's 128 columns goes through the warp's own piece of shared memory (broadcast reads; no barrier
        // between warps, so a warp that gives up on a wait cannot leave the others stuck).  Columns past the end of the
        // cloud get a huge norm and never enter a list.  The values of the next tile are fetched while this one is processed.
        float* my_e2 = s_e2[ew];
        float* my_sc = scratch + ew * 1024;                       // [32 columns][32 lanes] of the group being inserted
        float e2v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int col = t0 * CB_KNN_TN + half * 128 + u * 32 + lane;
            e2v[u] = (ntiles > 0 && col < a.ne) ? __ldg(a.e2 + col) : 3.0e38f;
        }
        for (int t = 0; t < ntiles && ok; ++t) {
            const int buf = t & 1;
            const unsigned int tph = (unsigned)(t >> 1) & 1u;
            __syncwarp();                                          // the previous tile's reads are done
#pragma unroll
            for (int u = 0; u < 4; ++u) my_e2[u * 32 + lane] = e2v[u];
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int col = (t0 + t + 1) * CB_KNN_TN + half * 128 + u * 32 + lane;
                e2v[u] = (t + 1 < ntiles && col < a.ne) ? __ldg(a.e2 + col) : 3.0e38f;
            }
            // the whole warp decides together whether the wait succeeded: the votes further down need all 32 lanes
            const bool arrived = !(*(volatile int*)&s_abort) && cbk_wait(bar_tfull + 8 * buf, tph);
            if (!__all_sync(0xffffffffu, arrived)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#define CBK_LD32(R, ADDR)                                                                                                  \
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                         \
                         "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                         \
                         "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"          \
                         : "=r"(R[0]), "=r"(R[1]), "=r"(R[2]), "=r"(R[3]), "=r"(R[4]), "=r"(R[5]), "=r"(R[6]), "=r"(R[7]), \
                           "=r"(R[8]), "=r"(R[9]), "=r"(R[10]), "=r"(R[11]), "=r"(R[12]), "=r"(R[13]), "=r"(R[14]),        \
                           "=r"(R[15]), "=r"(R[16]), "=r"(R[17]), "=r"(R[18]), "=r"(R[19]), "=r"(R[20]), "=r"(R[21]),      \
                           "=r"(R[22]), "=r"(R[23]), "=r"(R[24]), "=r"(R[25]), "=r"(R[26]), "=r"(R[27]), "=r"(R[28]),      \
                           "=r"(R[29]), "=r"(R[30]), "=r"(R[31])                                                           \
                         : "r"(ADDR) : "memory")
            const unsigned int taddr = tmem_base + ((unsigned)(wq * 32) << 16) + (unsigned)(buf * CB_KNN_TN + half * 128);
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {                  // 64 of the warp's 128 columns at a time
                unsigned int r[64];
                CBK_LD32((r), taddr + (unsigned)(pass * 64));
                CBK_LD32((r + 32), taddr + (unsigned)(pass * 64 + 32));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (pass == 1) {
                    // the whole accumulator has been read: hand the TMEM buffer back before the selection work
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_tempty + 8 * buf) : "memory");
                }
                const int cbase = (t0 + t) * CB_KNN_TN + half * 128 + pass * 64;
                const float4* e4 = reinterpret_cast<const float4*>(my_e2 + pass * 64);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    float sc[32];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 e = e4[c * 8 + j];
                        sc[4 * j + 0] = fmaf(-2.0f, __uint_as_float(r[c * 32 + 4 * j + 0]), e.x);
                        sc[4 * j + 1] = fmaf(-2.0f, __uint_as_float(r[c * 32 + 4 * j + 1]), e.y);
                        sc[4 * j + 2] = fmaf(-2.0f, __uint_as_float(r[c * 32 + 4 * j + 2]), e.z);
                        sc[4 * j + 3] = fmaf(-2.0f, __uint_as_float(r[c * 32 + 4 * j + 3]), e.w);
                    }
                    // smallest score of the 32 by a tree of three-input minima (17 instructions instead of 31): most
                    // groups hold nothing below the list's worst entry
                    float m[11];
#pragma unroll
                    for (int j = 0; j < 10; ++j) m[j] = cbk_min3(sc[3 * j], sc[3 * j + 1], sc[3 * j + 2]);
                    m[10] = fminf(sc[30], sc[31]);
                    m[0] = cbk_min3(cbk_min3(m[0], m[1], m[2]), cbk_min3(m[3], m[4], m[5]), cbk_min3(m[6], m[7], m[8]));
                    m[0] = cbk_min3(m[0], m[9], m[10]);
                    // A thread's list changes about CAND ln(columns / CAND) times in a whole scan, so a group of 32 columns
                    // holds a few insertions per warp.  The insertion is a compact loop, not 32 unrolled copies (those ran
                    // into instruction-fetch stalls: 12.6 stalled cycles per issue): the group's scores go to the warp's
                    // scratch in shared memory, every lane keeps a bit mask of its columns below the worst entry, and the
                    // warp loops while any lane has a bit left, one sorted insertion a turn.
                    if (__any_sync(0xffffffffu, m[0] < val[CAND - 1])) {
                        unsigned int hm = 0u;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            my_sc[j * 32 + lane] = sc[j];
                            hm |= (sc[j] < val[CAND - 1]) ? (1u << j) : 0u;
                        }
                        while (__any_sync(0xffffffffu, hm != 0u)) {
                            if (hm) {
                                const int j = __ffs(hm) - 1;
                                hm &= hm - 1u;
                                const float sv = my_sc[j * 32 + lane];
                                if (sv < val[CAND - 1]) { val[CAND - 1] = sv; idx[CAND - 1] = cbase + c * 32 + j; }
                            }
#pragma unroll
                            for (int q = CAND - 1; q > 0; --q) {
                                const bool sw = val[q] < val[q - 1];
                                const float lo = sw ? val[q] : val[q - 1], hi = sw ? val[q - 1] : val[q];
                                const int li = sw ? idx[q] : idx[q - 1], hi_i = sw ? idx[q - 1] : idx[q];
                                val[q - 1] = lo; val[q] = hi; idx[q - 1] = li; idx[q] = hi_i;
                            }
                        }
                    }
                }
            }
        }
        if (!ok) { atomicExch(a.status, CB_KNN_TIMEOUT); *(volatile int*)&s_abort = 1; }
        if (row < a.nq) {
            const long long o = ((long long)row * (gridDim.y * 2) + blockIdx.y * 2 + half) * CAND;
#pragma unroll
            for (int c = 0; c < CAND; ++c) { a.out_val[o + c] = val[c]; a.out_idx[o + c] = idx[c]; }
        }
    }
    __syncthreads();
    if (*(volatile int*)&s_abort) {
        // copies and MMAs that were issued before a wait ran out get time to land before the CTA's memory is given back
        for (int w = 0; w < 200; ++w) __nanosleep(1000);
        __syncthreads();
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 2)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
}

typedef CUresult (*CbkEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static CbkEncodeTiled cbk_encode_tiled() {
    static CbkEncodeTiled fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<CbkEncodeTiled>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

static int cbk_make_map(CUtensorMap* tm, const void* base, long long rows, int dpad, int box_rows) {
    CbkEncodeTiled enc = cbk_encode_tiled();
    if (!enc) return -2;
    const cuuint64_t gdim[2] = {(cuuint64_t)dpad, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)dpad * 2};
    const cuuint32_t box[2] = {CB_KNN_KC, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2;
}

CB_API int cb_knn_candidates(void) { return CB_KNN_CAND; }
// Largest dimension count (after padding to 64) the kernel takes; up to 256 the query tile stays in shared memory, above
// that its chunks are streamed with the cloud chunks.
CB_API int cb_knn_max_dim(void) { return 4096; }

// Number of cloud ranges (blockIdx.y); a range is never shorter than 4 tiles.
CB_API int cb_knn_splits(int nq, int ne) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int qt = (nq + CB_KNN_TM - 1) / CB_KNN_TM, et = (ne + CB_KNN_TN - 1) / CB_KNN_TN;
    // Ranges are only there to give every SM a CTA when there are few query tiles: every range keeps candidate lists of
    // its own, and a list over fewer columns changes more often per column (16 ln(columns / 16) insertions), which is
    // what the epilogue pays for.  Measured at 65536 x 131072 x 128: 1 range 4.39 ms, 2 ranges (fuller last round) 4.67 ms.
    int s = (sms + qt - 1) / (qt > 0 ? qt : 1);
    if (s > et / 4) s = et / 4;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return s;
}

// Q [nq][dpad] and E [ne][dpad] are bf16, row-major, 16-byte aligned, dpad a multiple of 64 and at most
// cb_knn_max_dim(); e2 [ne] fp32.  out_idx / out_val are [nq][splits][CB_KNN_CAND]; entries that were never filled hold
// index -1.  Returns 0 when the kernel was enqueued, -2 when the shape does not qualify, a CUDA error code otherwise.
// *status (device int, zero on entry) receives CB_KNN_TIMEOUT when a wait inside the kernel ran out.  cand = 8 or 16 is the
// length of a candidate list (the last dimension of the outputs): the epilogue's work grows with its square.
CB_API int cb_knn_tc(const void* Q, int nq, const void* E, int ne, int dpad, const float* e2, int splits, int cand, int* out_idx,
                     float* out_val, int* status, cudaStream_t st) {
    if (cand != 8 && cand != 16) return -2;
    if (nq <= 0 || ne <= 0) return 0;
    if (dpad <= 0 || dpad % CB_KNN_KC != 0 || dpad > 4096 || splits < 1 || splits > 65535) return -2;
    if ((reinterpret_cast<unsigned long long>(Q) & 15ull) || (reinterpret_cast<unsigned long long>(E) & 15ull)) return -2;
    CUtensorMap tmq, tme;
    if (cbk_make_map(&tmq, Q, nq, dpad, CB_KNN_TM) != 0 || cbk_make_map(&tme, E, ne, dpad, CB_KNN_TN) != 0) return -2;
    const int smem = CB_KNN_SMEM_BYTES;
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_knn_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(cb_knn_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    const int et = (ne + CB_KNN_TN - 1) / CB_KNN_TN;
    CbKnnArgs a{e2, nq, ne, dpad / CB_KNN_KC, dpad / CB_KNN_KC > CB_KNN_MAX_KCHUNKS ? 1 : 0, smem, (et + splits - 1) / splits, out_idx,
                out_val, status};
    dim3 grid((unsigned)((nq + CB_KNN_TM - 1) / CB_KNN_TM), (unsigned)splits);
    if (cand == 8) cb_knn_tc_kernel<8><<<grid, CB_KNN_THREADS, smem, st>>>(tmq, tme, a);
    else cb_knn_tc_kernel<16><<<grid, CB_KNN_THREADS, smem, st>>>(tmq, tme, a);
    const cudaError_t le = cudaGetLastError();
    return le == cudaSuccess ? 0 : (int)le;
}
