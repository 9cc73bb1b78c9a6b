// Device-side building blocks of one tree level: leaf-index update, streaming histogram accumulation,
// slot reduction + sibling subtraction + bin scan + split scoring, and best-split selection.
// They are used twice: by the stand-alone kernels (one launch per step; also the path that the
// NCCL-reduce-scatter baseline uses) and by the fused cooperative level kernel in cb_fused.cu.
//
// Behaviour reproduced from the reference (not its code): histogram contents and the sibling subtraction
// (catboost/cuda/methods/kernel/pointwise_hist2.cu:39-75), the bin prefix scan
// (split_properties_helpers.cuh:112-200), score functions (score_calcers.cuh:11-188), gain tie-break by
// (score, feature, bin) (catboost/cuda/gpu_data/gpu_structures.h:80-94) and the per-document leaf bit
// (catboost/cuda/gpu_data/kernel/split.cu:179).
#pragma once
#include "cb_common.cuh"
#include "cb_comm.cuh"

#define CB_HIST_MAX_DOCS_PER_TILE (1 << 19)

enum CbScoreFn : int { CB_SCORE_COSINE = 0, CB_SCORE_L2 = 1, CB_SCORE_SOLAR = 2, CB_SCORE_LOO = 3, CB_SCORE_SAT = 4 };

struct CbSplit {       // one record per (tree, level)
    int feature;       // flat feature index of the binned store (-1 = no split found)
    int bin;           // go right when bin(doc) > bin  (one-hot: bin(doc) == bin)
    float score;
    int flags;         // bit0 = one-hot comparison
};

struct CbData {        // the binned training shard of this rank
    const uint32_t* bins;
    long long npad;
    long long n;
    int G;
    int F;
    const int* feat_off;            // [F+1], multiples of 4
    const int* feat_nb;             // [F] real bin count (borders + 1), <= 256
    const unsigned char* feat_onehot;   // [F] or null
    const float* feat_weight;       // [F] gain multiplier (0 = ignored feature) or null
    int TB;                         // feat_off[F]
};

struct CbBundle {
    int g0, gcnt;      // feature groups g0 .. g0 + gcnt - 1
    int B;             // bins per feature inside the tile (multiple of 4, >= the widest feature of the bundle)
    int C;             // replicas of a cell (power of two)
    int spp;           // slots (leaves) per pass
    int npass;
    int nK;            // document chunks of this bundle
};

struct CbHistArgs {
    CbData d;
    const unsigned short* leaf;
    const float* stats;      // [S][npad]
    int S;
    int level;               // slots = level == 0 ? 1 : 1 << (level-1); slot = leaf & (slots-1)
    const unsigned int* small_mask;   // bit p set: the RIGHT child of parent p is the one accumulated
    int slots_per_pass;
    int B;                   // shared-memory bin stride per feature (max feat_nb rounded up to 4... <= 256)
    float* out;              // [slots][S][TB]  (zeroed by the caller)
    // Non-symmetric trees (depthwise / lossguide): leaf holds a node id and slot_table[node] is the slot the
    // document is accumulated into (-1 = skip).  When slot_table is set, level/small_mask are ignored.
    const short* slot_table;
    int nslots_table;
    // When `priv` is set the block does not add into `out`: it dumps its shared-memory tile, as is, into its own
    // region priv[item][slot][s][j][B] (item = chunk * G + group) with plain coalesced stores; a later phase sums
    // the chunks (cb_reduce_chunks).  No global atomics, no zero-fill of `out`, and a deterministic result.
    float* priv;
    // Fixed-point accumulation (needs `priv`): statmax[s] = max |stats[s][i]| of this iteration.  A value is scaled
    // to 24 signed bits and split into a signed high part (q >> 12) and an unsigned low part (q & 4095), each added
    // with a native 32-bit integer shared-memory atomic; fp32 shared atomics are compare-and-swap loops and were
    // measured 2x slower for twice fewer operations.  The sum is exact in integers (better than fp32 accumulation)
    // as long as a block sees at most 2^19 documents per tile, which cb_hist_chunks guarantees.
    const float* statmax;
    int nK;        // document chunks per feature group chosen by the host (0 = derive from the grid)
    int copies;    // power of two <= 8: replicas of every fixed-point cell, lane l uses replica l & (copies-1)
    // Dynamic work distribution (optional): work[G] hands out whole (group, chunk) items when there are more items than
    // blocks.  Zero on entry; the fused kernel clears it again after the level.
    unsigned int* work;
    int narrow;    // two-statistic fixed-point path: 1 = single int32 cells (scale limited by the tile's documents)
    int bundle;    // with narrow cells: feature groups accumulated together by one block (<= 8), 0 = one group per block
    // Leaf update fused into the bundled histogram pass: when set, `leaf` still holds the indices of two levels ago and
    // *prev_split is the split chosen at level - 1.  Every block works the new bit out for the documents it streams
    // (it has their bin words in registers anyway); the block of bundle 0 in the first slot pass writes the leaf back.
    // Blocks that read a leaf word before or after that store get the same result, because setting the bit twice
    // changes nothing.
    // The kernel arguments are never modified on the device, so the split is named by where it will be:
    // prev_splits[*prev_iter * prev_depth + level - 1]; prev_splits == nullptr switches the fusion off.
    // Dominant-bin skipping (bundled path): domw[g] packs, for the four features of group g, the bin that most of their
    // documents fall into (255 = none).  Documents are not accumulated into that bin; every slot keeps lane-replicated
    // totals of its two statistics instead and the bin is restored as total - sum of the other bins before the tile
    // is dumped.  On sparse data most (document, feature) pairs hit the dominant bin, so this removes most shared-memory
    // atomics and the hot spot they create.  nullptr = off.
    const unsigned int* domw;
    // Bundle table of the bundled path (nullptr = uniform bundles of `bundle` groups with B bins and `copies` replicas).
    // Feature groups differ in their number of bins (128-border float columns next to 16-bin CTR columns or binary
    // one-hot columns), and the shared-memory tile is what limits how many leaves one pass over the documents can take:
    // every bundle therefore has its own bin stride, replica count and slots per pass, and the work items
    // (bundle, document chunk, slot pass) are listed explicitly, heaviest first.
    const CbBundle* btab;
    const int2* bitems;         // x = bundle | pass << 16, y = document chunk
    int nbitems;
    const int* gchunks;         // [G] document chunks of the bundle every group belongs to
    const CbSplit* prev_splits;
    const int* prev_iter;
    int prev_depth;
    unsigned short* leaf_rw;
};

__device__ __forceinline__ int cb_hist_nslots(const CbHistArgs& a) {
    return a.slot_table ? a.nslots_table : (a.level == 0 ? 1 : (1 << (a.level - 1)));
}

// ------------------------------------------------------------------------------------------------------
// Leaf update: leaf |= bit << (level) for the split chosen at `level`.
__device__ __forceinline__ void cb_update_leaf_range(const CbData& d, unsigned short* leaf, CbSplit sp, int level,
                                                     long long tid, long long nthreads) {
    if (sp.feature < 0) return;
    const uint32_t* col = d.bins + (long long)(sp.feature >> 2) * d.npad;
    const int sh = (sp.feature & 3) * 8;
    const bool onehot = sp.flags & 1;
    const long long n4 = (d.n + 3) >> 2;
    for (long long q = tid; q < n4; q += nthreads) {
        const long long i = q << 2;
        uint4 w = *reinterpret_cast<const uint4*>(col + i);
        ushort4 lf = *reinterpret_cast<ushort4*>(leaf + i);
        unsigned int b0 = (w.x >> sh) & 255u, b1 = (w.y >> sh) & 255u, b2 = (w.z >> sh) & 255u, b3 = (w.w >> sh) & 255u;
        unsigned int t = (unsigned int)sp.bin;
        unsigned int r0 = onehot ? (b0 == t) : (b0 > t);
        unsigned int r1 = onehot ? (b1 == t) : (b1 > t);
        unsigned int r2 = onehot ? (b2 == t) : (b2 > t);
        unsigned int r3 = onehot ? (b3 == t) : (b3 > t);
        lf.x |= (unsigned short)(r0 << level);
        lf.y |= (unsigned short)(r1 << level);
        lf.z |= (unsigned short)(r2 << level);
        lf.w |= (unsigned short)(r3 << level);
        *reinterpret_cast<ushort4*>(leaf + i) = lf;
    }
}

// ------------------------------------------------------------------------------------------------------
// Histogram accumulation of one (feature group, document chunk, slot pass) into shared memory + flush.
// sh layout: [slot][s][j][B]; S is a run-time value (2 for pointwise losses, K+1 for K-class losses).
static __device__ void cb_hist_item(const CbHistArgs& a, float* sh, int g, long long item, long long d_begin,
                             long long d_end, int slot_begin, int slot_count) {
    const int B = a.B;
    const int S = a.S;
    const int total = slot_count * S * 4 * B;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0.0f;
    __syncthreads();

    const uint32_t* bg = a.d.bins + (long long)g * a.d.npad;
    const int level = a.level;
    const int nslots = cb_hist_nslots(a);
    const unsigned int pmask = (unsigned int)(nslots - 1);
    const int slot_stride = S * 4 * B;
    for (long long i = d_begin + (long long)threadIdx.x * 4; i < d_end; i += (long long)blockDim.x * 4) {
        const uint4 w = *reinterpret_cast<const uint4*>(bg + i);
        const ushort4 lf = *reinterpret_cast<const ushort4*>(a.leaf + i);
        const unsigned int wv[4] = {w.x, w.y, w.z, w.w};
        const unsigned int lv[4] = {lf.x, lf.y, lf.z, lf.w};
        int off[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int slot = 0;
            bool take = (i + k) < a.d.n;
            if (a.slot_table) {
                slot = a.slot_table[lv[k]];
                take = take && (slot >= 0);
            } else if (level > 0) {
                const unsigned int p = lv[k] & pmask;
                const unsigned int right = (lv[k] >> (level - 1)) & 1u;
                const unsigned int want = (a.small_mask[p >> 5] >> (p & 31)) & 1u;
                take = take && (right == want);
                slot = (int)p;
            }
            slot -= slot_begin;
            off[k] = (take && (unsigned)slot < (unsigned)slot_count) ? slot * slot_stride : -1;
        }
        for (int s = 0; s < S; ++s) {
            const float4 t = *reinterpret_cast<const float4*>(a.stats + (long long)s * a.d.npad + i);
            const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (off[k] >= 0) {
                    float* base = sh + off[k] + s * 4 * B;
#pragma unroll
                    for (int j = 0; j < 4; ++j) atomicAdd(base + j * B + ((wv[k] >> (8 * j)) & 255u), tv[k]);
                }
            }
        }
    }
    __syncthreads();
    if (a.priv) {
        float4* dst = reinterpret_cast<float4*>(a.priv + ((size_t)item * nslots + slot_begin) * slot_stride);
        const float4* src = reinterpret_cast<const float4*>(sh);
        for (int i = threadIdx.x; i < (total >> 2); i += blockDim.x) dst[i] = src[i];
        __syncthreads();
        return;
    }
    // flush (skip zeros: most (slot, bin) cells of a chunk are empty at deep levels)
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const float v = sh[i];
        if (v != 0.0f) {
            const int bin = i % B;
            const int r = i / B;
            const int j = r & 3;
            const int s = (r >> 2) % S;
            const int slot = (r >> 2) / S;
            const int f = g * 4 + j;
            if (f < a.d.F && bin < a.d.feat_nb[f]) {
                atomicAdd(a.out + ((size_t)(slot_begin + slot) * S + s) * a.d.TB + a.d.feat_off[f] + bin, v);
            }
        }
    }
    __syncthreads();
}

// Single-int32-cell variant of cb_hist_item for any number of statistics, used by the stand-alone histogram launcher
// (general learner: multi-class, depthwise, lossguide, ranking).  Statistic s is scaled by qmax / statmax[s] with
// qmax = (2^31 - 1) / documents of this chunk (capped at 2^23 - 1), rounded to nearest and added with a native integer
// atomic (fp32 shared atomics are compare-and-swap loops); the flush converts back and adds into `out` with global
// float atomics.  sh layout: int [slot][s][j][B].
static __device__ void cb_hist_item_n(const CbHistArgs& a, int* sh, int g, long long d_begin, long long d_end,
                                      int slot_begin, int slot_count) {
    const int B = a.B;
    const int S = a.S;
    const int total = slot_count * S * 4 * B;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    const uint32_t* bg = a.d.bins + (long long)g * a.d.npad;
    const int level = a.level;
    const int nslots = cb_hist_nslots(a);
    const unsigned int pmask = (unsigned int)(nslots - 1);
    const int slot_stride = S * 4 * B;
    const float qmax = fminf(8388607.0f, floorf(2147483647.0f / (float)max(1ll, d_end - d_begin)) - 1.0f);
    for (long long i = d_begin + (long long)threadIdx.x * 4; i < d_end; i += (long long)blockDim.x * 4) {
        const uint4 w = *reinterpret_cast<const uint4*>(bg + i);
        const ushort4 lf = *reinterpret_cast<const ushort4*>(a.leaf + i);
        const unsigned int wv[4] = {w.x, w.y, w.z, w.w};
        const unsigned int lv[4] = {lf.x, lf.y, lf.z, lf.w};
        int off[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int slot = 0;
            bool take = (i + k) < a.d.n;
            if (a.slot_table) {
                slot = a.slot_table[lv[k]];
                take = take && (slot >= 0);
            } else if (level > 0) {
                const unsigned int p = lv[k] & pmask;
                const unsigned int right = (lv[k] >> (level - 1)) & 1u;
                const unsigned int want = (a.small_mask[p >> 5] >> (p & 31)) & 1u;
                take = take && (right == want);
                slot = (int)p;
            }
            slot -= slot_begin;
            off[k] = (take && (unsigned)slot < (unsigned)slot_count) ? slot * slot_stride : -1;
        }
        for (int s = 0; s < S; ++s) {
            const float sc = qmax / fmaxf(a.statmax[s], 1e-30f);
            const float4 t = *reinterpret_cast<const float4*>(a.stats + (long long)s * a.d.npad + i);
            const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (off[k] >= 0) {
                    int* base = sh + off[k] + s * 4 * B;
                    const int q = __float2int_rn(tv[k] * sc);
#pragma unroll
                    for (int j = 0; j < 4; ++j) atomicAdd(base + j * B + ((wv[k] >> (8 * j)) & 255u), q);
                }
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int v = sh[i];
        if (v != 0) {
            const int bin = i % B;
            const int r = i / B;
            const int j = r & 3;
            const int s = (r >> 2) % S;
            const int slot = (r >> 2) / S;
            const int f = g * 4 + j;
            if (f < a.d.F && bin < a.d.feat_nb[f]) {
                atomicAdd(a.out + ((size_t)(slot_begin + slot) * S + s) * a.d.TB + a.d.feat_off[f] + bin,
                          (float)v * (fmaxf(a.statmax[s], 1e-30f) / qmax));
            }
        }
    }
    __syncthreads();
}

// Fixed-point variant of cb_hist_item (see CbHistArgs::statmax).  sh layout: int [slot][s][part][j][B], part 0 = high.
// NARROW: one int32 cell per (statistic, feature, bin) whose scale is (2^31 - 1) / (documents of this item), so that the
// cell cannot overflow (12-16 bits per addend); else a signed high / unsigned low pair of 12 + 12 bits (exact).
template <bool NARROW>
static __device__ void cb_hist_item_q(const CbHistArgs& a, int* sh, int g, long long item, long long d_begin,
                                      long long d_end, int slot_begin, int slot_count) {
    const int B = a.B;
    const int S = a.S;
    const int PS = NARROW ? 4 : 8;                  // rows of B cells per (slot, statistic)
    const int total = slot_count * S * PS * B;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0;
    __syncthreads();

    const uint32_t* bg = a.d.bins + (long long)g * a.d.npad;
    const int level = a.level;
    const int nslots = cb_hist_nslots(a);
    const unsigned int pmask = (unsigned int)(nslots - 1);
    const int slot_stride = S * PS * B;
    const float qmax = NARROW ? fminf(8388607.0f, floorf(2147483647.0f / (float)max(d_end - d_begin, 1ll)) - 1.0f) : 8388607.0f;
    for (long long i = d_begin + (long long)threadIdx.x * 4; i < d_end; i += (long long)blockDim.x * 4) {
        const uint4 w = *reinterpret_cast<const uint4*>(bg + i);
        const ushort4 lf = *reinterpret_cast<const ushort4*>(a.leaf + i);
        const unsigned int wv[4] = {w.x, w.y, w.z, w.w};
        const unsigned int lv[4] = {lf.x, lf.y, lf.z, lf.w};
        int off[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int slot = 0;
            bool take = (i + k) < a.d.n;
            if (a.slot_table) {
                slot = a.slot_table[lv[k]];
                take = take && (slot >= 0);
            } else if (level > 0) {
                const unsigned int p = lv[k] & pmask;
                const unsigned int right = (lv[k] >> (level - 1)) & 1u;
                const unsigned int want = (a.small_mask[p >> 5] >> (p & 31)) & 1u;
                take = take && (right == want);
                slot = (int)p;
            }
            slot -= slot_begin;
            off[k] = (take && (unsigned)slot < (unsigned)slot_count) ? slot * slot_stride : -1;
        }
        for (int s = 0; s < S; ++s) {
            const float sc = qmax / fmaxf(a.statmax[s], 1e-30f);
            const float4 t = *reinterpret_cast<const float4*>(a.stats + (long long)s * a.d.npad + i);
            const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (off[k] >= 0) {
                    const int q = __float2int_rn(tv[k] * sc);
                    int* base = sh + off[k] + s * PS * B;
                    if (NARROW) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) atomicAdd(base + j * B + ((wv[k] >> (8 * j)) & 255u), q);
                    } else {
                        const int hi = q >> 12;
                        const unsigned int lo = (unsigned int)q & 4095u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const unsigned int bin = (wv[k] >> (8 * j)) & 255u;
                            atomicAdd(base + j * B + bin, hi);
                            atomicAdd(reinterpret_cast<unsigned int*>(base) + (4 + j) * B + bin, lo);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    // dump as floats into the private region [item][slot][s][j][B]
    const int cells4 = (slot_count * S * 4 * B) >> 2;
    float4* dst = reinterpret_cast<float4*>(a.priv + ((size_t)item * nslots + slot_begin) * (size_t)(S * 4 * B));
    const int B4 = B >> 2;
    for (int c = threadIdx.x; c < cells4; c += blockDim.x) {
        const int b4 = c % B4;
        const int r = c / B4;            // (slot * S + s) * 4 + j
        const int j = r & 3;
        const int ss = r >> 2;           // slot * S + s
        const float inv = fmaxf(a.statmax[ss % S], 1e-30f) / qmax;
        float4 v;
        if (NARROW) {
            const int4 q4 = *reinterpret_cast<const int4*>(sh + (size_t)ss * 4 * B + j * B + b4 * 4);
            v = make_float4((float)q4.x * inv, (float)q4.y * inv, (float)q4.z * inv, (float)q4.w * inv);
        } else {
            const int4 hi = *reinterpret_cast<const int4*>(sh + (size_t)ss * 8 * B + j * B + b4 * 4);
            const uint4 lo = *reinterpret_cast<const uint4*>(sh + (size_t)ss * 8 * B + (4 + j) * B + b4 * 4);
            v.x = fmaf((float)hi.x, 4096.0f * inv, (float)lo.x * inv);
            v.y = fmaf((float)hi.y, 4096.0f * inv, (float)lo.y * inv);
            v.z = fmaf((float)hi.z, 4096.0f * inv, (float)lo.z * inv);
            v.w = fmaf((float)hi.w, 4096.0f * inv, (float)lo.w * inv);
        }
        dst[c] = v;
    }
    __syncthreads();
}

// Two-statistic fixed-point variant with warp-level compaction.  From level 1 on only the lighter child of every
// parent is accumulated, so about half of the documents are skipped; issuing the atomics straight from the streaming
// loop would leave half of the lanes idle in every atomic instruction.  Instead each warp appends its live documents
// (bins word, tile offset, two quantised statistics = 16 bytes) to a small ring in shared memory and drains it 32
// entries at a time, so every atomic instruction runs with all lanes busy.
// sh layout: int hist[slot][2][part][j][B], then uint4 ring[warps][64].
#ifndef CB_UPD_ON
#define CB_UPD_ON true
#endif
#define CB_RING 64
template <bool NARROW>
__device__ __forceinline__ void cb_hist_q_apply(int* sh, int B, int C, int copy, uint4 e) {
    int* base = sh + (int)e.y + copy;
    const int q0 = (int)e.z, q1 = (int)e.w;
    if (NARROW) {
        // one 32-bit cell per (statistic, feature, bin): the scale was chosen so that a tile cannot overflow it
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned int bin = (e.x >> (8 * j)) & 255u;
            atomicAdd(base + (j * B + bin) * C, q0);
            atomicAdd(base + ((4 + j) * B + bin) * C, q1);
        }
        return;
    }
    const int h0 = q0 >> 12, h1 = q1 >> 12;
    const unsigned int l0 = (unsigned int)q0 & 4095u, l1 = (unsigned int)q1 & 4095u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned int bin = (e.x >> (8 * j)) & 255u;
        atomicAdd(base + (j * B + bin) * C, h0);
        atomicAdd(reinterpret_cast<unsigned int*>(base) + ((4 + j) * B + bin) * C, l0);
        atomicAdd(base + ((8 + j) * B + bin) * C, h1);
        atomicAdd(reinterpret_cast<unsigned int*>(base) + ((12 + j) * B + bin) * C, l1);
    }
}

// Documents are dealt to the chunks of a group block-cyclically (block = blockDim.x * 4 documents): chunk k takes
// blocks k, k + nK, k + 2 nK, ... so that every chunk sees the same mix of the data and the blocks finish together.
//
// NARROW: every cell is a single int32 (half of the atomics and of the tile).  The fixed-point scale is then limited by
// the number of documents a cell can receive in this tile: qmax = (2^31 - 1) / (documents per chunk / replicas), about
// 14 bits at 250K documents per chunk with two replicas.  Rounding is to nearest, so the error of a bin sum is an
// unbiased random walk of at most half a quantum per document -- far below the sampling noise of the sum itself; the
// leaf values never come from these histograms (the leaf pass re-accumulates exact derivatives).
template <bool NARROW>
static __device__ void cb_hist_item_q2(const CbHistArgs& a, int* sh, int g, long long item, int chunk, int nK,
                                       int slot_begin, int slot_count) {
    const int B = a.B;
    const int C = a.copies > 0 ? a.copies : 1;
    constexpr int PL = NARROW ? 8 : 16;      // int planes per slot
    const int total = slot_count * PL * B * C;
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint4* ring = reinterpret_cast<uint4*>(sh + ((total + 3) & ~3)) + warp * CB_RING;
    const uint32_t* bg = a.d.bins + (long long)g * a.d.npad;
    const float* st0 = a.stats;
    const float* st1 = a.stats + a.d.npad;
    const int level = a.level;
    const int nslots = cb_hist_nslots(a);
    const unsigned int pmask = (unsigned int)(nslots - 1);
    const int slot_stride = PL * B * C;
    const int copy = lane & (C - 1);
    float qmax = 8388607.0f;
    if (NARROW) {
        const long long blkd = (long long)blockDim.x * 4;
        const long long nblk = (a.d.n + blkd - 1) / blkd;
        const long long cap = ((nblk + nK - 1) / nK) * blkd / C + 64;     // documents one replica of a cell can see
        qmax = fminf(qmax, floorf(2147483647.0f / (float)cap) - 1.0f);
    }
    const float sc0 = qmax / fmaxf(a.statmax[0], 1e-30f);
    const float sc1 = qmax / fmaxf(a.statmax[1], 1e-30f);
    const unsigned int lt = (1u << lane) - 1u;
    unsigned int head = 0, tail = 0;
    // Software pipeline: the four loads of the next step are issued before the atomics of the current one, so the
    // DRAM latency of a step overlaps the shared-memory work of the previous step.  All blocks that share a chunk
    // index walk the same documents at the same time, so the leaf / statistic rows are served from L2 to all but one.
    const long long d_end = a.d.n;
    const long long blk = (long long)blockDim.x * 4;
    const long long step = blk * nK;
    const long long ib0 = blk * chunk + (long long)(threadIdx.x & ~31) * 4;
    uint4 nw = make_uint4(0, 0, 0, 0);
    ushort4 nlf = make_ushort4(0, 0, 0, 0);
    float4 ns0 = make_float4(0, 0, 0, 0), ns1 = make_float4(0, 0, 0, 0);
    if (ib0 + lane * 4 < d_end) {
        const long long i = ib0 + lane * 4;
        nw = *reinterpret_cast<const uint4*>(bg + i);
        nlf = *reinterpret_cast<const ushort4*>(a.leaf + i);
        ns0 = *reinterpret_cast<const float4*>(st0 + i);
        ns1 = *reinterpret_cast<const float4*>(st1 + i);
    }
    for (long long ib = ib0; ib < d_end; ib += step) {
        const long long i = ib + lane * 4;
        const uint4 w = nw;
        const ushort4 lf = nlf;
        const float4 s0 = ns0, s1 = ns1;
        const bool valid = i < d_end;
        {
            const long long in = i + step;
            if (in < d_end) {
                nw = *reinterpret_cast<const uint4*>(bg + in);
                nlf = *reinterpret_cast<const ushort4*>(a.leaf + in);
                ns0 = *reinterpret_cast<const float4*>(st0 + in);
                ns1 = *reinterpret_cast<const float4*>(st1 + in);
            }
        }
        const unsigned int wv[4] = {w.x, w.y, w.z, w.w};
        const unsigned int lv[4] = {lf.x, lf.y, lf.z, lf.w};
        const float v0[4] = {s0.x, s0.y, s0.z, s0.w};
        const float v1[4] = {s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int slot = 0;
            bool take = valid && (i + k) < a.d.n;
            if (a.slot_table) {
                slot = a.slot_table[lv[k]];
                take = take && (slot >= 0);
            } else if (level > 0) {
                const unsigned int p = lv[k] & pmask;
                const unsigned int right = (lv[k] >> (level - 1)) & 1u;
                const unsigned int want = (a.small_mask[p >> 5] >> (p & 31)) & 1u;
                take = take && (right == want);
                slot = (int)p;
            }
            slot -= slot_begin;
            take = take && ((unsigned)slot < (unsigned)slot_count);
            const unsigned int m = __ballot_sync(0xffffffffu, take);
            if (take) {
                ring[(tail + __popc(m & lt)) & (CB_RING - 1)] =
                    make_uint4(wv[k], (unsigned int)(slot * slot_stride), (unsigned int)__float2int_rn(v0[k] * sc0),
                               (unsigned int)__float2int_rn(v1[k] * sc1));
            }
            tail += __popc(m);
            __syncwarp();
            if (tail - head >= 32u) {
                cb_hist_q_apply<NARROW>(sh, B, C, copy, ring[(head + lane) & (CB_RING - 1)]);
                head += 32u;
                __syncwarp();
            }
        }
    }
    if ((unsigned int)lane < tail - head) cb_hist_q_apply<NARROW>(sh, B, C, copy, ring[(head + lane) & (CB_RING - 1)]);
    __syncthreads();
    // dump as floats into the private region [item][slot][s][j][B]
    const int cells4 = (slot_count * 8 * B) >> 2;
    float4* dst = reinterpret_cast<float4*>(a.priv + ((size_t)item * nslots + slot_begin) * (size_t)(8 * B));
    const int B4 = B >> 2;
    const float inv0 = fmaxf(a.statmax[0], 1e-30f) / qmax;
    const float inv1 = fmaxf(a.statmax[1], 1e-30f) / qmax;
    for (int c = threadIdx.x; c < cells4; c += blockDim.x) {
        const int b4 = c % B4;
        const int r = c / B4;            // (slot * 2 + s) * 4 + j
        const int j = r & 3;
        const int ss = r >> 2;           // slot * 2 + s
        const float inv = (ss & 1) ? inv1 : inv0;
        if (NARROW) {
            long long q4[4] = {0, 0, 0, 0};      // the replicas together may exceed 32 bits
            const int* pq = sh + ((size_t)ss * 4 * B + j * B + b4 * 4) * C;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                for (int cc = 0; cc < C; ++cc) q4[q] += pq[q * C + cc];
            dst[c] = make_float4((float)q4[0] * inv, (float)q4[1] * inv, (float)q4[2] * inv, (float)q4[3] * inv);
            continue;
        }
        int hi[4] = {0, 0, 0, 0};
        unsigned int lo[4] = {0u, 0u, 0u, 0u};
        const int* ph = sh + ((size_t)ss * 8 * B + j * B + b4 * 4) * C;
        const int* pl = sh + ((size_t)ss * 8 * B + (4 + j) * B + b4 * 4) * C;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            for (int cc = 0; cc < C; ++cc) { hi[q] += ph[q * C + cc]; lo[q] += (unsigned int)pl[q * C + cc]; }
        float4 v;
        v.x = fmaf((float)hi[0], 4096.0f * inv, (float)lo[0] * inv);
        v.y = fmaf((float)hi[1], 4096.0f * inv, (float)lo[1] * inv);
        v.z = fmaf((float)hi[2], 4096.0f * inv, (float)lo[2] * inv);
        v.w = fmaf((float)hi[3], 4096.0f * inv, (float)lo[3] * inv);
        dst[c] = v;
    }
    __syncthreads();
}

// Bundled variant of the single-cell fixed-point path: one block accumulates `gcnt` consecutive feature groups of its
// documents in the same pass, so everything that is per document -- the leaf / statistic loads, the lighter-child
// test, the quantisation and the warp compaction -- is paid once for up to 32 features instead of once per 4.
// (Measured on 10.5M x 28, level 3: streaming loads 131 us, compaction 133 us, atomics 42 us with one group per block.)
// Every lane takes V consecutive documents per step (V = 1 for wide bundles, 2 otherwise, vector loads); the loads of
// the next step are issued before the current step is processed.  Measured alone on 10.5M x 28, level 3, all 7 groups
// in one bundle: loads 95 us, compaction 11 us, atomics 70 us (4.2e12 shared atomics/s, close to one per bank and clock).
// sh layout: int tile[slot][group][statistic][j][B][C], then uint32 ring[warp][3 + gcnt][CB_RING] (word-major, so
// that lanes touch consecutive banks).
#ifndef CB_BUNDLE_V
#define CB_BUNDLE_V(GMAX) ((GMAX) > 4 ? 1 : 2)     // documents per lane and step: bounded by the 64-register budget
#endif
#ifndef CB_BUNDLE_PF
#define CB_BUNDLE_PF 1       // 1 = keep the next step's loads in registers while the current step is processed
#endif
// One reduction into shared memory through a 32-bit shared-window address: no 64-bit pointer arithmetic.
__device__ __forceinline__ void cb_red_shared(unsigned int addr, int v) {
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Tile layout of the bundled path: int tile[slot][group][statistic][j][B][C].  sbase = shared-window address of the
// tile; cst4 = bytes per bin (4 C), fst4 = bytes per feature (B * 4 C), sst4 = bytes between the two statistics of a
// cell (4 features), gst4 = bytes per group.  (Keeping the two statistics of a cell next to each other would save the
// second address but halves the banks one reduction can spread over: measured 357 us against 281 us at level 0 of
// 10.5M x 28.)
template <int GMAX, bool SKIP>
__device__ __forceinline__ void cb_hist_bundle_drain(unsigned int sbase, const unsigned int* ring, int e, int gcnt,
                                                     unsigned int gst4, unsigned int fst4, unsigned int cst4, int copy,
                                                     const unsigned int* sdom, int* tot, int lane) {
    const unsigned int head_word = ring[e];          // SKIP: slot << 20 | tile offset (ints) of the slot; else the offset
    unsigned int ag = sbase + (((SKIP ? (head_word & 0xFFFFFu) : head_word) + (unsigned int)copy) << 2);
    const unsigned int sst4 = gst4 >> 1;
    const int q0 = (int)ring[CB_RING + e], q1 = (int)ring[2 * CB_RING + e];
    if (SKIP) {
        int* t = tot + (int)(head_word >> 20) * 64 + lane;
        atomicAdd(t, q0);
        atomicAdd(t + 32, q1);
    }
#pragma unroll
    for (int gl = 0; gl < GMAX; ++gl) {
        if (gl < gcnt) {
            const unsigned int w = ring[(3 + gl) * CB_RING + e];
            const unsigned int eq = SKIP ? __vcmpeq4(w, sdom[gl]) : 0u;
            unsigned int af = ag;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (!(SKIP && ((eq >> (8 * j)) & 1u))) {
                    const unsigned int addr = af + ((w >> (8 * j)) & 255u) * cst4;
                    cb_red_shared(addr, q0);
                    cb_red_shared(addr + sst4, q1);
                }
                af += fst4;
            }
            ag += gst4;
        }
    }
}

template <int V> struct CbVec;
template <> struct CbVec<1> { typedef unsigned int U; typedef unsigned short H; typedef float F; };
template <> struct CbVec<2> { typedef uint2 U; typedef ushort2 H; typedef float2 F; };
template <> struct CbVec<4> { typedef uint4 U; typedef ushort4 H; typedef float4 F; };

// The bin words of gcnt groups and the leaf / statistic values of V consecutive documents starting at i (i < n; the
// padded length is a multiple of 256, so a vector never straddles the end of the arrays).
template <int GMAX, int V>
__device__ __forceinline__ void cb_bundle_load(const uint32_t* bg, long long npad, const unsigned short* leaf,
                                               const float* st0, const float* st1, long long i, int gcnt,
                                               unsigned int (&w)[GMAX][V], unsigned int (&lf)[V], float (&s0)[V],
                                               float (&s1)[V]) {
    typedef typename CbVec<V>::U UV;
    typedef typename CbVec<V>::H HV;
    typedef typename CbVec<V>::F FV;
#pragma unroll
    for (int gl = 0; gl < GMAX; ++gl) {
        if (gl < gcnt) {
            const UV x = *reinterpret_cast<const UV*>(bg + gl * npad + i);
            const unsigned int* xp = reinterpret_cast<const unsigned int*>(&x);
#pragma unroll
            for (int k = 0; k < V; ++k) w[gl][k] = xp[k];
        }
    }
    const HV l = *reinterpret_cast<const HV*>(leaf + i);
    const FV f0 = *reinterpret_cast<const FV*>(st0 + i);
    const FV f1 = *reinterpret_cast<const FV*>(st1 + i);
    const unsigned short* lp = reinterpret_cast<const unsigned short*>(&l);
    const float* p0 = reinterpret_cast<const float*>(&f0);
    const float* p1 = reinterpret_cast<const float*>(&f1);
#pragma unroll
    for (int k = 0; k < V; ++k) { lf[k] = lp[k]; s0[k] = p0[k]; s1[k] = p1[k]; }
}

template <int GMAX, bool UPD, bool SKIP>
static __device__ void cb_hist_bundle(const CbHistArgs& a, int* sh, int g0, int gcnt, int chunk, int nK,
                                      int slot_begin, int slot_count, int B, int C) {
    constexpr int V = CB_BUNDLE_V(GMAX);
    const int cs = 31 - __clz(C);                // log2(C): shift of a (j, bin) cell index to ints
    const int gstride = 2 * 4 * B * C;
    const int slot_stride = gcnt * gstride;
    const int total = slot_count * slot_stride;
    // SKIP: per-slot totals [slot][2][32 lane copies] behind the rings of all warps
    int* tot = sh + ((total + 3) & ~3) + (int)(blockDim.x >> 5) * (3 + gcnt) * CB_RING;
    __shared__ unsigned int s_dom[8];
    for (int i = threadIdx.x; i < total; i += blockDim.x) sh[i] = 0;
    if (SKIP) {
        for (int i = threadIdx.x; i < slot_count * 64; i += blockDim.x) tot[i] = 0;
        if (threadIdx.x < 8) s_dom[threadIdx.x] = threadIdx.x < gcnt ? a.domw[g0 + threadIdx.x] : 0xFFFFFFFFu;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int* ring = reinterpret_cast<unsigned int*>(sh + ((total + 3) & ~3)) + warp * (3 + gcnt) * CB_RING;
    const uint32_t* bg = a.d.bins + (long long)g0 * a.d.npad;
    const long long npad = a.d.npad;
    const float* st0 = a.stats;
    const float* st1 = a.stats + npad;
    const int level = a.level;
    const int nslots = cb_hist_nslots(a);
    const unsigned int pmask = (unsigned int)(nslots - 1);
    const int copy = lane & (C - 1);
    const unsigned int sbase = (unsigned int)__cvta_generic_to_shared(sh);
    const unsigned int cst4 = 4u << cs, fst4 = (unsigned int)B * cst4, gst4 = 8u * fst4;
    const long long d_end = a.d.n;
    const long long blk = (long long)blockDim.x * V;
    float qmax = 8388607.0f;
    {
        const long long nblk = (d_end + blk - 1) / blk;
        const long long cap = ((nblk + nK - 1) / nK) * blk / C + 64;      // documents one replica of a cell can see
        qmax = fminf(qmax, floorf(2147483647.0f / (float)cap) - 1.0f);
    }
    const float sc0 = qmax / fmaxf(a.statmax[0], 1e-30f);
    const float sc1 = qmax / fmaxf(a.statmax[1], 1e-30f);
    const unsigned int lt = (1u << lane) - 1u;
    unsigned int head = 0, tail = 0;
    const long long step = blk * nK;
    // fused leaf update (see CbHistArgs::prev_splits; UPD is only used when this bundle holds every feature group).
    // upk packs what the inner loop needs: group inside the bundle | byte shift << 8 | bin << 16 | one-hot << 24,
    // or -1 when the previous level found no split.
    int upk = -1;
    if (UPD) {
        const CbSplit psp = a.prev_splits[(long long)(*a.prev_iter) * a.prev_depth + level - 1];
        if (psp.feature >= 0)
            upk = ((psp.feature >> 2) - g0) | (((psp.feature & 3) * 8) << 8) | ((psp.bin & 255) << 16) | ((psp.flags & 1) << 24);
    }
#if CB_BUNDLE_PF
    unsigned int nw[GMAX][V];
    unsigned int nlf[V];
    float ns0[V], ns1[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
#pragma unroll
        for (int gl = 0; gl < GMAX; ++gl) nw[gl][k] = 0u;
        nlf[k] = 0u; ns0[k] = 0.f; ns1[k] = 0.f;
    }
    if (blk * chunk + (long long)threadIdx.x * V < d_end)
        cb_bundle_load<GMAX, V>(bg, npad, a.leaf, st0, st1, blk * chunk + (long long)threadIdx.x * V, gcnt, nw, nlf, ns0, ns1);
#endif
    // i - lane * V is the same in all lanes of a warp, so the loop bound is warp-uniform (ballots inside)
    for (long long i = blk * chunk + (long long)threadIdx.x * V; i - lane * V < d_end; i += step) {
        unsigned int w[GMAX][V];
        unsigned int lf[V];
        float s0[V], s1[V];
#if CB_BUNDLE_PF
#pragma unroll
        for (int k = 0; k < V; ++k) {
#pragma unroll
            for (int gl = 0; gl < GMAX; ++gl) w[gl][k] = nw[gl][k];
            lf[k] = nlf[k]; s0[k] = ns0[k]; s1[k] = ns1[k];
        }
        if (i + step < d_end) cb_bundle_load<GMAX, V>(bg, npad, a.leaf, st0, st1, i + step, gcnt, nw, nlf, ns0, ns1);
#else
        if (i < d_end) cb_bundle_load<GMAX, V>(bg, npad, a.leaf, st0, st1, i, gcnt, w, lf, s0, s1);
#endif
        if (UPD && upk >= 0 && i < d_end) {
            typedef typename CbVec<V>::H HV;
            const int ugl = upk & 255, ush = (upk >> 8) & 255;
            const unsigned int ubin = (unsigned int)(upk >> 16) & 255u;
            HV out;
            unsigned short* op = reinterpret_cast<unsigned short*>(&out);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                unsigned int uw = 0u;
#pragma unroll
                for (int gl = 0; gl < GMAX; ++gl)
                    if (gl == ugl) uw = w[gl][k];
                const unsigned int b = (uw >> ush) & 255u;
                const unsigned int r = (upk >> 24) ? (b == ubin) : (b > ubin);
                lf[k] |= r << (level - 1);
                op[k] = (unsigned short)lf[k];
            }
            if (slot_begin == 0) *reinterpret_cast<HV*>(a.leaf_rw + i) = out;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) {
            bool take = (i + k) < d_end;
            int slot = 0;
            if (a.slot_table) {
                slot = take ? a.slot_table[lf[k]] : -1;
                take = take && (slot >= 0);
            } else if (level > 0) {
                const unsigned int p = lf[k] & pmask;
                const unsigned int right = (lf[k] >> (level - 1)) & 1u;
                const unsigned int want = (a.small_mask[p >> 5] >> (p & 31)) & 1u;
                take = take && (right == want);
                slot = (int)p;
            }
            slot -= slot_begin;
            take = take && ((unsigned)slot < (unsigned)slot_count);
            const unsigned int m = __ballot_sync(0xffffffffu, take);
            if (take) {
                const int e = (int)((tail + __popc(m & lt)) & (CB_RING - 1));
                ring[e] = (unsigned int)(slot * slot_stride) | (SKIP ? ((unsigned int)slot << 20) : 0u);
                ring[CB_RING + e] = (unsigned int)__float2int_rn(s0[k] * sc0);
                ring[2 * CB_RING + e] = (unsigned int)__float2int_rn(s1[k] * sc1);
#pragma unroll
                for (int gl = 0; gl < GMAX; ++gl)
                    if (gl < gcnt) ring[(3 + gl) * CB_RING + e] = w[gl][k];
            }
            tail += __popc(m);
            __syncwarp();
            if (tail - head >= 32u) {
                cb_hist_bundle_drain<GMAX, SKIP>(sbase, ring, (int)((head + lane) & (CB_RING - 1)), gcnt, gst4, fst4, cst4, copy,
                                                 s_dom, tot, lane);
                head += 32u;
                __syncwarp();
            }
        }
    }
    if ((unsigned int)lane < tail - head)
        cb_hist_bundle_drain<GMAX, SKIP>(sbase, ring, (int)((head + lane) & (CB_RING - 1)), gcnt, gst4, fst4, cst4, copy, s_dom,
                                         tot, lane);
    __syncthreads();
    if (SKIP) {
        // restore the skipped bin of every (slot, group, statistic, feature) row: slot total minus the other bins.  The
        // value is spread over the C replicas of the cell so that each stays inside 32 bits.
        const int rows = slot_count * gcnt * 8;
        for (int row = warp; row < rows; row += (int)(blockDim.x >> 5)) {
            const int sj = row & 7, gl = (row >> 3) % gcnt, slot = (row >> 3) / gcnt;
            const unsigned int dbin = (s_dom[gl] >> (8 * (sj & 3))) & 255u;
            if (dbin == 255u) continue;
            const int* src = sh + (size_t)slot * slot_stride + gl * gstride + (((sj >> 2) * 4 + (sj & 3)) * B << cs);
            long long part = 0;
            for (int i = lane; i < B * C; i += 32) part += src[i];
            long long t = tot[slot * 64 + (sj >> 2) * 32 + lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                part += __shfl_xor_sync(0xffffffffu, part, o);
                t += __shfl_xor_sync(0xffffffffu, t, o);
            }
            const long long rest = t - part;
            if (lane < C) {
                int* cell = const_cast<int*>(src) + ((int)dbin << cs) + lane;
                *cell = (int)(rest / C) + (lane == 0 ? (int)(rest % C) : 0);
            }
        }
        __syncthreads();
    }
    // dump as floats into the private regions [chunk * G + group][slot][s][j][a.B]: the region keeps the bin stride of
    // the widest feature of the data set, the tile only has the B bins this bundle needs
    const int B4 = B >> 2;
    const int cells4 = slot_count * gcnt * 8 * B4;
    const float inv0 = fmaxf(a.statmax[0], 1e-30f) / qmax;
    const float inv1 = fmaxf(a.statmax[1], 1e-30f) / qmax;
    for (int c = threadIdx.x; c < cells4; c += blockDim.x) {
        const int b4 = c % B4;
        int r = c / B4;                          // ((slot * gcnt + gl) * 2 + s) * 4 + j: the order of the tile
        const int sj = r & 7;
        r >>= 3;
        const int gl = r % gcnt;
        const int slot = r / gcnt;
        const int* src = sh + (((size_t)(slot * gcnt + gl) * 8 + sj) * B + b4 * 4) * C;
        long long q4[4] = {0, 0, 0, 0};          // the replicas together may exceed 32 bits
#pragma unroll
        for (int q = 0; q < 4; ++q)
            for (int cc = 0; cc < C; ++cc) q4[q] += src[q * C + cc];
        const float inv = (sj & 4) ? inv1 : inv0;
        float* dst = a.priv + (((size_t)chunk * a.d.G + g0 + gl) * nslots + slot_begin + slot) * (size_t)(8 * a.B)
                     + sj * a.B + b4 * 4;
        *reinterpret_cast<float4*>(dst) =
            make_float4((float)q4[0] * inv, (float)q4[1] * inv, (float)q4[2] * inv, (float)q4[3] * inv);
    }
    __syncthreads();
}

__device__ __forceinline__ int cb_hist_chunks(int G, int ncta, long long n, int host_choice = 0) {
    if (host_choice > 0) return host_choice;
    const int by_grid = (ncta >= G) ? (ncta / G) : 1;
    const int by_docs = (int)((n + CB_HIST_MAX_DOCS_PER_TILE - 1) / CB_HIST_MAX_DOCS_PER_TILE);
    return by_grid > by_docs ? by_grid : by_docs;
}

// Static work split used by both launch styles: item -> (group or bundle of groups, chunk).
static __device__ void cb_hist_phase(const CbHistArgs& a, float* sh, int cta, int ncta) {
    const int G = a.d.G;
    const int nK = cb_hist_chunks(G, ncta, a.d.n, a.nK);
    long long per = (a.d.n + nK - 1) / nK;
    per = (per + 3) & ~3ll;
    const int nslots = cb_hist_nslots(a);
    const bool quant2 = a.statmax && a.priv && a.S == 2;      // without private tiles: the stand-alone integer path
    const int gpc = (quant2 && a.narrow && a.bundle > 0) ? a.bundle : 0;      // groups per block, 0 = per-group paths
    const bool table = gpc && a.btab;                          // explicit work list (bundle, slot pass, chunk)
    const int spp = table ? nslots : a.slots_per_pass;         // the work list carries the passes of its bundles itself
    const bool one_pass = spp >= nslots;
    const int nb = gpc ? (G + gpc - 1) / gpc : G;
    const long long items = table ? (long long)a.nbitems : (long long)nb * nK;
    const bool dyn_items = a.work && quant2 && one_pass && items > ncta;     // whole items from one counter
    __shared__ unsigned int s_item;
    for (int sb0 = 0; sb0 < nslots; sb0 += spp) {
        for (long long item = cta;; item += ncta) {
            if (dyn_items) {
                __syncthreads();
                if (threadIdx.x == 0) s_item = atomicAdd(a.work + G, 1u);
                __syncthreads();
                item = s_item;
            }
            if (item >= items) break;
            int sb = sb0, sc = min(spp, nslots - sb0);
            int g = (int)(item % nb);
            long long k = item / nb;
            if (gpc) {
                int g0 = g * gpc, gcnt = min(gpc, G - g0), Bb = a.B, Cb = a.copies > 0 ? a.copies : 1;
                bool whole = gpc >= G;
                int nKb = nK;
                if (table) {
                    const int2 it = a.bitems[item];
                    const CbBundle bd = a.btab[it.x & 0xFFFF];
                    k = it.y;
                    nKb = bd.nK;
                    g0 = bd.g0; gcnt = bd.gcnt; Bb = bd.B; Cb = bd.C;
                    sb = (it.x >> 16) * bd.spp;
                    sc = min(bd.spp, nslots - sb);
                    whole = gcnt >= G && bd.npass == 1;
                }
                int* shi = reinterpret_cast<int*>(sh);
                const bool upd = CB_UPD_ON && a.prev_splits && a.level > 0 && whole;
#define CB_BUNDLE_CALL(GM) do { \
                    if (a.domw) { if (upd) cb_hist_bundle<GM, true, true>(a, shi, g0, gcnt, (int)k, nKb, sb, sc, Bb, Cb); \
                                  else cb_hist_bundle<GM, false, true>(a, shi, g0, gcnt, (int)k, nKb, sb, sc, Bb, Cb); } \
                    else { if (upd) cb_hist_bundle<GM, true, false>(a, shi, g0, gcnt, (int)k, nKb, sb, sc, Bb, Cb); \
                           else cb_hist_bundle<GM, false, false>(a, shi, g0, gcnt, (int)k, nKb, sb, sc, Bb, Cb); } } while (0)
                if (gcnt <= 2) CB_BUNDLE_CALL(2);
                else if (gcnt <= 4) CB_BUNDLE_CALL(4);
                else CB_BUNDLE_CALL(8);
#undef CB_BUNDLE_CALL
                continue;
            }
            const long long b = k * per;
            const long long e = min(a.d.n, b + per);
            const long long it2 = k * G + g;
            if (quant2 && a.narrow) cb_hist_item_q2<true>(a, reinterpret_cast<int*>(sh), g, it2, (int)k, nK, sb, sc);
            else if (quant2) cb_hist_item_q2<false>(a, reinterpret_cast<int*>(sh), g, it2, (int)k, nK, sb, sc);
            else if (a.statmax && !a.priv) { if (b < e) cb_hist_item_n(a, reinterpret_cast<int*>(sh), g, min(b, e), e, sb, sc); }
            else if (a.statmax && a.narrow) cb_hist_item_q<true>(a, reinterpret_cast<int*>(sh), g, it2, min(b, e), e, sb, sc);
            else if (a.statmax) cb_hist_item_q<false>(a, reinterpret_cast<int*>(sh), g, it2, min(b, e), e, sb, sc);
            else if (b < e || a.priv) cb_hist_item(a, sh, g, it2, min(b, e), e, sb, sc);
        }
    }
    if (dyn_items) __syncthreads();
}

// ------------------------------------------------------------------------------------------------------
// Scoring.  One warp (or several, splitting the leaves) per feature; bins in chunks of 32, one per lane.
struct CbScoreArgs {
    CbData d;
    const float* hsrc[CB_MAX_RANKS];   // per-source partial histograms [slots][S][W]; summed in index order
    int nsrc;
    const float* hprev;     // [L/2][S][W] complete histograms of the parent level (level > 0)
    float* hcur;            // [L][S][W]   complete histograms of this level (out)
    int W;                  // row width (floats) of the buffers above
    int col_base;           // buffer column = feat_off[f] - col_base + bin
    int f_begin, f_end;     // features scored by this rank
    int level;
    int S;
    const unsigned int* small_mask;
    float l2;
    int score_fn;
    float random_strength;
    const double* scal;     // [0]=sum w*loss [1]=sum w [2]=sum (w*der)^2 [3]=docs   (this iteration)
    const int* iter_ptr;
    unsigned long long seed;
    float learning_rate;
    unsigned long long* best_key;
    // Several ranks: hsrc[r] holds tagged words (float payload + 32-bit tag per 8 bytes, cb_comm.cuh) that source r
    // stores straight into this rank's arena; a load polls the word until its tag is that of level counter
    // *ll_epoch + 1 (bounded by ll_timeout_ns, then ll_status is set and 0 is used).  ll_epoch == nullptr: hsrc[r] are
    // plain floats.  The counter is advanced by the launch itself only after every score read of the level is done.
    const unsigned long long* ll_epoch;
    long long ll_timeout_ns;
    int* ll_status;
};

__device__ __forceinline__ unsigned int cb_score_tag(const CbScoreArgs& a) {
    return a.ll_epoch ? cb_ll_tag(*a.ll_epoch + 1ull) : 0u;
}

__device__ __forceinline__ float cb_score_src(const CbScoreArgs& a, int r, size_t idx, unsigned int tag) {
    if (tag == 0u) return __ldcg(a.hsrc[r] + idx);
    const unsigned long long* w = reinterpret_cast<const unsigned long long*>(a.hsrc[r]) + idx;
    return __uint_as_float(cb_ll_load(w, tag, a.ll_timeout_ns, a.ll_status, CB_TIMEOUT_HIST_ARRIVE, r));
}

__device__ __forceinline__ void cb_score_add_leaf(int fn, float l2, float s, float w, float& num, float& den) {
    switch (fn) {
        default:
        case CB_SCORE_COSINE: {
            const float mu = (w > 0.0f) ? s / (w + l2) : 0.0f;
            num += s * mu;
            den += w * mu * mu;
            break;
        }
        case CB_SCORE_L2:
            num += (w > 1e-20f) ? s * s / (w + l2) : 0.0f;
            break;
        case CB_SCORE_SOLAR:
            num += (w > 1e-20f) ? s * s * (1.0f + 2.0f * __logf(w + 1.0f)) / w : 0.0f;
            break;
        case CB_SCORE_LOO: {
            float adj = (w > 1.0f) ? w / (w - 1.0f) : 0.0f;
            num += (w > 0.0f) ? adj * adj * s * s / w : 0.0f;
            break;
        }
        case CB_SCORE_SAT: {
            float adj = (w > 2.0f) ? w * (w - 2.0f) / (w * w - 3.0f * w + 1.0f) : 0.0f;
            num += (w > 0.0f) ? adj * s * s / w : 0.0f;
            break;
        }
    }
}

__device__ __forceinline__ float cb_noise_std(const CbScoreArgs& a) {
    if (a.random_strength <= 0.0f) return 0.0f;
    const double docs = a.scal[3];
    if (docs <= 0.0) return 0.0f;
    const double sd = sqrt(a.scal[2] / docs);
    // modelLengthMult = m/(1+m), m = exp(ln N - iteration*learning_rate)
    const double m = exp(log(docs) - (double)(*a.iter_ptr) * a.learning_rate);
    return (float)(a.random_strength * sd * (m / (1.0 + m)));
}

// Scoring is written as short rolled loops over 32-bin chunks with its accumulators in shared memory: a level runs
// this code once, on a handful of warps, straight after a phase that evicted it from the instruction caches, so its
// run time is the number of instruction lines it has to fetch, not the arithmetic.
// Per-warp scratch (floats): num[256], den[256], pw[256] (prefix of the weight column), ps[256] (prefix of a
// derivative column).
#define CB_SCORE_WARP_FLOATS 1024

// Column `st` of leaf l for the 32 bins of chunk c: summed over the sources, completed from the parent when the leaf
// is the sibling that was not accumulated, stored into the complete histogram of this level.
__device__ __forceinline__ float cb_score_load(const CbScoreArgs& a, int l, int p, bool computed, int st, int col0,
                                               int bin, int nb, unsigned int tag) {
    float x = 0.0f;
    if (bin < nb) {
        const size_t idx = ((size_t)p * a.S + st) * a.W + col0 + bin;
        for (int r = 0; r < a.nsrc; ++r) x += cb_score_src(a, r, idx, tag);
        if (!computed) x = a.hprev[idx] - x;
        if (a.hcur) a.hcur[((size_t)l * a.S + st) * a.W + col0 + bin] = x;
    }
    return x;
}

// The same for the up to 8 bins a lane owns (bins lane * bpl + k), with every load issued before the first use.  Used
// when a warp walks many leaves of one feature: there the chain of dependent L2 round trips is what the warp waits for,
// and the longer code is fetched once and reused for every leaf.
__device__ __forceinline__ void cb_score_load8(const CbScoreArgs& a, int l, int p, bool computed, int st, int col0,
                                               int lane, int bpl, int nb, float* x, unsigned int tag) {
    const size_t base = ((size_t)p * a.S + st) * a.W + col0 + lane * bpl;
    const int left = nb - lane * bpl;                  // bins of this lane that exist
    float prev[8];
    if (tag != 0u) {
        // tagged words: peek at all of a source's words first (the loads overlap), then poll the ones not there yet
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            x[k] = 0.0f;
            prev[k] = (k < bpl && k < left && !computed) ? a.hprev[base + k] : 0.0f;
        }
        for (int r = 0; r < a.nsrc; ++r) {
            const unsigned long long* w = reinterpret_cast<const unsigned long long*>(a.hsrc[r]) + base;
            unsigned long long v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = (k < bpl && k < left) ? cb_ll_peek(w + k) : 0ull;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (k < bpl && k < left) {
                    unsigned int pay = (unsigned int)v[k];
                    if ((unsigned int)(v[k] >> 32) != tag)
                        pay = cb_ll_load(w + k, tag, a.ll_timeout_ns, a.ll_status, CB_TIMEOUT_HIST_ARRIVE, r);
                    x[k] += __uint_as_float(pay);
                }
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool ok = k < bpl && k < left;
            x[k] = ok ? __ldcg(a.hsrc[0] + base + k) : 0.0f;
            prev[k] = (ok && !computed) ? a.hprev[base + k] : 0.0f;
        }
        for (int r = 1; r < a.nsrc; ++r) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < bpl && k < left) x[k] += __ldcg(a.hsrc[r] + base + k);
        }
    }
    const size_t obase = ((size_t)l * a.S + st) * a.W + col0 + lane * bpl;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        if (k < bpl && k < left) {
            if (!computed) x[k] = prev[k] - x[k];
            if (a.hcur) a.hcur[obase + k] = x[k];
        }
    }
}

// Score terms of feature f accumulated over the leaves l0, l0 + lstep, ... into sc[0..255] (num) and sc[256..511]
// (den); sc[512..] is scratch.  One warp.
static __device__ void cb_score_accumulate(const CbScoreArgs& a, int f, int l0, int lstep, float* sc) {
    const int lane = threadIdx.x & 31;
    const int nb = a.d.feat_nb[f];
    const int col0 = a.d.feat_off[f] - a.col_base;
    const bool onehot = a.d.feat_onehot && a.d.feat_onehot[f];
    const int S = a.S;
    const int L = 1 << a.level;
    const int half = L >> 1;
    const int bpl = (nb + 31) >> 5;
    const unsigned int tag = cb_score_tag(a);
    float* num = sc;
    float* den = sc + 256;
    float* pw = sc + 512;
    float* ps = sc + 768;
    for (int b = lane; b < 512; b += 32) sc[b] = 0.0f;
    __syncwarp();
    const bool batched = (L / lstep) >= 4 && bpl <= 8;       // several leaves per warp: overlap the loads of a leaf
    for (int l = l0; l < L; l += lstep) {
        int p = 0;
        bool computed = true;
        if (a.level > 0) {
            p = l & (half - 1);
            const unsigned int right = (unsigned int)l >> (a.level - 1);
            computed = (((a.small_mask[p >> 5] >> (p & 31)) & 1u) == right);
        }
        float totw = 0.0f, exw = 0.0f;
        for (int pass = 0; pass < S; ++pass) {           // weight column first, then the derivative columns
            const bool is_w = pass == 0;
            const int c_st = is_w ? S - 1 : pass - 1;
            float* pre = is_w ? pw : ps;
            // lane owns bins [lane * bpl, lane * bpl + bpl): inclusive prefix inside the lane, then one warp scan.
            // (Issuing all loads of the leaf first in an unrolled loop was measured slower: more instruction lines to
            // fetch cost more than the overlapped load latency saved.)
            float run = 0.0f;
            if (batched) {
                float x8[8];
                cb_score_load8(a, l, p, computed, c_st, col0, lane, bpl, nb, x8, tag);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (k < bpl) {
                        run += x8[k];
                        pre[lane * bpl + k] = onehot ? x8[k] : run;
                    }
                }
            } else {
                for (int k = 0; k < bpl; ++k) {
                    const int bin = lane * bpl + k;
                    const float x = cb_score_load(a, l, p, computed, c_st, col0, bin, nb, tag);
                    run += x;
                    pre[bin] = onehot ? x : run;
                }
            }
            float inc = run;
            for (int o = 1; o < 32; o <<= 1) {
                const float t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            const float excl = onehot ? 0.0f : inc - run;
            const float total = __shfl_sync(0xffffffffu, inc, 31);
            if (is_w) { totw = total; exw = excl; continue; }
            for (int k = 0; k < bpl; ++k) {
                const int bin = lane * bpl + k;
                const float slk = excl + ps[bin], wlk = exw + pw[bin];
                float n_ = num[bin], d_ = den[bin];
                cb_score_add_leaf(a.score_fn, a.l2, slk, fmaxf(wlk, 0.0f), n_, d_);
                cb_score_add_leaf(a.score_fn, a.l2, total - slk, fmaxf(totw - wlk, 0.0f), n_, d_);
                num[bin] = n_; den[bin] = d_;
            }
        }
    }
}

// Best candidate of feature f from complete num/den (one warp); borders are bins 0 .. nb-2 (one-hot: every value).
static __device__ void cb_score_finalize(const CbScoreArgs& a, int f, const float* num, const float* den, float noise_std) {
    const int lane = threadIdx.x & 31;
    const int nb = a.d.feat_nb[f];
    const float fw = a.d.feat_weight ? a.d.feat_weight[f] : 1.0f;
    const bool onehot = a.d.feat_onehot && a.d.feat_onehot[f];
    unsigned long long best = 0ull;
    if (fw > 0.0f) {
        const int ncand = onehot ? nb : nb - 1;
        const unsigned long long it = (unsigned long long)(*a.iter_ptr);
        for (int bin = lane; bin < ncand; bin += 32) {
            float sc;
            if (a.score_fn == CB_SCORE_COSINE) sc = (den[bin] > 1e-15f) ? num[bin] * rsqrtf(den[bin] + 1e-10f) : -3.0e38f;
            else sc = num[bin];
            const unsigned int gb = (unsigned int)(a.d.feat_off[f] + bin);
            if (noise_std > 0.0f) {
                const unsigned long long h = cb_mix64(a.seed ^ cb_mix64((it << 8) + a.level) ^ ((unsigned long long)gb * 0x9E3779B97F4A7C15ull));
                sc += cb_normal(h) * noise_std;
            }
            sc *= fw;
            if (sc == sc) {
                const unsigned long long key = ((unsigned long long)cb_float_to_ordered(sc) << 32) | (unsigned long long)(0xFFFFFFFFu - gb);
                best = key > best ? key : best;
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xffffffffu, best, o);
        best = t > best ? t : best;
    }
    if (lane == 0 && best) atomicMax(a.best_key, best);
}

// `red` is scratch shared memory of `red_floats` floats (the histogram tile is no longer needed at this point), at
// least CB_SCORE_WARP_FLOATS per scoring warp.  With fewer features than warps several warps score one feature: they
// split the leaves and the first of them adds the partial terms up, so the per-feature chain of dependent loads is
// L / warps long instead of L.
// noise_in >= 0: the standard deviation of the score noise, already computed by the caller (it only depends on the
// iteration, so the fused kernel computes it while the histogram phase runs); < 0: compute it here.
static __device__ void cb_score_phase(const CbScoreArgs& a, int cta, int ncta, float* red, int red_floats,
                                      unsigned long long* ts = nullptr, float noise_in = -1.0f) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int wpc = min((int)(blockDim.x >> 5), red_floats / CB_SCORE_WARP_FLOATS);    // scoring warps per block
    float noise_std = fmaxf(noise_in, 0.0f);
    if (noise_in < 0.0f && a.random_strength > 0.0f) {
        if (lane == 0) noise_std = cb_noise_std(a);
        noise_std = __shfl_sync(0xffffffffu, noise_std, 0);
    }
    if (ts) ts[0] = cb_globaltimer();
    const int nf = a.f_end - a.f_begin;
    const int L = 1 << a.level;
    if (wpc < 1 || nf <= 0) return;
    // warps per feature: as many as there are idle warps in the grid (power of two, at most one per leaf)
    int wpf = 1;
    while (wpf * 2 <= min(wpc, L) && (long long)nf * wpf * 2 <= (long long)ncta * wpc) wpf *= 2;
    const int fpc = wpc / wpf;                           // features per block and round
    const int slot = warp / wpf, sub = warp - slot * wpf;
    float* sc = red + (size_t)warp * CB_SCORE_WARP_FLOATS;
    for (int fbase = a.f_begin + cta * fpc; fbase < a.f_end; fbase += ncta * fpc) {
        const int f = fbase + slot;
        const bool have = slot < fpc && f < a.f_end;
        if (have) cb_score_accumulate(a, f, sub, wpf, sc);
        if (ts) ts[1] = cb_globaltimer();
        if (wpf > 1) __syncthreads();
        if (have && sub == 0) {
            const int nb = a.d.feat_nb[f];
            for (int w = 1; w < wpf; ++w) {
                const float* o = sc + (size_t)w * CB_SCORE_WARP_FLOATS;
                for (int bin = lane; bin < nb; bin += 32) { sc[bin] += o[bin]; sc[256 + bin] += o[256 + bin]; }
            }
            __syncwarp();
            cb_score_finalize(a, f, sc, sc + 256, noise_std);
        }
        if (wpf > 1) __syncthreads();
    }
    if (ts) ts[2] = cb_globaltimer();
}

// ------------------------------------------------------------------------------------------------------
// Selection.  Message layout (unsigned long long words): [0] = key, [1..] = small-mask words for the next
// level packed two uint32 per word.  CB_SELECT_WORDS bounds the depth: 2^(depth-1) mask bits.
#define CB_SELECT_MAX_MASK_U32 1024     // depth <= 16  ->  2^15 bits = 1024 uint32
#define CB_SELECT_MSG_BYTES (8 + CB_SELECT_MAX_MASK_U32 * 4)

__device__ __forceinline__ int cb_find_feature(const int* feat_off, int F, int gb) {
    int lo = 0, hi = F - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (feat_off[mid] <= gb) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// One block.  Writes this rank's message: key + mask of "right child is the lighter one" per leaf of `level`.
static __device__ void cb_select_local(const CbScoreArgs& a, unsigned long long* msg) {
    __shared__ int s_f, s_bin;
    const unsigned long long key = *a.best_key;
    unsigned int* mask = reinterpret_cast<unsigned int*>(msg + 1);
    const int L = 1 << a.level;
    const int nwords = (L + 31) >> 5;
    if (threadIdx.x == 0) {
        msg[0] = key;
        if (key) {
            const int gb = (int)(0xFFFFFFFFu - (unsigned int)(key & 0xFFFFFFFFull));
            s_f = cb_find_feature(a.d.feat_off, a.d.F, gb);
            s_bin = gb - a.d.feat_off[s_f];
        } else { s_f = -1; s_bin = 0; }
    }
    for (int i = threadIdx.x; i < nwords; i += blockDim.x) mask[i] = 0u;
    __syncthreads();
    if (s_f < 0 || a.hcur == nullptr) return;
    const int f = s_f, bin = s_bin;
    const int nb = a.d.feat_nb[f];
    const int col0 = a.d.feat_off[f] - a.col_base;
    const bool onehot = a.d.feat_onehot && a.d.feat_onehot[f];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int l = warp; l < L; l += nwarps) {
        const float* row = a.hcur + ((size_t)l * a.S + (a.S - 1)) * a.W + col0;
        float wl = 0.0f, wt = 0.0f;
        for (int b = lane; b < nb; b += 32) {
            const float x = row[b];
            wt += x;
            if (onehot ? (b != bin) : (b <= bin)) wl += x;
        }
        wl = cb_warp_sum(wl);
        wt = cb_warp_sum(wt);
        if (lane == 0 && (wt - wl) < wl) atomicOr(&mask[l >> 5], 1u << (l & 31));
    }
}

// One block.  Picks the best of `nmsg` messages (highest key; equal keys are identical candidates) and
// publishes the split record and the small-child mask for the next level.
static __device__ void cb_select_final(const CbData& d, const unsigned long long* const* msgs, int nmsg, int level,
                                CbSplit* split_out, unsigned int* small_mask_out) {
    __shared__ int s_best;
    if (threadIdx.x == 0) {
        unsigned long long bk = 0ull;
        int bi = 0;
        for (int r = 0; r < nmsg; ++r) {
            const unsigned long long k = __ldcg(msgs[r]);
            if (k > bk) { bk = k; bi = r; }
        }
        s_best = bi;
        CbSplit sp;
        if (bk) {
            const int gb = (int)(0xFFFFFFFFu - (unsigned int)(bk & 0xFFFFFFFFull));
            sp.feature = cb_find_feature(d.feat_off, d.F, gb);
            sp.bin = gb - d.feat_off[sp.feature];
            sp.score = cb_ordered_to_float((unsigned int)(bk >> 32));
            sp.flags = (d.feat_onehot && d.feat_onehot[sp.feature]) ? 1 : 0;
        } else {
            sp.feature = -1; sp.bin = 0; sp.score = 0.0f; sp.flags = 0;
        }
        *split_out = sp;
    }
    __syncthreads();
    const unsigned int* mask = reinterpret_cast<const unsigned int*>(msgs[s_best] + 1);
    const int nwords = ((1 << level) + 31) >> 5;
    for (int i = threadIdx.x; i < nwords; i += blockDim.x) small_mask_out[i] = __ldcg(mask + i);
}
