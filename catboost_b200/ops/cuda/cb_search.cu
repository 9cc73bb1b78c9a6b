// Per-leaf best split from complete histograms with any number of derivative columns: the search step of the
// Depthwise / Lossguide / Region grow policies and of multi-dimensional losses.
//
// Behaviour reproduced from the reference (not its code): every leaf gets its own best (feature, border); the statistics
// of the "<=" side are bin prefix sums, one-hot candidates compare a single value
// (catboost/cuda/methods/greedy_subsets_searcher/kernel/compute_scores.cu:56-178, split_properties_helper.cpp), score
// functions as in catboost/cuda/methods/kernel/score_calcers.cuh summed over the derivative columns, candidates with an
// empty side or fewer than min_data_in_leaf documents on a side are skipped
// (greedy_search_helper.cpp:320-700), ties go to the lower (feature, bin).
//
// Two launches: one warp per (leaf, feature) finds that feature's best border; one warp per leaf picks the best
// feature.  The host reads 16 bytes per leaf.
#include "cb_common.cuh"
#include "cb_tree.cuh"

struct CbLeafSearchArgs {
    CbData d;
    const float* hist;       // [nleaf][S][TB]
    int nleaf, S, K;         // K derivative columns, column K = weight, column K + 1 = document count (when S == K + 2)
    float l2;
    int score_fn;
    float noise_std;
    unsigned long long seed; // already mixed with the iteration
    const int* leaf_id;      // [nleaf] node id of every slot (makes the noise independent of the slot order) or null
    const float* fmask;      // [F] 0 = feature not available to this tree (rsm), or null
    float min_data;          // per side, needs the count column; <= 0: off
    float* out_score;        // [nleaf][F]
    int* out_bin;            // [nleaf][F]
    float* out_gain;         // [nleaf][F]
};

// lane owns bins lane * bpl .. lane * bpl + bpl - 1 (bpl <= 8); returns inclusive prefixes in x[], the exclusive prefix
// of the lane's first bin in *excl and the row total.
__device__ __forceinline__ float cb_ls_scan(const float* row, int nb, int bpl, int lane, float* x, float* excl) {
    float run = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int b = lane * bpl + k;
        const float v = (k < bpl && b < nb) ? __ldg(row + b) : 0.0f;
        x[k] = v;
        run += v;
    }
    float inc = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    *excl = inc - run;
    return __shfl_sync(0xffffffffu, inc, 31);
}

__global__ void __launch_bounds__(256) cb_leaf_search_kernel(CbLeafSearchArgs a) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long total = (long long)a.nleaf * a.d.F;
    if (warp >= total) return;
    const int leaf = (int)(warp / a.d.F), f = (int)(warp % a.d.F);
    const int nb = a.d.feat_nb[f];
    const int col0 = a.d.feat_off[f];
    const bool onehot = a.d.feat_onehot && a.d.feat_onehot[f];
    const float fw = (a.d.feat_weight ? a.d.feat_weight[f] : 1.0f) * (a.fmask ? a.fmask[f] : 1.0f);
    const int ncand = onehot ? nb : nb - 1;
    const int bpl = (nb + 31) >> 5;
    const float* h = a.hist + (size_t)leaf * a.S * a.d.TB + col0;
    float best = -INFINITY, best_gain = 0.0f;
    int best_bin = -1;
    if (fw > 0.0f && ncand > 0 && bpl <= 8) {
        float x[8], excl;
        // weight column: left weights per candidate
        float wl[8], wtot;
        wtot = cb_ls_scan(h + (size_t)a.K * a.d.TB, nb, bpl, lane, x, &excl);
        {
            float run = excl;
#pragma unroll
            for (int k = 0; k < 8; ++k) { run += x[k]; wl[k] = onehot ? x[k] : run; }
        }
        // one-hot: the "left" side of value v is every other value, as in the level-wise searcher
        bool ok[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float l = onehot ? wtot - wl[k] : wl[k];
            const float r = wtot - l;
            wl[k] = l;
            ok[k] = (k < bpl) && (lane * bpl + k < ncand) && l > 0.0f && r > 0.0f;
        }
        if (a.min_data > 0.0f && a.S > a.K + 1) {
            float ctot = cb_ls_scan(h + (size_t)(a.K + 1) * a.d.TB, nb, bpl, lane, x, &excl);
            float run = excl;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                run += x[k];
                const float cl = onehot ? ctot - x[k] : run;
                ok[k] = ok[k] && cl >= a.min_data && (ctot - cl) >= a.min_data;
            }
        }
        float num[8], den[8], l2n[8], parent = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) { num[k] = 0.0f; den[k] = 0.0f; l2n[k] = 0.0f; }
        for (int c = 0; c < a.K; ++c) {
            const float stot = cb_ls_scan(h + (size_t)c * a.d.TB, nb, bpl, lane, x, &excl);
            parent += stot * stot / (fmaxf(wtot, 0.0f) + a.l2);
            float run = excl;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                run += x[k];
                const float sl = onehot ? stot - x[k] : run;
                const float sr = stot - sl;
                const float wL = fmaxf(wl[k], 0.0f), wR = fmaxf(wtot - wl[k], 0.0f);
                cb_score_add_leaf(a.score_fn, a.l2, sl, wL, num[k], den[k]);
                cb_score_add_leaf(a.score_fn, a.l2, sr, wR, num[k], den[k]);
                l2n[k] += sl * sl / (wL + a.l2) + sr * sr / (wR + a.l2);
            }
        }
        const unsigned long long lid = (unsigned long long)(a.leaf_id ? a.leaf_id[leaf] : leaf);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (!ok[k]) continue;
            const int bin = lane * bpl + k;
            float sc = (a.score_fn == CB_SCORE_COSINE) ? ((den[k] > 1e-15f) ? num[k] * rsqrtf(den[k] + 1e-10f) : -3.0e38f) : num[k];
            if (a.noise_std > 0.0f) {
                const unsigned long long hsh = cb_mix64(a.seed ^ cb_mix64(lid * 0x9E3779B97F4A7C15ull + (unsigned long long)(col0 + bin)));
                sc += cb_normal(hsh) * a.noise_std;
            }
            sc *= fw;
            if (sc == sc && (sc > best || (sc == best && bin < best_bin))) { best = sc; best_bin = bin; best_gain = l2n[k] - parent; }
        }
    }
    // warp argmax, ties to the lower bin
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, best, o);
        const int ob = __shfl_xor_sync(0xffffffffu, best_bin, o);
        const float og = __shfl_xor_sync(0xffffffffu, best_gain, o);
        const bool take = (ob >= 0) && (best_bin < 0 || os > best || (os == best && ob < best_bin));
        if (take) { best = os; best_bin = ob; best_gain = og; }
    }
    if (lane == 0) {
        a.out_score[warp] = best_bin >= 0 ? best : -INFINITY;
        a.out_bin[warp] = best_bin;
        a.out_gain[warp] = best_gain;
    }
}

// One warp per leaf: best feature (ties to the lower feature).  best[leaf] = {score, feature, bin, gain} as 4 x 32 bits.
__global__ void __launch_bounds__(256) cb_leaf_search_pick_kernel(const float* score, const int* bin, const float* gain,
                                                                  int nleaf, int F, float* best) {
    const int lane = threadIdx.x & 31;
    const int leaf = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (leaf >= nleaf) return;
    float bs = -INFINITY, bg = 0.0f;
    int bf = -1, bb = -1;
    for (int f = lane; f < F; f += 32) {
        const float s = score[(size_t)leaf * F + f];
        const int b = bin[(size_t)leaf * F + f];
        if (b >= 0 && (bf < 0 || s > bs)) { bs = s; bf = f; bb = b; bg = gain[(size_t)leaf * F + f]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, bs, o);
        const int of = __shfl_xor_sync(0xffffffffu, bf, o);
        const int ob = __shfl_xor_sync(0xffffffffu, bb, o);
        const float og = __shfl_xor_sync(0xffffffffu, bg, o);
        const bool take = (of >= 0) && (bf < 0 || os > bs || (os == bs && of < bf));
        if (take) { bs = os; bf = of; bb = ob; bg = og; }
    }
    if (lane == 0) {
        float* o = best + (size_t)leaf * 4;
        o[0] = bf >= 0 ? bs : -INFINITY;
        reinterpret_cast<int*>(o)[1] = bf;
        reinterpret_cast<int*>(o)[2] = bb;
        o[3] = bg;
    }
}

CB_API int cb_leaf_search(const CbData* d, const float* hist, int nleaf, int S, int K, float l2, int score_fn, float noise_std,
                          unsigned long long seed, const int* leaf_id, const float* fmask, float min_data, float* out_score,
                          int* out_bin, float* out_gain, float* best, cudaStream_t st) {
    if (nleaf <= 0 || d->F <= 0) return 0;
    CbLeafSearchArgs a{*d, hist, nleaf, S, K, l2, score_fn, noise_std, seed, leaf_id, fmask, min_data, out_score, out_bin, out_gain};
    const long long warps = (long long)nleaf * d->F;
    cb_leaf_search_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    cb_leaf_search_pick_kernel<<<(unsigned)((nleaf + 7) / 8), 256, 0, st>>>(out_score, out_bin, out_gain, nleaf, d->F, best);
    return (int)cudaGetLastError();
}
