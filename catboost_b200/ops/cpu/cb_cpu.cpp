// CPU-side native code of catboost_b200 (OpenMP): border selection, quantisation, histograms, leaf index
// and batch apply.  It is the task_type='CPU' backend and the oracle for the CUDA kernels.
// C ABI, called through ctypes with numpy buffers.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <queue>
#include <vector>
#ifdef _OPENMP
#include <omp.h>

#include "cb_cityhash.h"
#endif

#define CBC_API extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------------------------------------------
// Border selection on a sorted sample of one feature.
// Behaviour follows library/cpp/grid_creator/binarization.cpp: GreedyLogSum / GreedyMinEntropy split the
// widest-gain bin first (priority queue keyed by the penalty gain of a median split, :1378-1520), Median =
// equal-frequency quantiles, Uniform = equally spaced between min and max, UniformAndQuantiles = half each.
// A border always lies between two distinct sample values (their mean).
namespace {

enum BorderType { kMedian = 0, kGreedyLogSum = 1, kUniform = 2, kUniformAndQuantiles = 3, kMinEntropy = 4, kMaxLogSum = 5, kGreedyMinEntropy = 6 };

inline double Penalty(double w, bool entropy) { return entropy ? w * std::log(w + 1e-8) : -std::log(w + 1e-8); }

struct Bin {
    uint32_t begin, end, split;
    double gain;
    bool operator<(const Bin& o) const { return gain < o.gain; }
    bool can_split() const { return split != begin && split != end; }
};

struct GreedySplitter {
    const float* v;
    bool entropy;
    double score(const Bin& b, uint32_t pos) const {
        if (pos == b.begin || pos == b.end) return -std::numeric_limits<double>::infinity();
        return -Penalty(double(pos - b.begin), entropy) - Penalty(double(b.end - pos), entropy) +
               Penalty(double(b.end - b.begin), entropy);
    }
    void refresh(Bin& b) const {
        const uint32_t mid = b.begin + (b.end - b.begin) / 2;
        const float mv = v[mid];
        const uint32_t lb = uint32_t(std::lower_bound(v + b.begin, v + mid, mv) - v);
        const uint32_t ub = uint32_t(std::upper_bound(v + mid, v + b.end, mv) - v);
        const double sl = score(b, lb), sr = score(b, ub);
        if (sl >= sr) { b.split = lb; b.gain = sl; } else { b.split = ub; b.gain = sr; }
    }
};

void GreedyBorders(const float* v, uint32_t n, int max_borders, bool entropy, std::vector<float>& out) {
    GreedySplitter sp{v, entropy};
    std::priority_queue<Bin> q;
    Bin root{0, n, 0, 0.0};
    sp.refresh(root);
    q.push(root);
    while ((int)q.size() <= max_borders && q.top().can_split()) {
        Bin top = q.top();
        q.pop();
        Bin left{top.begin, top.split, 0, 0.0};
        sp.refresh(left);
        top.begin = top.split;
        sp.refresh(top);
        q.push(left);
        q.push(top);
    }
    while (!q.empty()) {
        const Bin& b = q.top();
        if (b.begin != 0) out.push_back(0.5f * v[b.begin - 1] + 0.5f * v[b.begin]);
        q.pop();
    }
}

void MedianBorders(const float* v, uint32_t n, int max_borders, std::vector<float>& out) {
    for (int k = 1; k <= max_borders; ++k) {
        const uint64_t pos = uint64_t(k) * n / (max_borders + 1);
        if (pos == 0 || pos >= n) continue;
        if (v[pos - 1] != v[pos]) out.push_back(0.5f * v[pos - 1] + 0.5f * v[pos]);
        else {
            // move to the nearest change of value so that heavy ties still get a border
            const float* lo = std::lower_bound(v, v + n, v[pos]);
            if (lo != v) out.push_back(0.5f * lo[-1] + 0.5f * lo[0]);
        }
    }
}

void UniformBorders(const float* v, uint32_t n, int max_borders, std::vector<float>& out) {
    const float lo = v[0], hi = v[n - 1];
    if (!(hi > lo)) return;
    for (int k = 1; k <= max_borders; ++k) out.push_back(lo + (hi - lo) * float(k) / float(max_borders + 1));
}

}  // namespace

// values: sorted ascending, NaN-free.  Returns the number of borders written (sorted, unique).
CBC_API int cbc_select_borders(const float* values, long long n, int max_borders, int type, float* out) {
    if (n <= 1 || max_borders <= 0 || values[0] == values[n - 1]) return 0;
    std::vector<float> b;
    switch (type) {
        case kMedian: MedianBorders(values, (uint32_t)n, max_borders, b); break;
        case kUniform: UniformBorders(values, (uint32_t)n, max_borders, b); break;
        case kUniformAndQuantiles:
            UniformBorders(values, (uint32_t)n, max_borders / 2, b);
            MedianBorders(values, (uint32_t)n, max_borders - max_borders / 2, b);
            break;
        case kMinEntropy:
        case kGreedyMinEntropy: GreedyBorders(values, (uint32_t)n, max_borders, true, b); break;
        default: GreedyBorders(values, (uint32_t)n, max_borders, false, b); break;
    }
    std::sort(b.begin(), b.end());
    b.erase(std::unique(b.begin(), b.end()), b.end());
    if ((int)b.size() > max_borders) b.resize(max_borders);
    std::copy(b.begin(), b.end(), out);
    return (int)b.size();
}

// Ascending sort of NaN-free floats: four 8-bit counting passes over the order-preserving integer image of the
// values (sign bit flipped for positives, all bits for negatives).  About 15 times faster than std::sort on 200K values,
// which is what border selection spends its time on.
static void cbc_radix_sort_floats(std::vector<float>& v, std::vector<uint32_t>& a, std::vector<uint32_t>& b) {
    const size_t n = v.size();
    if (n < 2048) { std::sort(v.begin(), v.end()); return; }
    a.resize(n);
    b.resize(n);
    for (size_t i = 0; i < n; ++i) {
        uint32_t u;
        std::memcpy(&u, &v[i], 4);
        a[i] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    }
    uint32_t* src = a.data();
    uint32_t* dst = b.data();
    // all four digit histograms in one read; 256 write streams per pass stay within the L1 cache and the TLB
    uint32_t cnt[4][256] = {{0}};
    for (size_t i = 0; i < n; ++i) {
        const uint32_t k = src[i];
        ++cnt[0][k & 255u]; ++cnt[1][(k >> 8) & 255u]; ++cnt[2][(k >> 16) & 255u]; ++cnt[3][k >> 24];
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = pass * 8;
        uint32_t run = 0;
        for (int k = 0; k < 256; ++k) { const uint32_t c = cnt[pass][k]; cnt[pass][k] = run; run += c; }
        uint32_t* pos = cnt[pass];
        for (size_t i = 0; i < n; ++i) { const uint32_t k = src[i]; dst[pos[(k >> shift) & 255u]++] = k; }
        std::swap(src, dst);
    }
    for (size_t i = 0; i < n; ++i) {
        const uint32_t k = src[i];
        const uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
        std::memcpy(&v[i], &u, 4);
    }
}

// Column-wise border selection for a row-major float matrix sample [n][F] (ld = row stride).
// out_borders: [F][max_borders]; out_counts: [F]; has_nan: [F] (1 when the sample holds a NaN).
// A thread takes 16 neighbouring columns at a time, so every 64-byte line of a row is read once (one column at a time
// re-read the whole matrix once per column: 25 GB of traffic for 200K x 2000).
CBC_API void cbc_select_borders_matrix(const float* X, long long n, int F, long long ld, int max_borders, int type,
                                       float* out_borders, int* out_counts, unsigned char* has_nan) {
    const int CBMAX = 16;
    int nthr = 1;
#ifdef _OPENMP
    nthr = omp_get_max_threads();
#endif
    // narrow matrices: fewer columns per work item so that every thread has one (28 columns in blocks of 16 kept 2 busy)
    const int CB = std::max(1, std::min(CBMAX, F / (2 * std::max(nthr, 1))));
    const int nblocks = (F + CB - 1) / CB;
#pragma omp parallel
    {
        std::vector<float> col[CBMAX];
        std::vector<uint32_t> ka, kb;
#pragma omp for schedule(dynamic, 1)
        for (int blk = 0; blk < nblocks; ++blk) {
            const int f0 = blk * CB, w = std::min(CB, F - f0);
            bool nan[CBMAX] = {false};
            for (int j = 0; j < w; ++j) { col[j].clear(); col[j].reserve((size_t)n); }
            for (long long i = 0; i < n; ++i) {
                const float* row = X + i * ld + f0;
                for (int j = 0; j < w; ++j) {
                    const float v = row[j];
                    if (v != v) nan[j] = true; else col[j].push_back(v);
                }
            }
            for (int j = 0; j < w; ++j) {
                const int f = f0 + j;
                cbc_radix_sort_floats(col[j], ka, kb);
                has_nan[f] = nan[j] ? 1 : 0;
                out_counts[f] = col[j].empty() ? 0
                                               : cbc_select_borders(col[j].data(), (long long)col[j].size(), max_borders, type,
                                                                    out_borders + (size_t)f * max_borders);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Quantise a row-major matrix into the packed group store used by both backends:
// bins[g][npad] uint32, byte j of group g = bin of feature 4g+j; bin = number of borders < value.
CBC_API void cbc_quantize(const float* X, long long n, int F, long long ld, const float* borders, const int* border_off,
                          const unsigned char* nan_is_max, uint32_t* bins, long long npad, long long doc_offset) {
    const int G = (F + 3) / 4;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const float* row = X + i * ld;
        for (int g = 0; g < G; ++g) {
            uint32_t word = 0;
            for (int j = 0; j < 4; ++j) {
                const int f = 4 * g + j;
                if (f >= F) break;
                const float v = row[f];
                const float* b0 = borders + border_off[f];
                const float* b1 = borders + border_off[f + 1];
                int bin;
                if (v != v) bin = (nan_is_max && nan_is_max[f]) ? int(b1 - b0) : 0;
                else bin = int(std::lower_bound(b0, b1, v) - b0);
                word |= uint32_t(bin) << (8 * j);
            }
            bins[(size_t)g * npad + doc_offset + i] = word;
        }
    }
}

CBC_API void cbc_pack_bins(const unsigned char* cols, long long n, long long ld, int F, int f_dst_begin, uint32_t* bins,
                           long long npad, long long doc_offset) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        for (int f = 0; f < F; ++f) {
            const int fd = f_dst_begin + f;
            uint32_t& w = bins[(size_t)(fd >> 2) * npad + doc_offset + i];
            const int sh = (fd & 3) * 8;
            w = (w & ~(255u << sh)) | (uint32_t(cols[(size_t)f * ld + i]) << sh);
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Histogram: out[slot][s][feat_off[f] + bin] += stats[s][i] for documents whose slot_of_leaf[leaf[i]] >= 0.
// Thread-private accumulation in double then reduction, so the result does not depend on the thread count
// beyond rounding of the final float conversion.
CBC_API void cbc_hist(const uint32_t* bins, long long npad, long long n, int F, const int* feat_off, int TB,
                      const uint16_t* leaf, const float* stats, int S, const short* slot_of_leaf, int nslots,
                      float* out) {
    const int G = (F + 3) / 4;
    const size_t total = (size_t)nslots * S * TB;
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    std::vector<std::vector<double>> priv(nthreads);
#pragma omp parallel
    {
        int t = 0;
#ifdef _OPENMP
        t = omp_get_thread_num();
#endif
        std::vector<double>& h = priv[t];
        h.assign(total, 0.0);
        // a thread's documents are walked once per feature group: the cells one pass touches (slots x statistics x the
        // bins of 4 features) stay in the core's cache, where walking all groups per document spread the updates over the
        // whole private histogram
        long long i0 = 0, i1 = n;
#ifdef _OPENMP
        {
            const int nt = omp_get_num_threads();
            i0 = n * t / nt;
            i1 = n * (t + 1) / nt;
        }
#endif
        for (int g = 0; g < G; ++g) {
            const uint32_t* row = bins + (size_t)g * npad;
            const int fcount = std::min(4, F - 4 * g);
            int off4[4] = {0, 0, 0, 0};
            for (int j = 0; j < fcount; ++j) off4[j] = feat_off[4 * g + j];
            for (long long i = i0; i < i1; ++i) {
                const int slot = slot_of_leaf[leaf[i]];
                if (slot < 0) continue;
                const uint32_t w = row[i];
                double* hs = h.data() + (size_t)slot * S * TB;
                for (int s = 0; s < S; ++s) {
                    const double v = (double)stats[(size_t)s * npad + i];
                    double* hh = hs + (size_t)s * TB;
                    for (int j = 0; j < fcount; ++j) hh[off4[j] + int((w >> (8 * j)) & 255u)] += v;
                }
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (long long k = 0; k < (long long)total; ++k) {
        double acc = 0.0;
        for (int t = 0; t < nthreads; ++t) if (!priv[t].empty()) acc += priv[t][k];
        out[k] = float(acc);
    }
}

// leaf |= (bin > thr) << level   (one-hot: bin == thr)
CBC_API void cbc_update_leaf(const uint32_t* bins, long long npad, long long n, int feature, int bin, int onehot,
                             int level, uint16_t* leaf) {
    const uint32_t* col = bins + (size_t)(feature >> 2) * npad;
    const int sh = (feature & 3) * 8;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const unsigned b = (col[i] >> sh) & 255u;
        const unsigned r = onehot ? (b == (unsigned)bin) : (b > (unsigned)bin);
        leaf[i] = uint16_t(leaf[i] | (r << level));
    }
}

// node-id update for non-symmetric trees; node_split rows = {feature, bin, flags, left_child}
CBC_API void cbc_update_nodes(const uint32_t* bins, long long npad, long long n, const int* node_split, int n_nodes,
                              uint16_t* leaf) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const int node = leaf[i];
        if (node >= n_nodes) continue;
        const int* sp = node_split + 4 * node;
        if (sp[0] < 0) continue;
        const unsigned b = (bins[(size_t)(sp[0] >> 2) * npad + i] >> ((sp[0] & 3) * 8)) & 255u;
        const bool right = (sp[2] & 1) ? (b == (unsigned)sp[1]) : (b > (unsigned)sp[1]);
        leaf[i] = uint16_t(sp[3] + (right ? 1 : 0));
    }
}

// oblivious leaf index from `depth` splits {feature, bin, score(bits), flags} (same 16-byte record as the GPU)
CBC_API void cbc_leaf_index(const uint32_t* bins, long long npad, long long n, const int* splits, int depth,
                            uint16_t* leaf) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        int l = 0;
        for (int k = 0; k < depth; ++k) {
            const int f = splits[4 * k];
            if (f < 0) continue;
            const unsigned b = (bins[(size_t)(f >> 2) * npad + i] >> ((f & 3) * 8)) & 255u;
            const unsigned thr = (unsigned)splits[4 * k + 1];
            l |= int((splits[4 * k + 3] & 1) ? (b == thr) : (b > thr)) << k;
        }
        leaf[i] = uint16_t(l);
    }
}

// per-leaf sums: sums[leaf][c] += cols[c][i]
CBC_API void cbc_leaf_sums(const uint16_t* leaf, long long n, const float* cols, long long ld, int C, int L, double* sums) {
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    std::vector<std::vector<double>> priv(nthreads);
#pragma omp parallel
    {
        int t = 0;
#ifdef _OPENMP
        t = omp_get_thread_num();
#endif
        priv[t].assign((size_t)L * C, 0.0);
        double* h = priv[t].data();
#pragma omp for schedule(static)
        for (long long i = 0; i < n; ++i) {
            const int l = leaf[i];
            for (int c = 0; c < C; ++c) h[(size_t)l * C + c] += cols[(size_t)c * ld + i];
        }
    }
    for (size_t k = 0; k < (size_t)L * C; ++k) {
        double acc = 0.0;
        for (int t = 0; t < nthreads; ++t) if (!priv[t].empty()) acc += priv[t][k];
        sums[k] = acc;
    }
}

// Split scores of one level of a symmetric tree from the level's histograms: hist [L][S][TB] floats (S statistics: K
// derivative sums, then the weight), out [F][B] floats.  Candidate (f, b): "bin <= b goes left" (one-hot: "bin != b goes
// left"); every leaf contributes both sides; fn 0 = Cosine: sum s mu / sqrt(sum w mu^2) with mu = s / (w + l2),
// fn 1 = L2: sum s^2 / (w + l2).  The same formulas as SplitScorer in train/generic.py (its oracle), accumulated in
// doubles; positions that are no candidates (b >= candidates of f) get -3e38.
CBC_API void cbc_symmetric_scores(const float* hist, int L, int S, int K, int TB, int F, const int* feat_off, const int* nb,
                                  const unsigned char* onehot, int fn, double l2, int B, float* out) {
#pragma omp parallel
    {
        std::vector<double> num, den, cum, tot;
#pragma omp for schedule(dynamic, 1)
        for (int f = 0; f < F; ++f) {
            const int n = nb[f], off = feat_off[f];
            const int ncand = onehot[f] ? n : n - 1;
            num.assign((size_t)std::max(n, 1), 0.0);
            den.assign((size_t)std::max(n, 1), 0.0);
            cum.resize((size_t)(K + 1));
            tot.resize((size_t)(K + 1));
            for (int l = 0; l < L; ++l) {
                const float* hl = hist + (size_t)l * S * TB + off;
                for (int k = 0; k <= K; ++k) {
                    double t = 0.0;
                    const float* row = hl + (size_t)k * TB;
                    for (int b = 0; b < n; ++b) t += (double)row[b];
                    tot[k] = t;
                    cum[k] = 0.0;
                }
                for (int b = 0; b < ncand; ++b) {
                    double lw, rw;
                    if (onehot[f]) {
                        rw = (double)hl[(size_t)K * TB + b];
                        lw = tot[K] - rw;
                    } else {
                        cum[K] += (double)hl[(size_t)K * TB + b];
                        lw = cum[K];
                        rw = tot[K] - lw;
                    }
                    lw = std::max(lw, 0.0);
                    rw = std::max(rw, 0.0);
                    for (int k = 0; k < K; ++k) {
                        double ls, rs;
                        if (onehot[f]) { rs = (double)hl[(size_t)k * TB + b]; ls = tot[k] - rs; }
                        else { cum[k] += (double)hl[(size_t)k * TB + b]; ls = cum[k]; rs = tot[k] - ls; }
                        if (fn == 0) {
                            const double ml = lw > 0.0 ? ls / (lw + l2) : 0.0, mr = rw > 0.0 ? rs / (rw + l2) : 0.0;
                            num[b] += ls * ml + rs * mr;
                            den[b] += lw * ml * ml + rw * mr * mr;
                        } else {
                            num[b] += (lw > 1e-20 ? ls * ls / (lw + l2) : 0.0) + (rw > 1e-20 ? rs * rs / (rw + l2) : 0.0);
                        }
                    }
                }
            }
            float* o = out + (size_t)f * B;
            for (int b = 0; b < B; ++b) {
                if (b >= ncand) { o[b] = -3.0e38f; continue; }
                o[b] = fn == 0 ? (den[b] > 1e-15 ? (float)(num[b] / std::sqrt(den[b] + 1e-10)) : -3.0e38f) : (float)num[b];
            }
        }
    }
}

// All Newton / gradient steps of the leaf estimation of one tree for the losses with a closed formula here (0 RMSE,
// 1 Logloss, 2 CrossEntropy, 3 Poisson): per step one pass over the documents (loss value and derivatives at
// approx + delta[leaf], per-leaf sums in per-thread doubles), then delta += sum der / (sum hess or sum weight + l2).
// backtrack = 1 (AnyImprovement) / 2 (Armijo): a point whose loss fails the condition is dropped and the next pass tries
// half the step from the last accepted point; a rejected try uses up one step (the step-length control of the general
// learner's tensor formulation, which stays the path of every other loss and is the oracle of this routine).
// Returns 0, or -1 when the loss has no formula here.  delta [L] (unscaled), leaf_w [L].
CBC_API int cbc_leaf_newton(int loss, const float* approx, const float* target, const float* weight, const uint16_t* leaf,
                            long long n, int L, int steps, int newton, double l2, int backtrack, double* delta,
                            double* leaf_w) {
    if (loss < 0 || loss > 3) return -1;
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    if (steps < 1) steps = 1;
    if (steps == 1) backtrack = 0;
    std::vector<std::vector<double>> priv(nthreads);
    std::vector<float> dl((size_t)L, 0.0f), base((size_t)L, 0.0f), dir((size_t)L, 0.0f);
    std::vector<double> sd((size_t)L), sh((size_t)L), sw((size_t)L);
    for (int l = 0; l < L; ++l) { delta[l] = 0.0; leaf_w[l] = 0.0; }
    double f_base = 0.0, dirgrad = 0.0, cur_step = 1.0;
    bool have_w = false;
    for (int step = 0; step < steps; ++step) {
#pragma omp parallel
        {
            int t = 0;
#ifdef _OPENMP
            t = omp_get_thread_num();
#endif
            priv[t].assign((size_t)L * 3 + 1, 0.0);
            double* h = priv[t].data();
            double vsum = 0.0;
#pragma omp for schedule(static)
            for (long long i = 0; i < n; ++i) {
                const int l = leaf[i];
                const float a = approx[i] + dl[l], y = target[i], w = weight ? weight[i] : 1.0f;
                float d, hs, v;
                if (loss == 0) { d = y - a; hs = 1.0f; v = d * d; }
                else if (loss == 3) { const float e = std::exp(a); d = y - e; hs = e; v = e - y * a; }
                else {
                    const float p = 1.0f / (1.0f + std::exp(-a));
                    d = y - p; hs = std::max(p * (1.0f - p), 1e-16f);
                    v = backtrack ? (std::max(a, 0.0f) + std::log1p(std::exp(-std::fabs(a))) - y * a) : 0.0f;
                }
                h[(size_t)l * 3] += (double)(d * w);
                h[(size_t)l * 3 + 1] += (double)(hs * w);
                h[(size_t)l * 3 + 2] += (double)w;
                vsum += (double)(v * w);
            }
            h[(size_t)L * 3] = vsum;
        }
        double v = 0.0;
        for (int t = 0; t < nthreads; ++t) if (!priv[t].empty()) v += priv[t][(size_t)L * 3];
        if (backtrack && step > 0 && !(v <= f_base - (backtrack == 2 ? 1e-5 * cur_step * dirgrad : 0.0))) {
            cur_step *= 0.5;
            for (int l = 0; l < L; ++l) dl[l] = base[l] + (float)cur_step * dir[l];
            continue;
        }
        for (int l = 0; l < L; ++l) {
            double a = 0.0, b = 0.0, c = 0.0;
            for (int t = 0; t < nthreads; ++t)
                if (!priv[t].empty()) { a += priv[t][(size_t)l * 3]; b += priv[t][(size_t)l * 3 + 1]; c += priv[t][(size_t)l * 3 + 2]; }
            sd[l] = a; sh[l] = b; sw[l] = c;
        }
        if (!have_w) { for (int l = 0; l < L; ++l) leaf_w[l] = sw[l]; have_w = true; }
        dirgrad = 0.0;
        for (int l = 0; l < L; ++l) {
            const double den = (newton ? sh[l] : sw[l]) + l2;
            // the general learner keeps its running leaf values in float32: so does this
            const float stepv = den > 0.0 ? (float)(sd[l] / den) : 0.0f;
            base[l] = dl[l];
            dir[l] = stepv;
            dirgrad += sd[l] * (double)stepv;
            dl[l] += stepv;
        }
        f_base = v;
        cur_step = 1.0;
    }
    for (int l = 0; l < L; ++l) delta[l] = (double)dl[l];
    return 0;
}

// ------------------------------------------------------------------------------------------------------
// Batch apply of an oblivious ensemble to raw float rows (CPU evaluator).  Blocks of 128 rows are quantised
// for the used features, then every tree is walked for the block (libs/model/cpu/evaluator_impl.cpp:13-260
// describes the same blocking idea).  out: [dims][n] doubles.
CBC_API void cbc_predict_oblivious(const float* X, long long n, long long ld, const int* used_feat, const float* borders,
                                   const int* border_off, const unsigned char* nan_is_max, int U, const int* tree_depth,
                                   const int* tree_split_off, const uint16_t* split_feat, const uint8_t* split_bin,
                                   const long long* tree_leaf_off, const double* leaf_vals, int T, int dims,
                                   double scale, const double* bias, double* out) {
    const int BLK = 128;
    const long long nblk = (n + BLK - 1) / BLK;
#pragma omp parallel
    {
        std::vector<uint8_t> q((size_t)U * BLK);
        std::vector<int> idx(BLK);
        std::vector<double> acc((size_t)BLK * dims);
#pragma omp for schedule(dynamic, 4)
        for (long long b = 0; b < nblk; ++b) {
            const long long r0 = b * BLK;
            const int m = (int)std::min<long long>(BLK, n - r0);
            for (int u = 0; u < U; ++u) {
                const float* b0 = borders + border_off[u];
                const float* b1 = borders + border_off[u + 1];
                const int col = used_feat[u];
                for (int r = 0; r < m; ++r) {
                    const float v = X[(r0 + r) * ld + col];
                    int bin;
                    if (v != v) bin = (nan_is_max && nan_is_max[u]) ? int(b1 - b0) : 0;
                    else bin = int(std::lower_bound(b0, b1, v) - b0);
                    q[(size_t)u * BLK + r] = (uint8_t)bin;
                }
            }
            std::fill(acc.begin(), acc.end(), 0.0);
            for (int t = 0; t < T; ++t) {
                const int depth = tree_depth[t], so = tree_split_off[t];
                std::fill(idx.begin(), idx.begin() + m, 0);
                for (int k = 0; k < depth; ++k) {
                    const uint8_t* qc = q.data() + (size_t)split_feat[so + k] * BLK;
                    const uint8_t thr = split_bin[so + k];
                    for (int r = 0; r < m; ++r) idx[r] |= int(qc[r] > thr) << k;
                }
                const double* lv = leaf_vals + tree_leaf_off[t] * dims;
                for (int r = 0; r < m; ++r)
                    for (int d = 0; d < dims; ++d) acc[(size_t)r * dims + d] += lv[(size_t)idx[r] * dims + d];
            }
            for (int r = 0; r < m; ++r)
                for (int d = 0; d < dims; ++d)
                    out[(size_t)d * n + r0 + r] = acc[(size_t)r * dims + d] * scale + (bias ? bias[d] : 0.0);
        }
    }
}

CBC_API int cbc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
CBC_API void cbc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ------------------------------------------------------------------------------------------------------
// String hash of categorical values.  The reference hashes the string form of a categorical value with the
// 64-bit CityHash of 2011 (version 1) and keeps the low 32 bits (catboost/libs/cat_feature/cat_feature.cpp:4-6);
// model files store those hashes, so the function below has to produce the same numbers.


CBC_API unsigned long long cbc_cityhash64(const char* s, long long n) { return city1::hash(s, (size_t)n); }

// strings concatenated in `buf`; string k = buf[off[k] .. off[k+1])
CBC_API void cbc_cat_hash_batch(const char* buf, const long long* off, long long count, uint32_t* out) {
#pragma omp parallel for schedule(static)
    for (long long k = 0; k < count; ++k) out[k] = uint32_t(city1::hash(buf + off[k], size_t(off[k + 1] - off[k])) & 0xffffffffULL);
}

// decimal string form of integers, hashed (the reference stringifies integer categorical values)
CBC_API void cbc_cat_hash_ints(const long long* vals, long long count, uint32_t* out) {
#pragma omp parallel for schedule(static)
    for (long long k = 0; k < count; ++k) {
        char tmp[24];
        const int len = std::snprintf(tmp, sizeof(tmp), "%lld", vals[k]);
        out[k] = uint32_t(city1::hash(tmp, size_t(len)) & 0xffffffffULL);
    }
}

// One categorical column of integers with a small value range [mn, mn + range): the hash of every row through a direct
// table, filled on first use.  `table` [range] and `seen` [range] (zero-initialised by the caller) come back holding the
// hash of every value that occurs.  Two threads may fill the same entry: they write the same number.
CBC_API void cbc_cat_hash_dense_ints(const long long* vals, long long n, long long mn, long long range, uint32_t* out,
                                     uint32_t* table, unsigned char* seen) {
    (void)range;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < n; ++i) {
        const long long off = vals[i] - mn;
        if (!__atomic_load_n(&seen[off], __ATOMIC_ACQUIRE)) {
            char tmp[24];
            const int len = std::snprintf(tmp, sizeof(tmp), "%lld", vals[i]);
            table[off] = uint32_t(city1::hash(tmp, size_t(len)) & 0xffffffffULL);
            __atomic_store_n(&seen[off], (unsigned char)1, __ATOMIC_RELEASE);
        }
        out[i] = table[off];
    }
}

// Row-major matrix [n][F] from F separate float32 columns (blocks of rows per thread, so that reads stream and the
// writes of a block stay in cache).
CBC_API void cbc_interleave_f32(const float* const* cols, int F, long long n, float* out) {
    const long long BLK = 2048;
#pragma omp parallel for schedule(static)
    for (long long b0 = 0; b0 < n; b0 += BLK) {
        const long long b1 = std::min(n, b0 + BLK);
        for (int j = 0; j < F; ++j) {
            const float* c = cols[j];
            float* o = out + b0 * F + j;
            for (long long r = b0; r < b1; ++r, o += F) *o = c[r];
        }
    }
}
