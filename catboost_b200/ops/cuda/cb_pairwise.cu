// Pairwise split search (PairLogitPairwise / YetiRankPairwise) as kernels: pairwise histograms, bin prefix sums,
// assembly of one 2L x 2L linear system per candidate border, Cholesky solve and gain, all on the device.
//
// Behaviour reproduced from the reference (not its code): a pair (winner i, loser j, weight w) contributes w to the
// off-diagonal cell (child of i, child of j) of the candidate's leaf-pair matrix; the four configurations of a pair
// under a border come from four histograms per (leaf pair, bin) and bin prefix sums
// (catboost/cuda/methods/kernel/pairwise_hist_one_byte_6bit.cuh:260, pairwise_hist.cu, split_pairwise.cu:21-419); the
// candidate's leaf values solve (Laplacian + regularisation) x = derivative sums with the last unknown pinned
// (catboost/cuda/methods/kernel/linear_solver.cu:71-398, catboost/private/libs/algo/pairwise_scoring.cpp:123-260) and
// its score is x.d - x'Mx / 2.
//
// Histogram layout (floats): H[f][bin][a][b][4] for the ordered leaf pair (a = leaf of the winner, b = leaf of the
// loser).  Float features, lo / hi = smaller / larger bin of the pair:
//   [0] += w at bin lo when the winner has the smaller bin     [1] += w at bin hi when the winner has the smaller bin
//   [2] += w at bin lo otherwise (loser smaller, or equal)     [3] += w at bin hi otherwise
// After an inclusive prefix sum over the bins, for border t (a document goes right iff bin > t):
//   both left  = ([1] + [3])(t)               winner left, loser right = ([0] - [1])(t)
//   both right = total - ([0] + [2])(t)       winner right, loser left = ([2] - [3])(t)
// One-hot features (right iff bin == v), no prefix sum:
//   [0] += w at v = bin_i = bin_j (both right)   [1] += w at v = bin_i != bin_j (winner right)
//   [2] += w at v = bin_j != bin_i (loser right)  both left = total - [0] - [1] - [2]
#include "cb_common.cuh"
#include <cstdlib>
#include "cb_tree.cuh"

struct CbPairHistArgs {
    CbData d;
    const unsigned short* leaf;     // current leaf of every document (< L)
    const int* wi; const int* li;   // winner / loser document of every pair
    const float* w;                 // pair weights
    long long npairs;
    int L, B;                       // leaves, bins per feature in the layout (>= max feat_nb)
    int g0, ng;                     // feature groups [g0, g0 + ng) of the store are accumulated
    float* H;                       // [ng * 4][B][L][L][4]
};

// One thread per pair and range of feature groups (blockIdx.y = range): the thread reads its pair once (documents, leaves,
// weight) and walks the groups of the range; all pairs of a range run before the next range, so the range's bin columns
// (4 bytes per document and group) and its histograms stay in L2 while the pairs stream past.  (Pair-major over all
// groups touched every column of the store at once: 2.0 s per tree at 2M documents x 700 features and 20M pairs;
// group-major with one group per thread re-read the pair for every group.)  The two bin words of a group give four
// features at once; 8 atomics.
__global__ void __launch_bounds__(256) cb_pair_hist_kernel(CbPairHistArgs a, int gpr) {
    const int gl_lo = blockIdx.y * gpr, gl_hi = min(a.ng, gl_lo + gpr);
    const long long stride = (long long)gridDim.x * blockDim.x;
    const size_t fstride = (size_t)a.B * a.L * a.L * 4;
    const size_t bs = (size_t)a.L * a.L * 4;
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < a.npairs; p += stride) {
        const float w = a.w[p];
        if (w == 0.0f) continue;
        const int i = a.wi[p], j = a.li[p];
        const int la = a.leaf[i], lb = a.leaf[j];
        const size_t cell = ((size_t)la * a.L + lb) * 4;
        for (int gl = gl_lo; gl < gl_hi; ++gl) {
            const int g = a.g0 + gl;
            const uint32_t wi_ = a.d.bins[(long long)g * a.d.npad + i], wj_ = a.d.bins[(long long)g * a.d.npad + j];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int f = g * 4 + q;
                if (f >= a.d.F) break;
                const int bi = (int)((wi_ >> (8 * q)) & 255u), bj = (int)((wj_ >> (8 * q)) & 255u);
                float* Hf = a.H + (size_t)(gl * 4 + q) * fstride;
                if (a.d.feat_onehot && a.d.feat_onehot[f]) {
                    if (bi == bj) atomicAdd(Hf + bi * bs + cell, w);
                    else { atomicAdd(Hf + bi * bs + cell + 1, w); atomicAdd(Hf + bj * bs + cell + 2, w); }
                } else {
                    const bool wsmall = bi < bj;
                    const int lo = wsmall ? bi : bj, hi = wsmall ? bj : bi;
                    atomicAdd(Hf + lo * bs + cell + (wsmall ? 0 : 2), w);
                    atomicAdd(Hf + hi * bs + cell + (wsmall ? 1 : 3), w);
                }
            }
        }
    }
}

// Shallow levels (the histogram of a group -- NFEAT = 4 features, or of one feature -- fits in shared memory): a block
// takes a chunk of CB_PAIR_CHUNK pairs of one group, accumulates in shared int32 cells in fixed point (scale = 2^31 /
// (chunk x largest pair weight), 17 bits of the largest weight: the cell cannot overflow) and adds its non-zero cells to
// the global histogram at the end.  Native integer reductions in shared memory replace two global float atomics per
// (pair, feature); the flush costs one global atomic per non-zero cell and chunk.  blockIdx.x (fastest) walks the
// chunks of one group, so the group's bin column stays in L2.
#define CB_PAIR_CHUNK 16384

template <int NFEAT>
__global__ void __launch_bounds__(256) cb_pair_hist_smem_kernel(CbPairHistArgs a, float qs) {
    extern __shared__ int cb_ph[];                  // [NFEAT][B][L][L][4]
    const size_t bs = (size_t)a.L * a.L * 4;
    const int per_feat = a.B * (int)bs;
    const int cells = NFEAT * per_feat;
    for (int c = threadIdx.x; c < cells; c += blockDim.x) cb_ph[c] = 0;
    __syncthreads();
    const int gl = NFEAT == 4 ? (int)blockIdx.y : (int)(blockIdx.y >> 2);
    const int q_lo = NFEAT == 4 ? 0 : (int)(blockIdx.y & 3), q_hi = NFEAT == 4 ? 4 : q_lo + 1;
    const int g = a.g0 + gl;
    bool onehot[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) onehot[q] = (g * 4 + q < a.d.F) && a.d.feat_onehot && a.d.feat_onehot[g * 4 + q];
    const long long begin = (long long)blockIdx.x * CB_PAIR_CHUNK;
    const long long end = min(a.npairs, begin + CB_PAIR_CHUNK);
    const uint32_t* col = a.d.bins + (long long)g * a.d.npad;
    for (long long p = begin + threadIdx.x; p < end; p += blockDim.x) {
        const float w = a.w[p];
        if (w == 0.0f) continue;
        const int i = a.wi[p], j = a.li[p];
        const int cell = (a.leaf[i] * a.L + a.leaf[j]) * 4;
        const uint32_t wi_ = col[i], wj_ = col[j];
        const int qw = __float2int_rn(w * qs);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (q < q_lo || q >= q_hi || g * 4 + q >= a.d.F) continue;
            const int bi = (int)((wi_ >> (8 * q)) & 255u), bj = (int)((wj_ >> (8 * q)) & 255u);
            int* Hf = cb_ph + (NFEAT == 4 ? q * per_feat : 0);
            if (onehot[q]) {
                if (bi == bj) atomicAdd(Hf + bi * (int)bs + cell, qw);
                else { atomicAdd(Hf + bi * (int)bs + cell + 1, qw); atomicAdd(Hf + bj * (int)bs + cell + 2, qw); }
            } else {
                const bool wsmall = bi < bj;
                const int lo = wsmall ? bi : bj, hi = wsmall ? bj : bi;
                atomicAdd(Hf + lo * (int)bs + cell + (wsmall ? 0 : 2), qw);
                atomicAdd(Hf + hi * (int)bs + cell + (wsmall ? 1 : 3), qw);
            }
        }
    }
    __syncthreads();
    const float inv = 1.0f / qs;
    const size_t fstride = (size_t)a.B * bs;
    for (int c = threadIdx.x; c < cells; c += blockDim.x) {
        const int v = cb_ph[c];
        if (v == 0) continue;
        const int q = NFEAT == 4 ? c / per_feat : q_lo;
        const int rem = NFEAT == 4 ? c - q * per_feat : c;
        atomicAdd(a.H + (size_t)(gl * 4 + q) * fstride + rem, (float)v * inv);
    }
}

// Deep levels (L x L leaf pairs no longer fit in shared memory): the caller sorts the pairs by leaf pair and cuts every
// leaf pair's run into chunks of at most CB_PAIR_CHUNK pairs; a block takes one chunk of one group, so all its pairs share
// the (leaf of winner, leaf of loser) cell and the shared histogram is just [4 features][B bins][4] int32 cells.  No leaf
// look-ups in the kernel, native shared-memory integer reductions, one global atomic per non-zero cell at the end.
// chunks[c] = (first pair, one past the last pair, leaf pair number la * L + lb, unused).
__global__ void __launch_bounds__(256) cb_pair_hist_sorted_kernel(CbPairHistArgs a, const int4* chunks, float qs) {
    __shared__ int hist[4 * 256 * 4];
    const int cells = 4 * a.B * 4;
    for (int c = threadIdx.x; c < cells; c += blockDim.x) hist[c] = 0;
    __syncthreads();
    const int4 ch = chunks[blockIdx.x];
    const int gl = blockIdx.y, g = a.g0 + gl;
    bool onehot[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) onehot[q] = (g * 4 + q < a.d.F) && a.d.feat_onehot && a.d.feat_onehot[g * 4 + q];
    const uint32_t* col = a.d.bins + (long long)g * a.d.npad;
    for (int p = ch.x + (int)threadIdx.x; p < ch.y; p += blockDim.x) {
        const float w = a.w[p];
        if (w == 0.0f) continue;
        const uint32_t wi_ = col[a.wi[p]], wj_ = col[a.li[p]];
        const int qw = __float2int_rn(w * qs);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (g * 4 + q >= a.d.F) continue;
            const int bi = (int)((wi_ >> (8 * q)) & 255u), bj = (int)((wj_ >> (8 * q)) & 255u);
            int* Hf = hist + q * a.B * 4;
            if (onehot[q]) {
                if (bi == bj) atomicAdd(Hf + bi * 4, qw);
                else { atomicAdd(Hf + bi * 4 + 1, qw); atomicAdd(Hf + bj * 4 + 2, qw); }
            } else {
                const bool wsmall = bi < bj;
                const int lo = wsmall ? bi : bj, hi = wsmall ? bj : bi;
                atomicAdd(Hf + lo * 4 + (wsmall ? 0 : 2), qw);
                atomicAdd(Hf + hi * 4 + (wsmall ? 1 : 3), qw);
            }
        }
    }
    __syncthreads();
    const float inv = 1.0f / qs;
    const size_t bs = (size_t)a.L * a.L * 4, fstride = (size_t)a.B * bs;
    const size_t cell = (size_t)ch.z * 4;
    for (int c = threadIdx.x; c < cells; c += blockDim.x) {
        const int v = hist[c];
        if (v == 0) continue;
        const int q = c / (a.B * 4), rem = c - q * a.B * 4;
        atomicAdd(a.H + (size_t)(gl * 4 + q) * fstride + (size_t)(rem >> 2) * bs + cell + (rem & 3), (float)v * inv);
    }
}

// Pair histograms from pairs sorted by leaf pair (see the kernel above).  H zeroed by the caller; B <= 256.
CB_API int cb_pair_hist_sorted(const CbData* d, const int* wi, const int* li, const float* w, long long npairs,
                               const int* chunks, int nchunks, int L, int B, int g0, int ng, float* H, float wmax,
                               cudaStream_t st) {
    if (npairs <= 0 || nchunks <= 0 || ng <= 0) return 0;
    if (B > 256 || wmax <= 0.0f) return (int)cudaErrorInvalidValue;
    CbPairHistArgs a{*d, nullptr, wi, li, w, npairs, L, B, g0, ng, H};
    const float qs = 2147483647.0f / ((float)CB_PAIR_CHUNK * wmax) * 0.999f;
    cb_pair_hist_sorted_kernel<<<dim3((unsigned)nchunks, (unsigned)ng), 256, 0, st>>>(a, reinterpret_cast<const int4*>(chunks), qs);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
CB_API int cb_pair_chunk_pairs(void) { return CB_PAIR_CHUNK; }

// Per-document derivative sums D[f][bin][leaf] for the same features (one thread per (document, group)).
__global__ void __launch_bounds__(256) cb_pair_der_hist_kernel(CbData d, const unsigned short* leaf, const float* der, int L,
                                                               int B, int g0, int ng, float* D) {
    const long long total = d.n * ng;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int gl = (int)(idx / d.n);
        const long long i = idx - (long long)gl * d.n;
        const int g = g0 + gl;
        const float v = der[i];
        const uint32_t wd = d.bins[(long long)g * d.npad + i];
        const int l = leaf[i];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (g * 4 + q >= d.F) break;
            const int b = (int)((wd >> (8 * q)) & 255u);
            atomicAdd(D + ((size_t)(gl * 4 + q) * B + b) * L + l, v);
        }
    }
}

// Inclusive prefix sum over the bins of every column (cols = floats per bin) of the float features; one-hot features
// are left as they are.
__global__ void __launch_bounds__(256) cb_pair_scan_kernel(CbData d, int f0, int nf, int B, long long cols, float* H) {
    const long long total = (long long)nf * cols;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int fl = (int)(idx / cols);
        const long long c = idx - (long long)fl * cols;
        const int f = f0 + fl;
        if (f >= d.F || (d.feat_onehot && d.feat_onehot[f])) continue;
        float* col = H + (size_t)fl * B * cols + c;
        float run = 0.0f;
        for (int b = 0; b < B; ++b) { run += col[(size_t)b * cols]; col[(size_t)b * cols] = run; }
    }
}

struct CbPairSolveArgs {
    CbData d;
    const float* H;          // scanned pair histograms of features [f0, f0 + nf)
    const float* D;          // scanned derivative histograms [nf][B][L]
    int f0, nf, L, B;
    float l2, prior;
    float* gain;             // [nf][B]: gain of candidate (feature, bin); -inf where there is no candidate
};

// One block per candidate (feature, bin).  S = 2L unknowns, children ordered [left of leaf 0 .. L-1, right of 0 .. L-1].
// Shared memory: A [S][S] doubles (symmetrised weights, then the system, then its Cholesky factor), dvec [S], x [S],
// mx [S].  blockDim.x >= S.
__global__ void __launch_bounds__(128) cb_pair_solve_kernel(CbPairSolveArgs a) {
    extern __shared__ double sm[];
    const int L = a.L, S = 2 * L;
    double* A = sm;
    double* W = A + (size_t)S * S;          // symmetric weights (kept for the gain)
    double* dv = W + (size_t)S * S;
    double* x = dv + S;
    double* red = x + S;
    const int fl = blockIdx.x / a.B, t = blockIdx.x % a.B;
    const int f = a.f0 + fl;
    const int tid = threadIdx.x, nt = blockDim.x;
    const bool onehot = a.d.feat_onehot && a.d.feat_onehot[f];
    const int nb = a.d.feat_nb[f];
    const int ncand = onehot ? nb : nb - 1;
    const float fw = a.d.feat_weight ? a.d.feat_weight[f] : 1.0f;
    if (t >= ncand || fw <= 0.0f) {
        if (tid == 0) a.gain[(size_t)fl * a.B + t] = -INFINITY;
        return;
    }
    const size_t bs = (size_t)L * L * 4;
    const float* Hf = a.H + (size_t)fl * a.B * bs;
    const float* Ht = Hf + (size_t)t * bs;
    const float* Hlast = Hf + (size_t)(nb - 1) * bs;      // float features: totals = prefix at the last bin
    for (int c = tid; c < S * S; c += nt) W[c] = 0.0;
    __syncthreads();
    // off-diagonal weights of the directed pair cells, then symmetrise: W[u][v] = w(u -> v) + w(v -> u)
    for (int c = tid; c < L * L; c += nt) {
        const int la = c / L, lb = c % L;
        const float* h = Ht + (size_t)c * 4;
        double ll, lr, rl, rr;
        if (onehot) {
            // totals of a one-hot feature: sum over its values of the three stored configurations
            double tot = 0.0;
            for (int v = 0; v < nb; ++v) {
                const float* hv = Hf + (size_t)v * bs + (size_t)c * 4;
                tot += (double)hv[0] + 0.5 * ((double)hv[1] + (double)hv[2]);
            }
            rr = h[0]; rl = h[1]; lr = h[2];
            ll = tot - rr - rl - lr;
        } else {
            const float* hl = Hlast + (size_t)c * 4;
            const double tot = (double)hl[0] + (double)hl[2];
            ll = (double)h[1] + (double)h[3];
            lr = (double)h[0] - (double)h[1];
            rl = (double)h[2] - (double)h[3];
            rr = tot - ((double)h[0] + (double)h[2]);
        }
        // directed cell (child of winner, child of loser): add to both orientations of the symmetric matrix
        atomicAdd(&W[(size_t)la * S + lb], ll);             atomicAdd(&W[(size_t)lb * S + la], ll);
        atomicAdd(&W[(size_t)la * S + (lb + L)], lr);       atomicAdd(&W[(size_t)(lb + L) * S + la], lr);
        atomicAdd(&W[(size_t)(la + L) * S + lb], rl);       atomicAdd(&W[(size_t)lb * S + (la + L)], rl);
        atomicAdd(&W[(size_t)(la + L) * S + (lb + L)], rr); atomicAdd(&W[(size_t)(lb + L) * S + (la + L)], rr);
    }
    // derivative sums of the children
    for (int l = tid; l < L; l += nt) {
        const float* Df = a.D + (size_t)fl * a.B * L;
        double left, tot;
        if (onehot) {
            tot = 0.0;
            for (int v = 0; v < nb; ++v) tot += (double)Df[(size_t)v * L + l];
            left = tot - (double)Df[(size_t)t * L + l];
        } else {
            tot = (double)Df[(size_t)(nb - 1) * L + l];
            left = (double)Df[(size_t)t * L + l];
        }
        dv[l] = left;
        dv[l + L] = tot - left;
    }
    __syncthreads();
    // Laplacian M = diag(rowsum W) - W; system = M[:-1, :-1] + non_diag + I * (diag - non_diag + 1e-9)
    const double cellp = 1.0 / (double)S;
    const double non_diag = -(double)a.prior * cellp;
    const double diag = (double)a.prior * (1.0 - cellp) + (double)a.l2;
    const int n = S - 1;
    for (int r = tid; r < S; r += nt) {
        double rs = 0.0;
        for (int c = 0; c < S; ++c) rs += W[(size_t)r * S + c];
        x[r] = rs;                                  // row sums (x is free until the solve)
    }
    __syncthreads();
    for (int c = tid; c < S * S; c += nt) {
        const int r = c / S, k = c % S;
        const double m = (r == k ? x[r] : 0.0) - W[c];
        A[c] = m + non_diag + (r == k ? (diag - non_diag + 1e-9) : 0.0);
    }
    __syncthreads();
    // Cholesky of the leading n x n block (lower triangle, in place), right-looking
    for (int k = 0; k < n; ++k) {
        if (tid == 0) A[(size_t)k * S + k] = sqrt(fmax(A[(size_t)k * S + k], 1e-300));
        __syncthreads();
        const double dk = A[(size_t)k * S + k];
        for (int r = k + 1 + tid; r < n; r += nt) A[(size_t)r * S + k] /= dk;
        __syncthreads();
        const int m = n - k - 1;
        for (int c = tid; c < m * m; c += nt) {
            const int r = k + 1 + c / m, q = k + 1 + c % m;
            if (q <= r) A[(size_t)r * S + q] -= A[(size_t)r * S + k] * A[(size_t)q * S + k];
        }
        __syncthreads();
    }
    // forward and backward substitution by one warp-sized loop (n <= 127)
    if (tid == 0) {
        for (int r = 0; r < n; ++r) {
            double v = dv[r];
            for (int q = 0; q < r; ++q) v -= A[(size_t)r * S + q] * x[q];
            x[r] = v / A[(size_t)r * S + r];
        }
        for (int r = n - 1; r >= 0; --r) {
            double v = x[r];
            for (int q = r + 1; q < n; ++q) v -= A[(size_t)q * S + r] * x[q];
            x[r] = v / A[(size_t)r * S + r];
        }
        x[n] = 0.0;
        double mean = 0.0;
        for (int r = 0; r < S; ++r) mean += x[r];
        mean /= (double)S;
        for (int r = 0; r < S; ++r) x[r] -= mean;
    }
    __syncthreads();
    // gain = x.d - x'Mx / 2 with M x = rowsum * x - W x
    double part = 0.0;
    for (int r = tid; r < S; r += nt) {
        double rs = 0.0, wx = 0.0;
        for (int c = 0; c < S; ++c) { rs += W[(size_t)r * S + c]; wx += W[(size_t)r * S + c] * x[c]; }
        part += x[r] * dv[r] - 0.5 * x[r] * (rs * x[r] - wx);
    }
    part = cb_warp_sum_d(part);
    if ((tid & 31) == 0) red[tid >> 5] = part;
    __syncthreads();
    if (tid == 0) {
        double g = 0.0;
        for (int w = 0; w < (nt >> 5); ++w) g += red[w];
        a.gain[(size_t)fl * a.B + t] = (float)(g * (double)fw);
    }
}

CB_API long long cb_pair_hist_floats(int nfeat, int L, int B) { return (long long)nfeat * B * L * L * 4; }

// Pair histograms + derivative histograms of feature groups [g0, g0 + ng) (H and D zeroed by the caller), scanned.
CB_API int cb_pair_hist(const CbData* d, const unsigned short* leaf, const int* wi, const int* li, const float* w,
                        long long npairs, const float* der, int L, int B, int g0, int ng, float* H, float* D, float wmax,
                        int grid, cudaStream_t st) {
    CbPairHistArgs a{*d, leaf, wi, li, w, npairs, L, B, g0, ng, H};
    // wmax: the largest pair weight (> 0 selects the shared-memory kernel where the level's histogram fits)
    const size_t per_feat_bytes = (size_t)B * L * L * 4 * 4;
    // (one feature per block also fits up to 8 leaves, but then every block flushes 16K cells for a quarter of the work:
    // 108 ms per level at 2M x 700 against 22 ms for the sorted-pair kernel, which the caller uses from there on)
    bool smem_ok = wmax > 0.0f && npairs > 0 && ng > 0 && 4 * per_feat_bytes <= 96 * 1024;
    if (const char* e = getenv("CB200_PAIR_SMEM")) smem_ok = smem_ok && atoi(e) != 0;
    if (smem_ok) {
        static unsigned long long set = 0ull;
        if (cb_first_on_device(&set)) {
            cudaError_t e = cudaFuncSetAttribute(cb_pair_hist_smem_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
        }
        const float qs = 2147483647.0f / ((float)CB_PAIR_CHUNK * wmax) * 0.999f;
        const unsigned chunks = (unsigned)((npairs + CB_PAIR_CHUNK - 1) / CB_PAIR_CHUNK);
        cb_pair_hist_smem_kernel<4><<<dim3(chunks, (unsigned)ng), 256, 4 * per_feat_bytes, st>>>(a, qs);
    } else if (npairs > 0 && ng > 0) {
        // groups per range: the range's bin columns and histograms together within about half of the 126 MB L2
        const double per_group = (double)d->npad * 4.0 + 4.0 * (double)B * L * L * 16.0;
        int gpr = (int)(60.0e6 / per_group);
        if (gpr < 1) gpr = 1;
        if (gpr > 16) gpr = 16;
        if (gpr > ng) gpr = ng;
        const int ranges = (ng + gpr - 1) / gpr;
        cb_pair_hist_kernel<<<dim3((unsigned)grid, (unsigned)ranges), 256, 0, st>>>(a, gpr);
    }
    cb_pair_der_hist_kernel<<<grid, 256, 0, st>>>(*d, leaf, der, L, B, g0, ng, D);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    return 0;
}

CB_API int cb_pair_scan(const CbData* d, int f0, int nf, int L, int B, float* H, float* D, int grid, cudaStream_t st) {
    cb_pair_scan_kernel<<<grid, 256, 0, st>>>(*d, f0, nf, B, (long long)L * L * 4, H);
    cb_pair_scan_kernel<<<grid, 256, 0, st>>>(*d, f0, nf, B, (long long)L, D);
    return (int)cudaGetLastError();
}

CB_API int cb_pair_solve_smem_bytes(int L) { const int S = 2 * L; return (2 * S * S + 2 * S + 8) * 8; }

CB_API int cb_pair_solve(const CbData* d, const float* H, const float* D, int f0, int nf, int L, int B, float l2, float prior,
                         float* gain, cudaStream_t st) {
    const int smem = cb_pair_solve_smem_bytes(L);
    int dev = 0, optin = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (smem > optin) return -2;
    static unsigned long long set = 0ull;
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_pair_solve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    CbPairSolveArgs a{*d, H, D, f0, nf, L, B, l2, prior, gain};
    cb_pair_solve_kernel<<<(unsigned)(nf * B), 128, smem, st>>>(a);
    return (int)cudaGetLastError();
}
