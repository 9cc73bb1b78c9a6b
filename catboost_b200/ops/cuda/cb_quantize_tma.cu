// K1 with TMA staging: float32 rows -> packed one-byte bins  (same contract as cb_quantize in cb_kernels.cu; reference:
// catboost/cuda/gpu_data/kernel/binarize.cu:37, catboost/libs/data/quantization.cpp).
//
// The input is row-major [n][F] while the store is feature-group-major, so the matrix has to be transposed on the way:
// a tile of 256 rows x 32 features is brought into shared memory by one tiled bulk copy (cp.async.bulk.tensor.2d, the
// 128-byte swizzle keeps the later column-wise reads free of bank conflicts), double-buffered so that the copy of the
// next tile overlaps the search of the current one.  The borders of the 32 features sit in shared memory; a thread
// owns one row of the tile, reads it as eight float4 (one per feature group), runs the four binary searches of a group
// and writes one packed word per group -- consecutive lanes write consecutive documents of the same group row.
//
// Every wait on a copy is bounded: when it runs out the block records CB_QUANTIZE_TMA_TIMEOUT in *status, gives its
// copies in flight a second bounded chance to land, and returns.
#include "cb_common.cuh"
#include <cuda.h>

#define CBQ_ROWS 256
#define CBQ_FBOX 32
#define CBQ_STAGE_BYTES (CBQ_ROWS * CBQ_FBOX * 4)
#define CBQ_BORDER_STRIDE 256
#define CB_QUANTIZE_TMA_TIMEOUT 0x51

__device__ __forceinline__ unsigned int cbq_smem_u32(const void* p) {
    return (unsigned int)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ bool cbq_wait(unsigned int bar, unsigned int parity, int limit) {
    for (int it = 0; it < limit; ++it) {
        unsigned int ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__global__ void __launch_bounds__(CBQ_ROWS) cb_quantize_tma_kernel(const __grid_constant__ CUtensorMap tmap, long long n,
                                                                   int F, const float* __restrict__ borders,
                                                                   const int* __restrict__ border_off,
                                                                   const unsigned char* __restrict__ nan_is_max,
                                                                   uint32_t* __restrict__ bins, long long npad,
                                                                   long long doc_offset, int* status) {
    extern __shared__ unsigned char cbq_smem_raw[];
    // the swizzle pattern repeats every 1024 bytes: the stages start on a 1024-byte boundary of the shared window
    unsigned char* cbq_smem = cbq_smem_raw + ((1024u - (cbq_smem_u32(cbq_smem_raw) & 1023u)) & 1023u);
    // [2 stages][256 rows][128 B] | borders [32][256] floats | counts [32] | nan flags [32] | 2 mbarriers
    float* sb = reinterpret_cast<float*>(cbq_smem + 2 * CBQ_STAGE_BYTES);
    int* snb = reinterpret_cast<int*>(sb + CBQ_FBOX * CBQ_BORDER_STRIDE);
    int* snan = snb + CBQ_FBOX;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(snan + CBQ_FBOX);
    const unsigned int bar0 = cbq_smem_u32(bars), bar1 = cbq_smem_u32(bars + 1);
    const unsigned int st0 = cbq_smem_u32(cbq_smem), st1 = cbq_smem_u32(cbq_smem + CBQ_STAGE_BYTES);
    const int tid = threadIdx.x;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long tiles = (n + CBQ_ROWS - 1) / CBQ_ROWS;
    const int nbox = (F + CBQ_FBOX - 1) / CBQ_FBOX;
    const int G = (F + 3) >> 2;
    unsigned int phase0 = 0, phase1 = 0;
    __shared__ int s_fail;
    if (tid == 0) s_fail = 0;
    for (int fb = 0; fb < nbox; ++fb) {
        __syncthreads();                             // everyone is done with the previous box's borders
        for (int j = 0; j < CBQ_FBOX; ++j) {
            const int f = fb * CBQ_FBOX + j;
            const int b0 = f < F ? border_off[f] : 0, b1 = f < F ? border_off[f + 1] : 0;
            for (int k = tid; k < b1 - b0; k += blockDim.x) sb[j * CBQ_BORDER_STRIDE + k] = borders[b0 + k];
            if (tid == 0) { snb[j] = b1 - b0; snan[j] = (f < F && nan_is_max && nan_is_max[f]) ? 1 : 0; }
        }
        __syncthreads();
        // first copy of this box
        long long t = blockIdx.x;
        int stage = 0;
        if (tid == 0 && t < tiles) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar0), "r"(CBQ_STAGE_BYTES) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                         :: "r"(st0), "l"(&tmap), "r"(fb * CBQ_FBOX), "r"((int)(t * CBQ_ROWS)), "r"(bar0) : "memory");
        }
        for (; t < tiles; t += gridDim.x) {
            const long long tn = t + gridDim.x;
            // the other stage was released by the barrier at the end of the previous round
            if (tid == 0 && tn < tiles) {
                const unsigned int nb_ = stage ? bar0 : bar1, ns_ = stage ? st0 : st1;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(nb_), "r"(CBQ_STAGE_BYTES) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             :: "r"(ns_), "l"(&tmap), "r"(fb * CBQ_FBOX), "r"((int)(tn * CBQ_ROWS)), "r"(nb_) : "memory");
            }
            const unsigned int bar = stage ? bar1 : bar0;
            const unsigned int parity = stage ? phase1 : phase0;
            if (!cbq_wait(bar, parity, 1 << 22)) {
                atomicExch(status, CB_QUANTIZE_TMA_TIMEOUT);
                cbq_wait(bar, parity, 1 << 22);      // a second bounded chance for the copy in flight to land
                s_fail = 1;
            }
            __syncthreads();
            if (s_fail) {
                // let the other stage's copy land as well before the shared memory is given back
                cbq_wait(stage ? bar0 : bar1, stage ? phase0 : phase1, 1 << 22);
                return;
            }
            if (stage) phase1 ^= 1u; else phase0 ^= 1u;
            const unsigned char* tile = cbq_smem + stage * CBQ_STAGE_BYTES;
            const long long i = t * CBQ_ROWS + tid;
            const unsigned char* row = tile + tid * 128;
#pragma unroll 2
            for (int gl = 0; gl < CBQ_FBOX / 4; ++gl) {
                const int g = fb * (CBQ_FBOX / 4) + gl;
                if (g >= G) break;
                const float4 v4 = *reinterpret_cast<const float4*>(row + ((gl ^ (tid & 7)) << 4));
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
                uint32_t word = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int fj = gl * 4 + j;
                    const int nbd = snb[fj];
                    const float v = vv[j];
                    // count of borders < v by fixed power-of-two steps: no data-dependent trip count, so the four
                    // searches of a group (and those of the next group) overlap their shared-memory latency
                    const float* b = sb + fj * CBQ_BORDER_STRIDE;
                    int pos = 0;
#pragma unroll
                    for (int step = 128; step > 0; step >>= 1) {
                        const int idx = pos + step;
                        const float bv = (idx <= nbd) ? b[idx - 1] : 3.4e38f;
                        if (idx <= nbd && bv < v) pos = idx;
                    }
                    const int bin = (v != v) ? (snan[fj] ? nbd : 0) : pos;
                    word |= (uint32_t)bin << (8 * j);
                }
                if (i < n) bins[(long long)g * npad + doc_offset + i] = word;
            }
            __syncthreads();                         // the stage may be refilled from here on
            stage ^= 1;
        }
        // nothing is in flight here; the next box starts again on stage 0, whose barrier keeps its own parity
    }
}

typedef CUresult (*CbEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static CbEncodeTiled cb_encode_tiled() {
    static CbEncodeTiled fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<CbEncodeTiled>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// Returns 0 when the kernel was enqueued, -2 when the layout does not qualify (row pitch or base not 16-byte aligned,
// no tensor-map encoder) -- the caller then uses cb_quantize --, a CUDA error code otherwise.  *status (device int,
// zero on entry) receives CB_QUANTIZE_TMA_TIMEOUT if a copy did not arrive in time.
CB_API int cb_quantize_tma(const float* X, long long n, int F, long long ldx, const float* borders, const int* border_off,
                           const unsigned char* nan_is_max, uint32_t* bins, long long npad, long long doc_offset,
                           int* status, cudaStream_t st) {
    if (n <= 0) return 0;
    if ((ldx * 4) % 16 != 0 || (reinterpret_cast<unsigned long long>(X) & 15ull) != 0 || n >= (1ll << 31)) return -2;
    CbEncodeTiled enc = cb_encode_tiled();
    if (!enc) return -2;
    CUtensorMap tm;
    const cuuint64_t gdim[2] = {(cuuint64_t)F, (cuuint64_t)n};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 4};
    const cuuint32_t box[2] = {CBQ_FBOX, CBQ_ROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(X), gdim, gstride, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -2;
    const int smem = 1024 + 2 * CBQ_STAGE_BYTES + CBQ_FBOX * CBQ_BORDER_STRIDE * 4 + 2 * CBQ_FBOX * 4 + 16;
    static unsigned long long set = 0ull;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cb_first_on_device(&set)) {
        cudaError_t e = cudaFuncSetAttribute(cb_quantize_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { cudaGetLastError(); set = 0ull; return (int)e; }
    }
    const long long tiles = (n + CBQ_ROWS - 1) / CBQ_ROWS;
    long long grid = (long long)sms * 2;
    if (grid > tiles) grid = tiles;
    cb_quantize_tma_kernel<<<(unsigned)grid, CBQ_ROWS, smem, st>>>(tm, n, F, borders, border_off, nan_is_max, bins, npad,
                                                                  doc_offset, status);
    const cudaError_t le = cudaGetLastError();
    return le == cudaSuccess ? 0 : (int)le;
}
