// Matrix product for a handful of rows, fed by the tensor memory accelerator:
//   C[M, N] = X[M, K] * W[N, K]^T,  bfloat16 in, 32-bit accumulation, M <= 16.
//
// A decode step is a stream of weights through the SMs.  Here one elected thread per block
// issues cp.async.bulk.tensor (TMA) copies of 128-feature x 64-k tiles of W into a deep ring
// in shared memory (128-byte swizzle, so ldmatrix reads them without bank conflicts); four
// consumer warps wait on the tiles' mbarriers, multiply with mma.m16n8k16 (the 16 output
// features of a tile row are the rows of the instruction, the step's tokens its columns) and
// hand the slots back through a second set of mbarriers.  Issuing a 16 KB tile costs one
// instruction instead of a thousand 16-byte copies, which is what lets a block keep about
// 150 KB in flight and the SM stream at its full rate.
//
// The weights do not depend on the kernel that runs before this one, so under programmatic
// dependent launch the producer fills the ring before it waits for that kernel; only the copy
// of X (the kernel's activations, one TMA box per 64 k) comes after the wait.
//
// Matrices with few output features are also cut along k (grid.y = splits) so that every SM
// has a block; the partial sums go to out[split][M][N] and the consumer of the product adds
// them in order.  Every wait on an mbarrier is bounded: a block that waits too long sets the
// error word, drains and leaves.
// The reference uses cuBLAS here (nn.Linear, engine/model/layers.py:126-129, 273-275).
#include "common.cuh"
#include <cuda.h>

namespace {
typedef __nv_bfloat16 bf16;
constexpr int CWARPS = 4;                 // consumer warps
constexpr int THREADS = (CWARPS + 1) * 32;  // + one producer warp
constexpr int BN = 128;                   // features per block (32 per consumer warp)
constexpr int BK = 64;                    // k per stage: 128 bytes per row, one swizzle atom
constexpr int XROWS = 16;                 // rows of X staged (M <= 16; missing rows read as zero)
constexpr int STAGE_BYTES = BN * BK * 2;  // 16 KB
constexpr int XBOX_BYTES = XROWS * BK * 2;  // 2 KB per 64 k
constexpr int MAX_KBLOCKS = 32;           // k-slice of a block: at most 2048
constexpr int MAX_STAGES = 9;
constexpr long long SPIN_LIMIT = 20000000;  // about ten milliseconds of polling

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false when the phase did not complete within SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, int parity) {
    unsigned addr = smem_u32(bar);
    for (long long spin = 0; spin < SPIN_LIMIT; ++spin) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared memory: [ring: stages x 16 KB][X: kblocks x 2 KB][barriers], 1024-byte aligned.
template <int NT, typename OutT>
__global__ void __launch_bounds__(THREADS)
gemm_tma_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                OutT* __restrict__ out, int M, int N, int K, int kblocks_per_split, int stages, int* err) {
    extern __shared__ unsigned char smem_raw[];
    // swizzled TMA tiles want 1024-byte alignment; the launch reserves the slack
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * BN;
    int split = blockIdx.y;
    int total_kblocks = (K + BK - 1) / BK;
    int kb0 = split * kblocks_per_split;
    int nkb = min(kblocks_per_split, total_kblocks - kb0);
    if (nkb < 0) nkb = 0;
    unsigned char* ring = smem;
    unsigned char* xs = smem + (size_t)stages * STAGE_BYTES;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(xs + (size_t)MAX_KBLOCKS * XBOX_BYTES);
    unsigned long long* empty = full + MAX_STAGES;
    unsigned long long* x_full = empty + MAX_STAGES;
    __shared__ int failed;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CWARPS);
        }
        mbar_init(x_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    ie_pdl_trigger();

    if (warp == CWARPS) {
        // ---- producer: one thread ----
        if (lane == 0) {
            int issued = 0;
            // the weights need nobody's results: fill the ring right away
            for (; issued < nkb && issued < stages; ++issued) {
                mbar_expect_tx(&full[issued], STAGE_BYTES);
                tma_load_2d(ring + (size_t)issued * STAGE_BYTES, &w_map, (kb0 + issued) * BK, n0, &full[issued]);
            }
            ie_pdl_wait();  // X is the previous kernel's output
            if (nkb > 0) {
                mbar_expect_tx(x_full, nkb * XBOX_BYTES);
                for (int kb = 0; kb < nkb; ++kb)
                    tma_load_2d(xs + (size_t)kb * XBOX_BYTES, &x_map, (kb0 + kb) * BK, 0, x_full);
            }
            for (; issued < nkb; ++issued) {
                int s = issued % stages;
                int round = issued / stages;  // this slot's round-th reuse: wait for its release
                if (!mbar_wait(&empty[s], (round - 1) & 1)) { failed = 1; break; }
                mbar_expect_tx(&full[s], STAGE_BYTES);
                tma_load_2d(ring + (size_t)s * STAGE_BYTES, &w_map, (kb0 + issued) * BK, n0, &full[s]);
            }
        } else {
            ie_pdl_wait();
        }
    } else {
        // ---- consumers: warp w owns features n0 + 32 w .. + 31 (two 16-row tiles) ----
        ie_pdl_wait();
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int n = 0; n < NT; ++n) acc[mt][n][0] = acc[mt][n][1] = acc[mt][n][2] = acc[mt][n][3] = 0.f;
        bool ok = nkb == 0 || mbar_wait(x_full, 0);
        unsigned ring_addr = smem_u32(ring), xs_addr = smem_u32(xs);
        for (int kb = 0; kb < nkb && ok; ++kb) {
            int s = kb % stages;
            if (!mbar_wait(&full[s], (kb / stages) & 1)) { ok = false; break; }
            unsigned wt = ring_addr + s * STAGE_BYTES;
            unsigned xt = xs_addr + kb * XBOX_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
                unsigned xb[4];
                {   // tokens (lane & 7) + 8 (lane >> 4), k chunk ks*2 + ((lane >> 3) & 1)
                    int r = (lane & 7) + ((lane >> 4) << 3);
                    int c = ks * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(xb, xt + r * 128 + ((c ^ (r & 7)) << 4));
                }
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    unsigned a[4];
                    int r = warp * 32 + mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    int c = ks * 2 + (lane >> 4);
                    ldmatrix_x4(a, wt + r * 128 + ((c ^ (r & 7)) << 4));
                    mma_bf16(acc[mt][0], a, xb[0], xb[1]);
                    if (NT == 2) mma_bf16(acc[mt][NT - 1], a, xb[2], xb[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) failed = 1;
        // acc[mt][n][0,1]: feature f + lane/4, tokens n*8 + (lane%4)*2 + {0,1}; [2,3]: feature + 8
        OutT* dst = out + (size_t)split * M * N;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int f = n0 + warp * 32 + mt * 16 + (lane >> 2) + ((j >> 1) << 3);
                    int m = n * 8 + (lane & 3) * 2 + (j & 1);
                    if (f < N && m < M) ie_store(dst + (size_t)m * N + f, acc[mt][n][j]);
                }
    }
    __syncthreads();
    if (threadIdx.x == 0 && failed) ie_report(err, IE_ERR_TIMEOUT, blockIdx.x, blockIdx.y);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// A row-major [rows, cols] bfloat16 matrix as a 2-D tensor map with boxes of box_rows x 64
// columns and the 128-byte swizzle; out-of-range elements read as zero.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, typename OutT>
int launch(const CUtensorMap& wm, const CUtensorMap& xm, OutT* out, int M, int N, int K, int kblocks_per_split,
           int splits, int* err, cudaStream_t s) {
    int stages = MAX_STAGES;
    size_t smem = (size_t)stages * STAGE_BYTES + (size_t)MAX_KBLOCKS * XBOX_BYTES + (2 * MAX_STAGES + 1) * 8 + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tma_kernel<NT, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, splits);
    return ie_launch(gemm_tma_kernel<NT, OutT>, grid, dim3(THREADS), smem, s, wm, xm, out, M, N, K,
                     kblocks_per_split, stages, err);
}
}  // namespace

// 1 if the driver offers tensor-map encoding (it always does on the GPUs this library targets).
IE_API int ie_gemm_tma_available() { return encode_fn() != nullptr ? 1 : 0; }

// `out`: [splits, M, N]; with splits > 1 32-bit partial sums over slices of `kblocks_per_split`
// blocks of 64 k (at most 32 blocks per slice); with splits == 1 the product, 32-bit or
// bfloat16.  X and W must be 16-byte aligned with K a multiple of 8.
IE_API int ie_gemm_tma_bf16(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K,
                            int kblocks_per_split, int splits, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    int total_kblocks = (K + BK - 1) / BK;
    if (M > XROWS || K % 8 != 0 || splits < 1 || kblocks_per_split < 1 || kblocks_per_split > MAX_KBLOCKS ||
        (long long)kblocks_per_split * splits < total_kblocks || (splits > 1 && out_dtype != IE_F32) ||
        ((uintptr_t)X & 15) != 0 || ((uintptr_t)W & 15) != 0)
        return (int)cudaErrorInvalidValue;
    CUtensorMap wm, xm;
    if (!make_map(&wm, W, N, K, BN) || !make_map(&xm, X, M, K, XROWS)) return (int)cudaErrorNotSupported;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_F32)
        return M <= 8 ? launch<1, float>(wm, xm, (float*)out, M, N, K, kblocks_per_split, splits, err, s)
                      : launch<2, float>(wm, xm, (float*)out, M, N, K, kblocks_per_split, splits, err, s);
    return M <= 8 ? launch<1, bf16>(wm, xm, (bf16*)out, M, N, K, kblocks_per_split, splits, err, s)
                  : launch<2, bf16>(wm, xm, (bf16*)out, M, N, K, kblocks_per_split, splits, err, s);
}
