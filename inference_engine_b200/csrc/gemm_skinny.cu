// Matrix product for a handful of rows (decode steps):  C[M, N] = X[M, K] * W[N, K]^T  in
// bfloat16 with 32-bit accumulation, M <= 16.
//
// With so few rows the product is a stream of the weight matrix through the SMs, so the kernel
// is built around keeping many bytes in flight rather than around the tensor cores' rate:
//   * the roles are swapped: 16 output features are the rows of the mma.m16n8k16 tile (A = a
//     16 x 16 piece of W), the step's tokens are its 8 columns (B = X^T), one or two column
//     tiles for M <= 8 or <= 16;
//   * every warp streams its own 16 features x K-slice of W with cp.async into its own shared
//     memory ring (16 features x 128 k per stage, XOR-swizzled for ldmatrix), independent of
//     the other warps: no block-wide barrier anywhere;
//   * matrices with few output features (the attention and down projections) would occupy few
//     SMs, so the inner dimension is cut into `splits` slices handled by different warps; the
//     partial sums go to `out[split][M][N]` and whoever consumes the product (the norm, the
//     rotary kernel, the activation) adds them in order -- no atomics, the same sum each time.
// The reference uses cuBLAS here (nn.Linear, engine/model/layers.py:126-129, 273-275).
#include "common.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int WARPS = 4;
constexpr int FB = 16;            // features per warp
#ifndef IE_SKINNY_BK
#define IE_SKINNY_BK 128
#endif
#ifndef IE_SKINNY_STAGES
#define IE_SKINNY_STAGES 7
#endif
constexpr int BK = IE_SKINNY_BK;  // k per stage (a multiple of 64)
constexpr int CH = BK / 8;        // 16-byte chunks per row and stage
constexpr int STAGES = IE_SKINNY_STAGES;
constexpr int STAGE_ELEMS = FB * BK;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Stage 16 rows x BK k of W, starting at (f0, k0); rows >= N and k >= k_end are zero-filled.
__device__ __forceinline__ void load_stage(bf16* stage, const bf16* __restrict__ W, int f0, int k0,
                                           int N, int K, int k_end, int lane) {
#pragma unroll
    for (int i = 0; i < FB * CH / 32; ++i) {
        int idx = i * 32 + lane;
        int r = idx / CH, c = idx % CH;
        int k = k0 + c * 8;
        bool valid = (f0 + r) < N && k < k_end;
        const bf16* src = valid ? W + (size_t)(f0 + r) * K + k : W;
        cp_async16(stage + (r * CH + (c ^ (r & 7))) * 8, src, valid);
    }
}

template <int NT, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, OutT* __restrict__ out,
                   int M, int N, int K, int k_per_split, int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int fblock = blockIdx.x * WARPS + warp;
    int f0 = fblock * FB;
    int split = blockIdx.y;
    if (f0 >= N) {  // whole warps leave; there is no block-wide barrier below
        ie_pdl_trigger();
        ie_pdl_wait();
        return;
    }
    bf16* ring = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * STAGES * STAGE_ELEMS;
    int k_begin = split * k_per_split;
    int k_end = min(K, k_begin + k_per_split);
    int n_tiles = k_begin < k_end ? (k_end - k_begin + BK - 1) / BK : 0;

    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

    // The weights do not depend on the kernel before this one: their first stages are on
    // their way before we wait for it (its output is our X).
    ie_pdl_trigger();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_tiles) load_stage(ring + s * STAGE_ELEMS, W, f0, k_begin + s * BK, N, K, k_end, lane);
        cp_async_commit();
    }
    ie_pdl_wait();
    int tok = lane >> 2;  // the token (column) whose X values this lane feeds
    for (int t = 0; t < n_tiles; ++t) {
        int pre = t + STAGES - 1;
        if (pre < n_tiles)
            load_stage(ring + (pre % STAGES) * STAGE_ELEMS, W, f0, k_begin + pre * BK, N, K, k_end, lane);
        cp_async_commit();
        // X fragments of this tile straight from global memory (small, shared by all warps:
        // they stay in L1/L2); issued before the wait so they overlap the weight stream
        int k0 = k_begin + t * BK;
        unsigned xb[NT][BK / 16][2];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            int row = n * 8 + tok;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
                int k = k0 + ks * 16 + (lane & 3) * 2;
                bool ok = row < M;
                xb[n][ks][0] = (ok && k < k_end) ? *reinterpret_cast<const unsigned*>(X + (size_t)row * K + k) : 0u;
                xb[n][ks][1] = (ok && k + 8 < k_end) ? *reinterpret_cast<const unsigned*>(X + (size_t)row * K + k + 8) : 0u;
            }
        }
        cp_async_wait<STAGES - 1>();
        __syncwarp();
        const bf16* stage = ring + (t % STAGES) * STAGE_ELEMS;
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            unsigned a[4];
            int r = (lane & 7) + (((lane >> 3) & 1) << 3);
            int c = ks * 2 + (lane >> 4);
            ldmatrix_x4(a, stage + (r * CH + (c ^ (r & 7))) * 8);
#pragma unroll
            for (int n = 0; n < NT; ++n) mma_bf16(acc[n], a, xb[n][ks][0], xb[n][ks][1]);
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    // acc[n][0,1]: feature f0 + lane/4, tokens n*8 + (lane%4)*2 + {0,1}; acc[n][2,3]: feature + 8
    OutT* dst = out + (size_t)split * M * N;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int f = f0 + (lane >> 2) + ((j >> 1) << 3);
            int m = n * 8 + (lane & 3) * 2 + (j & 1);
            if (f < N && m < M) ie_store(dst + (size_t)m * N + f, acc[n][j]);
        }
    }
}

constexpr size_t SMEM_BYTES = (size_t)WARPS * STAGES * STAGE_ELEMS * sizeof(bf16);

template <int NT, typename OutT>
int launch(const bf16* X, const bf16* W, OutT* out, int M, int N, int K, int k_per_split, int splits,
           cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NT, OutT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int fblocks = (N + FB - 1) / FB;
    dim3 grid((fblocks + WARPS - 1) / WARPS, splits);
    return ie_launch(gemm_skinny_kernel<NT, OutT>, grid, dim3(WARPS * 32), SMEM_BYTES, s, X, W, out, M, N, K,
                     k_per_split, splits);
}
}  // namespace

IE_API void ie_set_pdl(int enabled) { ie_pdl_enabled() = enabled ? 1 : 0; }

// `out`: [splits, M, N].  With splits > 1 it must be 32-bit and holds partial sums over slices
// of `k_per_split` (a multiple of 16) of the inner dimension; with splits == 1 it is the
// product, 32-bit or bfloat16.  K must be a multiple of 8 (rows of W start on 16 bytes).
IE_API int ie_gemm_skinny_bf16(const void* X, const void* W, void* out, int out_dtype, int M, int N,
                               int K, int k_per_split, int splits, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K % 8 != 0 || splits < 1 || k_per_split % 16 != 0 || (long long)k_per_split * splits < K ||
        (splits > 1 && out_dtype != IE_F32))
        return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (out_dtype == IE_F32)
        return M <= 8 ? launch<1, float>(x, w, (float*)out, M, N, K, k_per_split, splits, s)
                      : launch<2, float>(x, w, (float*)out, M, N, K, k_per_split, splits, s);
    return M <= 8 ? launch<1, bf16>(x, w, (bf16*)out, M, N, K, k_per_split, splits, s)
                  : launch<2, bf16>(x, w, (bf16*)out, M, N, K, k_per_split, splits, s);
}
