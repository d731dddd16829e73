// True 32-bit matrix product on the CUDA cores:  C[M, N] = A[M, K] * W[N, K]^T.
//
// No tensor-core mode is involved (tcgen05 has no 32-bit input kind and TF32 drops mantissa
// bits), so this is the matrix product of the engine's 32-bit path.  Every output element is
// one chain of fused multiply-adds over k = 0 .. K-1 in increasing order: the result of a row
// does not depend on how many other rows the step has, on where the row sits in the batch or
// on the tile it falls into.  That makes 32-bit logits identical however the tokens were cut
// into steps.  The reference's 32-bit path is cuBLAS with TF32 off (PyTorch's default).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    ie_pdl_trigger();
    ie_pdl_wait();
    int tid = threadIdx.x;
    int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, each a 4 x 4 patch
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // Each thread loads 4 consecutive k of one row of A and of W per tile.
    int lr = tid / 4, lk = (tid % 4) * 4;
    bool vec = (K % 4 == 0);
    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
        if (gm < M) {
            const float* p = A + (size_t)gm * K + gk;
            if (vec && gk + 3 < K) { float4 v = *reinterpret_cast<const float4*>(p); a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
            else { for (int i = 0; i < 4; ++i) if (gk + i < K) a[i] = p[i]; }
        }
        if (gn < N) {
            const float* p = W + (size_t)gn * K + gk;
            if (vec && gk + 3 < K) { float4 v = *reinterpret_cast<const float4*>(p); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
            else { for (int i = 0; i < 4; ++i) if (gk + i < K) w[i] = p[i]; }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { As[lk + i][lr] = a[i]; Ws[lk + i][lr] = w[i]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float4 av = *reinterpret_cast<const float4*>(&As[k][ty * TM]);
            float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * TN]);
            float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}
}  // namespace

IE_API int ie_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, W, C, M, N, K);
    return IE_LAUNCH_CHECK();
}
