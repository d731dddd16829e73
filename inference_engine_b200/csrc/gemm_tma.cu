// Matrix product for a handful of rows, fed by the tensor memory accelerator:
//   C[M, N] = X[M, K] * W[N, K]^T,  bfloat16 in, 32-bit accumulation, M <= 16.
//
// A decode step is a stream of weights through the SMs.  Here one elected thread per block
// issues cp.async.bulk.tensor (TMA) copies of W into a ring in shared memory (128-byte
// swizzle, so ldmatrix reads the tiles without bank conflicts); four consumer warps wait on
// the copies' mbarriers, multiply with mma.m16n8k16 (the 16 output features of a tile row are
// the rows of the instruction, the step's tokens its columns) and hand the slots back through
// a second set of mbarriers.
//
// The copy engine spends a fixed time on every copy before it streams (measured on this part:
// 16 KB boxes of a 2-D map reach 5.0 TB/s over all SMs, 64 KB boxes of a 3-D map 6.7 TB/s, the
// rate of a plain copy).  So W[N, K] is described as a 3-D tensor (64 k, N features, K/64 k
// blocks) and one copy brings 128 features x up to four k blocks, which land as consecutive
// 128 x 64 tiles of the ring.  When K is no multiple of 64 the 2-D form with one k block per
// copy is used.
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
#include "tma.cuh"

using namespace ie_tma;

namespace {
constexpr int CWARPS = 4;                 // consumer warps
constexpr int THREADS = (CWARPS + 1) * 32;  // + one producer warp
constexpr int BN = 128;                   // features per block (32 per consumer warp)
constexpr int BK = 64;                    // k per stage: 128 bytes per row, one swizzle atom
constexpr int STAGE_BYTES = BN * BK * 2;  // 16 KB: one k block of 128 features
constexpr int MAX_KBLOCKS = 32;           // k-slice of a block: at most 2048
constexpr int MAX_OPS = 12;               // copies in flight (ring slots)
constexpr int MAX_KPO = 4;                // k blocks per copy
// Shared memory for tiles: what the 227 KB of an SM leave beside X (8 NT rows x 2048 k)
__host__ __device__ constexpr int ring_bytes(int nt) { return nt == 1 ? 192 * 1024 : 160 * 1024; }

#ifdef IE_TEST_STARVE
// Self-test build only (kernels/build.py: build_selftest).  While this flag is set, every block
// leaves out the last box of X although the barrier was told to expect all of them: the
// consumers' wait for X must run out, the block must record IE_ERR_TIMEOUT and return.  The
// copies of W that were asked for meanwhile are few and complete long before the wait gives up.
static __device__ int g_starve_last_x;
#endif

// Shared memory: [ring: ops x kpo x 16 KB][X: kblocks x (8 NT rows x 128 B)][barriers], 1024-byte aligned.
// NT: 8-token column tiles (1: M <= 8, 2: M <= 16).  `kpo` k blocks per copy (3-D map) or 1 (2-D map).
// GATED: W holds gates and ups alternating in blocks of 16 rows (rows 32 b .. 32 b + 15 the gates
// 16 b .. 16 b + 15, the next 16 rows their ups), so a consumer warp's two 16-row tiles are 16
// gates and their ups, and a thread holds a gate and its up for the same token.  The kernel then
// writes out[m][i] = silu(gate_i) * up_i, silu(g) = g / (1 + exp(-g)) (engine/model/layers.py:277-281),
// N / 2 values per token, instead of the product itself; the inner dimension is not cut (one split).
template <int NT, typename OutT, bool GATED = false>
__global__ void __launch_bounds__(THREADS)
gemm_tma_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                OutT* __restrict__ out, int M, int N, int K, int kblocks_per_split, int ops, int kpo, int w3d,
                int* err) {
    constexpr int XR = 8 * NT;                 // rows of X staged (missing rows read as zero)
    constexpr int XBOX_BYTES = XR * BK * 2;
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
    int nops = (nkb + kpo - 1) / kpo;          // copies this block asks for
    int op_bytes = kpo * STAGE_BYTES;
    unsigned char* ring = smem;
    unsigned char* xs = smem + (size_t)ring_bytes(NT);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(xs + (size_t)MAX_KBLOCKS * XBOX_BYTES);
    unsigned long long* empty = full + MAX_OPS;
    unsigned long long* x_full = empty + MAX_OPS;
    __shared__ int failed;

    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < ops; ++s) {
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
            auto copy_w = [&](int o) {  // copy o of this block into slot o % ops
                int s = o % ops;
                mbar_expect_tx(&full[s], op_bytes);
                if (w3d)
                    tma_load_3d(ring + (size_t)s * op_bytes, &w_map, 0, n0, kb0 + o * kpo, &full[s]);
                else
                    tma_load_2d(ring + (size_t)s * op_bytes, &w_map, (kb0 + o) * BK, n0, &full[s]);
            };
            int issued = 0;
            // the weights need nobody's results: fill the ring right away
            for (; issued < nops && issued < ops; ++issued) copy_w(issued);
            ie_pdl_wait();  // X is the previous kernel's output
            if (nkb > 0) {
                mbar_expect_tx(x_full, nkb * XBOX_BYTES);
                for (int kb = 0; kb < nkb; ++kb) {
#ifdef IE_TEST_STARVE
                    if (g_starve_last_x && kb == nkb - 1) break;
#endif
                    tma_load_2d(xs + (size_t)kb * XBOX_BYTES, &x_map, (kb0 + kb) * BK, 0, x_full);
                }
            }
            for (; issued < nops; ++issued) {
                int round = issued / ops;  // this slot's round-th reuse: wait for its release
                if (!mbar_wait(&empty[issued % ops], (round - 1) & 1)) { failed = 1; break; }
                copy_w(issued);
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
        for (int o = 0; o < nops && ok; ++o) {
            int s = o % ops;
            if (!mbar_wait(&full[s], (o / ops) & 1)) { ok = false; break; }
            int kbs = min(kpo, nkb - o * kpo);  // a copy may reach beyond the block's slice of k
            for (int j = 0; j < kbs; ++j) {
                unsigned wt = ring_addr + s * op_bytes + j * STAGE_BYTES;
                unsigned xt = xs_addr + (o * kpo + j) * XBOX_BYTES;
#pragma unroll
                for (int ks2 = 0; ks2 < BK / 32; ++ks2) {
                    // X as B fragments of two 16-wide k steps
                    unsigned xb[2][2 * NT];
                    if (NT == 1) {  // 8 tokens: one ldmatrix brings both steps (k chunks 4 ks2 .. + 3)
                        unsigned t[4];
                        int r = lane & 7, c = ks2 * 4 + (lane >> 3);
                        ldmatrix_x4(t, xt + r * 128 + ((c ^ (r & 7)) << 4));
                        xb[0][0] = t[0]; xb[0][1] = t[1]; xb[1][0] = t[2]; xb[1][1] = t[3];
                    } else {        // 16 tokens: tokens (lane & 7) + 8 (lane >> 4), k chunk + ((lane >> 3) & 1)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            unsigned t[4];
                            int r = (lane & 7) + ((lane >> 4) << 3);
                            int c = (ks2 * 2 + h) * 2 + ((lane >> 3) & 1);
                            ldmatrix_x4(t, xt + r * 128 + ((c ^ (r & 7)) << 4));
                            xb[h][0] = t[0]; xb[h][1] = t[1]; xb[h][2 * NT - 2] = t[2]; xb[h][2 * NT - 1] = t[3];
                        }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        int ks = ks2 * 2 + h;
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            unsigned a[4];
                            int r = warp * 32 + mt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                            int c = ks * 2 + (lane >> 4);
                            ldmatrix_x4(a, wt + r * 128 + ((c ^ (r & 7)) << 4));
                            mma_bf16(acc[mt][0], a, xb[h][0], xb[h][1]);
                            if (NT == 2) mma_bf16(acc[mt][NT - 1], a, xb[h][2 * NT - 2], xb[h][2 * NT - 1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) failed = 1;
        // acc[mt][n][0,1]: feature f + lane/4, tokens n*8 + (lane%4)*2 + {0,1}; [2,3]: feature + 8
        OutT* dst = out + (size_t)split * M * N;
        if constexpr (GATED) {
            int inter = N / 2;
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int gate_row = n0 + warp * 32 + (lane >> 2) + ((j >> 1) << 3);  // its up: 16 rows on
                    int i = (n0 >> 1) + warp * 16 + (lane >> 2) + ((j >> 1) << 3);
                    int m = n * 8 + (lane & 3) * 2 + (j & 1);
                    float g = acc[0][n][j], u = acc[1][n][j];
                    if (gate_row + 16 < N && m < M)
                        ie_store(out + (size_t)m * inter + i, __fdividef(g, 1.0f + __expf(-g)) * u);
                }
        } else
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

template <int NT, typename OutT, bool GATED = false>
int launch(const void* X, const void* W, OutT* out, int M, int N, int K, int kblocks_per_split, int splits,
           int* err, cudaStream_t s) {
    // k blocks per copy: as many as divide the block's slice (a copy must not reach into the
    // next block's slice: that would read those bytes twice)
    int kpo = 1, w3d = 0;
    CUtensorMap wm, xm;
    if (K % BK == 0) {
        // (16 tokens leave room for 160 KB of tiles: 32 KB copies keep five of them in flight)
        for (kpo = NT == 1 ? MAX_KPO : 2; kpo > 1 && kblocks_per_split % kpo != 0; kpo >>= 1) {}
        w3d = 1;
        if (!make_map_bf16_3d(&wm, W, N, K, BN, kpo)) return (int)cudaErrorNotSupported;
    } else if (!make_map_bf16(&wm, W, N, K, BN)) {
        return (int)cudaErrorNotSupported;
    }
    if (!make_map_bf16(&xm, X, M, K, 8 * NT)) return (int)cudaErrorNotSupported;
    int ops = ring_bytes(NT) / (kpo * STAGE_BYTES);
    if (ops > MAX_OPS) ops = MAX_OPS;
    size_t smem = (size_t)ring_bytes(NT) + (size_t)MAX_KBLOCKS * 8 * NT * BK * 2 + (2 * MAX_OPS + 1) * 8 + 1024;
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, gemm_tma_kernel<NT, OutT, GATED>, smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((N + BN - 1) / BN, splits);
    return ie_launch(gemm_tma_kernel<NT, OutT, GATED>, grid, dim3(THREADS), smem, s, wm, xm, out, M, N, K,
                     kblocks_per_split, ops, kpo, w3d, err);
}
}  // namespace

#ifdef IE_TEST_STARVE
IE_API int ie_test_starve_tma(int on) {
    return (int)cudaMemcpyToSymbol(g_starve_last_x, &on, sizeof(int));
}
#endif

// 1 if the driver offers tensor-map encoding (it always does on the GPUs this library targets).
IE_API int ie_gemm_tma_available() { return encode_fn() != nullptr ? 1 : 0; }

// `out`: [splits, M, N]; with splits > 1 32-bit partial sums over slices of `kblocks_per_split`
// blocks of 64 k (at most 32 blocks per slice); with splits == 1 the product, 32-bit or
// bfloat16.  X and W must be 16-byte aligned with K a multiple of 8.
IE_API int ie_gemm_tma_bf16(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K,
                            int kblocks_per_split, int splits, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    int total_kblocks = (K + BK - 1) / BK;
    if (M > 16 || K % 8 != 0 || splits < 1 || kblocks_per_split < 1 || kblocks_per_split > MAX_KBLOCKS ||
        (long long)kblocks_per_split * splits < total_kblocks || (splits > 1 && out_dtype != IE_F32) ||
        ((uintptr_t)X & 15) != 0 || ((uintptr_t)W & 15) != 0)
        return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_F32)
        return M <= 8 ? launch<1, float>(X, W, (float*)out, M, N, K, kblocks_per_split, splits, err, s)
                      : launch<2, float>(X, W, (float*)out, M, N, K, kblocks_per_split, splits, err, s);
    return M <= 8 ? launch<1, bf16>(X, W, (bf16*)out, M, N, K, kblocks_per_split, splits, err, s)
                  : launch<2, bf16>(X, W, (bf16*)out, M, N, K, kblocks_per_split, splits, err, s);
}

// The gated feed-forward's first half in one kernel: W [N, K] holds gates and ups alternating in
// blocks of 16 rows (see the kernel), `out` [M, N / 2] receives silu(gate) * up in bfloat16.  The
// inner dimension is not cut: K at most 2048, a multiple of 8; N a multiple of 32; M <= 16.
IE_API int ie_gemm_tma_gated_bf16(const void* X, const void* W, void* out, int M, int N, int K, int* err,
                                  void* stream) {
    if (M <= 0 || N <= 0) return 0;
    int total_kblocks = (K + BK - 1) / BK;
    if (M > 16 || K % 8 != 0 || N % 32 != 0 || total_kblocks > MAX_KBLOCKS || ((uintptr_t)X & 15) != 0 ||
        ((uintptr_t)W & 15) != 0)
        return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    return M <= 8 ? launch<1, bf16, true>(X, W, (bf16*)out, M, N, K, total_kblocks, 1, err, s)
                  : launch<2, bf16, true>(X, W, (bf16*)out, M, N, K, total_kblocks, 1, err, s);
}
