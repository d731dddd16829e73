// Matrix product for a batch of decode tokens on the fifth-generation tensor cores:
//   C[M, N] = X[M, K] * W[N, K]^T,  bfloat16 in, 32-bit accumulation in tensor memory,
//   16 < M <= 256, K a multiple of 64.
//
// With a few dozen tokens the product is still a stream of weights through the SMs, so the
// roles of the operands are swapped: the 128 output features of a block are the M = 128 rows of
// tcgen05.mma (TMEM lanes), the step's tokens its N columns.  One block = 128 features x a
// slice of k (the inner dimension is cut into splits so that every SM has a block; partial
// sums go to out[split][M][N] and the consumer of the product adds them in order).
//   * warp 0, one thread: TMA copies of W (3-D tensor map: 128 features x kpo k blocks in one
//     copy) and of X (all tokens x the same k blocks) into a ring of shared memory.  The
//     weights need nobody's results, so under programmatic dependent launch the ring's first
//     round of W is asked for before the wait for the previous kernel; X comes after it.
//   * warp 1, one thread: tcgen05.mma (both operands K-major from shared memory, 128-byte
//     swizzle) over the block's slice of k, accumulating in TMEM; tcgen05.commit hands every
//     ring slot back and, at the end, tells the epilogue that the accumulator is complete.
//   * warps 2-5: read the accumulator (tcgen05.ld, thread = feature, columns = tokens) and
//     store it; for a fixed token the 32 lanes of a warp write 32 neighbouring features.
// Every wait is bounded; a block that waits too long records IE_ERR_TIMEOUT, frees its tensor
// memory and leaves.  The reference uses cuBLAS here (nn.Linear, engine/model/layers.py:126-129).
#include "tma.cuh"

using namespace ie_tma;

namespace {
constexpr int BN = 128;                    // features per block = rows of the instruction
constexpr int BK = 64;                     // k per tile: 128 bytes per row, one swizzle atom
constexpr int W_TILE_BYTES = BN * BK * 2;  // 16 KB
constexpr int THREADS = 6 * 32;
constexpr int MAX_OPS = 8;                 // ring slots
constexpr int RING_BYTES = 192 * 1024;

struct Tc5Plan {
    int M, N, K;
    int m_pad;              // tokens rounded up to 16: the instruction's N
    int kblocks_per_split;
    int kpo;                // k blocks per copy
    int ops;                // ring slots
    int tmem_cols;          // power of two >= max(32, m_pad)
};

#ifdef IE_TEST_STARVE
// Self-test build only (kernels/build.py: build_selftest).  While this flag is set, every block
// leaves out the last copy of X although it has told the slot's mbarrier to expect its bytes:
// the tensor-core thread's wait for that slot must run out, the block must record
// IE_ERR_TIMEOUT, give its tensor memory back and return.  Nothing is in flight when it does:
// every copy that was asked for is tracked by a barrier that completed long before the wait
// gives up.  The library that serves generation is built without this code.
static __device__ int g_starve_last_x;
#endif

struct __align__(8) Tc5Shared {
    unsigned long long full[MAX_OPS], empty[MAX_OPS], acc_done;
    unsigned tmem_base;
    int failed;
};

template <typename OutT>
__global__ void __launch_bounds__(THREADS)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                OutT* __restrict__ out, Tc5Plan p, int* err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* ring = smem;
    Tc5Shared* sh = reinterpret_cast<Tc5Shared*>(ring + RING_BYTES);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * BN, split = blockIdx.y;
    int total_kblocks = p.K / BK;
    int kb0 = split * p.kblocks_per_split;
    int nkb = min(p.kblocks_per_split, total_kblocks - kb0);
    if (nkb < 0) nkb = 0;
    int nops = (nkb + p.kpo - 1) / p.kpo;
    int x_tile_bytes = p.m_pad * BK * 2;
    int op_bytes = p.kpo * (W_TILE_BYTES + x_tile_bytes);   // W tiles first, then X tiles

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.ops; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->empty[s], 1);
        }
        mbar_init(&sh->acc_done, 1);
        sh->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {  // one warp allocates the block's tensor-memory columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ie_pdl_trigger();
    unsigned tmem = sh->tmem_base;

    if (warp == 0) {
        // ---- copies ----
        if (lane == 0) {
            auto copy_w = [&](int o) {
                int s = o % p.ops;
                mbar_expect_tx(&sh->full[s], op_bytes);
                tma_load_3d(ring + (size_t)s * op_bytes, &w_map, 0, n0, kb0 + o * p.kpo, &sh->full[s]);
            };
            auto copy_x = [&](int o) {
#ifdef IE_TEST_STARVE
                if (g_starve_last_x && o == nops - 1) return;
#endif
                int s = o % p.ops;
                tma_load_3d(ring + (size_t)s * op_bytes + p.kpo * W_TILE_BYTES, &x_map, 0, 0, kb0 + o * p.kpo,
                            &sh->full[s]);
            };
            int first = min(nops, p.ops);
            for (int o = 0; o < first; ++o) copy_w(o);   // the weights need nobody's results
            ie_pdl_wait();                               // X is the previous kernel's output
            for (int o = 0; o < first; ++o) copy_x(o);
            for (int o = first; o < nops; ++o) {
                if (!mbar_wait(&sh->empty[o % p.ops], ((o / p.ops) - 1) & 1)) { sh->failed = 1; break; }
                copy_w(o);
                copy_x(o);
            }
        } else {
            ie_pdl_wait();
        }
    } else if (warp == 1) {
        // ---- tensor core ----
        if (lane == 0) {
            unsigned idesc = umma_idesc_bf16(BN, p.m_pad);
            bool ok = true;
            for (int o = 0; o < nops && ok; ++o) {
                int s = o % p.ops;
                if (!mbar_wait(&sh->full[s], (o / p.ops) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned wbase = smem_u32(ring + (size_t)s * op_bytes);
                unsigned xbase = wbase + p.kpo * W_TILE_BYTES;
                int kbs = min(p.kpo, nkb - o * p.kpo);  // the last copy may reach beyond k: zeros
                for (int j = 0; j < kbs; ++j) {
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)  // 32 bytes further along k per step
                        umma_ss(tmem, umma_desc_sw128(wbase + j * W_TILE_BYTES + ks * 32),
                                umma_desc_sw128(xbase + j * x_tile_bytes + ks * 32), idesc,
                                (o > 0 || j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(&sh->empty[s]);  // the slot is free once these products have read it
            }
            umma_commit(&sh->acc_done);
            if (!ok) sh->failed = 1;
        }
        ie_pdl_wait();
    } else {
        // ---- epilogue: thread = feature = TMEM lane ----
        ie_pdl_wait();
        int lane_group = warp & 3;  // a warp may read the 32 lanes 32 (warp % 4) ..
        int f = n0 + lane_group * 32 + lane;
        bool ok = mbar_wait(&sh->acc_done, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && nkb > 0) {
            OutT* dst = out + (size_t)split * p.M * p.N;
            unsigned taddr = tmem + ((unsigned)(lane_group * 32) << 16);
            for (int c0 = 0; c0 < p.m_pad; c0 += 16) {
                float v[16];
                tmem_ld16(v, taddr + c0);
                if (f < p.N) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c0 + i < p.M) ie_store(dst + (size_t)(c0 + i) * p.N + f, v[i]);
                }
            }
        } else if (ok) {  // an empty slice of k (cannot happen with the host's plans): zeros
            OutT* dst = out + (size_t)split * p.M * p.N;
            if (f < p.N)
                for (int m = 0; m < p.M; ++m) ie_store(dst + (size_t)m * p.N + f, 0.f);
        }
        if (!ok) sh->failed = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(p.tmem_cols) : "memory");
    if (threadIdx.x == 0 && sh->failed) ie_report(err, IE_ERR_TIMEOUT, blockIdx.x, blockIdx.y);
}

constexpr size_t SMEM_BYTES = (size_t)RING_BYTES + sizeof(Tc5Shared) + 1024;

template <typename OutT>
int launch(const void* X, const void* W, OutT* out, const Tc5Plan& p, int splits, int* err, cudaStream_t s) {
    CUtensorMap wm, xm;
    if (!make_map_bf16_3d(&wm, W, p.N, p.K, BN, p.kpo) || !make_map_bf16_3d(&xm, X, p.M, p.K, p.m_pad, p.kpo))
        return (int)cudaErrorNotSupported;
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, gemm_tc5_kernel<OutT>, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((p.N + BN - 1) / BN, splits);
    return ie_launch(gemm_tc5_kernel<OutT>, grid, dim3(THREADS), SMEM_BYTES, s, wm, xm, out, p, err);
}
}  // namespace

#ifdef IE_TEST_STARVE
IE_API int ie_test_starve_tc5(int on) {
    return (int)cudaMemcpyToSymbol(g_starve_last_x, &on, sizeof(int));
}
#endif

// 1 if the product of these sizes can run here: 16 < M <= 256, K a multiple of 64.
IE_API int ie_gemm_tc5_ok(int M, int N, int K) {
    return encode_fn() != nullptr && M > 16 && M <= 256 && N > 0 && K > 0 && K % BK == 0 ? 1 : 0;
}

// `out`: [splits, M, N]; with splits > 1 32-bit partial sums over slices of `kblocks_per_split`
// blocks of 64 k; with splits == 1 the product, 32-bit or bfloat16.  X and W must be 16-byte
// aligned.
IE_API int ie_gemm_tc5_bf16(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K,
                            int kblocks_per_split, int splits, int* err, void* stream) {
    if (!ie_gemm_tc5_ok(M, N, K)) return (int)cudaErrorInvalidValue;
    int total_kblocks = K / BK;
    if (splits < 1 || kblocks_per_split < 1 || (long long)kblocks_per_split * splits < total_kblocks ||
        (long long)kblocks_per_split * (splits - 1) >= total_kblocks || (splits > 1 && out_dtype != IE_F32) ||
        ((uintptr_t)X & 15) != 0 || ((uintptr_t)W & 15) != 0)
        return (int)cudaErrorInvalidValue;
    Tc5Plan p;
    p.M = M; p.N = N; p.K = K;
    p.m_pad = (M + 15) / 16 * 16;
    p.kblocks_per_split = kblocks_per_split;
    // k blocks per copy: as many as divide the slice and leave at least three copies in the ring
    int tile_pair = W_TILE_BYTES + p.m_pad * BK * 2;
    p.kpo = 4;
    while (p.kpo > 1 && (kblocks_per_split % p.kpo != 0 || RING_BYTES / (p.kpo * tile_pair) < 3)) p.kpo >>= 1;
    p.ops = RING_BYTES / (p.kpo * tile_pair);
    if (p.ops > MAX_OPS) p.ops = MAX_OPS;
    if (p.ops < 2) return (int)cudaErrorInvalidValue;
    p.tmem_cols = 32;
    while (p.tmem_cols < p.m_pad) p.tmem_cols <<= 1;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_F32) return launch<float>(X, W, (float*)out, p, splits, err, s);
    return launch<__nv_bfloat16>(X, W, (__nv_bfloat16*)out, p, splits, err, s);
}
