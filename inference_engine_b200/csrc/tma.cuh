// Device and host helpers for kernels fed by the tensor memory accelerator: mbarriers with
// bounded waits, tiled copies with the 128-byte swizzle, tcgen05 (fifth-generation tensor
// core) descriptors, issue, commit and tensor-memory access, and the tensor-map encoder (taken
// from the driver at run time, no link against libcuda).
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace ie_tma {
typedef __nv_bfloat16 bf16;
// Polls of an mbarrier before a wait gives up.  A poll that fails comes back after about two
// microseconds (the hardware suspends the thread meanwhile), so this is some tenths of a second:
// far longer than any kernel a waiting block may sit behind, short enough to notice.
// (IE_SPIN_LIMIT: the self-test build sets a few dozen polls, so that a wait which is made to
// run out on purpose does so in a fraction of a millisecond.)
#ifndef IE_SPIN_LIMIT
#define IE_SPIN_LIMIT 200000
#endif
constexpr int SPIN_LIMIT = IE_SPIN_LIMIT;

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
// Bounded wait: false when the phase did not complete within SPIN_LIMIT polls.  The compiler
// unrolls this loop, which suits the matrix products (few waits, each on the critical path of a
// short kernel: 0.823 against 0.857 ms per decode step).
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, int parity) {
    unsigned addr = smem_u32(bar);
    for (int spin = 0; spin < SPIN_LIMIT; ++spin) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// The same wait as a loop that is not unrolled, for kernels with many waits in long loops (the
// prefill attention: 42 against 50 us on a 2,048-token prompt).
__device__ __forceinline__ bool mbar_wait_compact(unsigned long long* bar, int parity) {
    unsigned addr = smem_u32(bar);
#pragma unroll 1
    for (int spin = 0; spin < SPIN_LIMIT; ++spin) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// One box of a 2-D tensor map into shared memory; x is the inner (contiguous) coordinate and
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// ---- tcgen05 ----
// Shared-memory matrix descriptor of a K-major bfloat16 tile whose rows are 128 bytes (64 k)
// with the 128-byte swizzle: 8-row groups 1024 bytes apart.  `addr` may point 32 bytes further
// for every 16 k inside the tile.
__device__ __forceinline__ unsigned long long umma_desc_sw128(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr >> 4) & 0x3FFF);   // start address, 16-byte units
    d |= (unsigned long long)64 << 16;                 // leading byte offset (unused with this swizzle)
    d |= (unsigned long long)64 << 32;                 // stride byte offset: 1024 B between 8-row groups
    d |= (unsigned long long)1 << 46;                  // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                  // layout: 128-byte swizzle
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, D is m x n.
__device__ __forceinline__ unsigned umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
// D (tensor memory) = or += A B^T with A and B in shared memory; issued by one thread.
__device__ __forceinline__ void umma_ss(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                        unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier gets one arrival when all tcgen05 operations this thread issued so far are done.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 16 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld16(float (&v)[16], unsigned taddr) {
    unsigned* r = reinterpret_cast<unsigned*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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
// A barrier among `count` threads of the block (count a multiple of 32), id 1..15.
__device__ __forceinline__ void named_barrier(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
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

// A row-major [rows, cols] bfloat16 matrix (cols a multiple of 64) as a 3-D tensor (64 k, rows,
// cols / 64 k blocks) with boxes of 64 x box_rows x box_kbs: in shared memory box_kbs consecutive
// K-major tiles of box_rows x 64 with the 128-byte swizzle.  One large copy instead of several
// small ones: the copy engine spends a fixed time on every copy.
inline bool make_map_bf16_3d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows,
                             int box_kbs) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr || cols % 64 != 0 || box_rows < 1 || box_rows > 256 || box_kbs < 1 || box_kbs > 256) return false;
    cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128u};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)box_kbs};
    cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A row-major [rows, cols] bfloat16 matrix as a 2-D tensor map with boxes of box_rows x 64
// columns (128 bytes, one swizzle atom wide) and the 128-byte swizzle; out-of-range elements
// read as zero.  `base` must be 16-byte aligned and cols a multiple of 8.
inline bool make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr || box_rows < 1 || box_rows > 256) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace ie_tma
