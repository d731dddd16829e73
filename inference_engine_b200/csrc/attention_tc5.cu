// Paged prefill attention on the fifth-generation tensor cores (tcgen05 + TMEM + TMA), bfloat16,
// head sizes 64 and 128, pages of 8 to 64 tokens.  One build per head size (-DIE_HD=64 or 128);
// for other head sizes the file compiles to a stub that reports "not available".  With head
// size 128 a row of K or V is two 128-byte halves (two TMA boxes, two products of 64 output
// dims) and a block takes 320 columns of tensor memory, so one block runs per SM instead of two.
//
// One block = 128 query tokens of one head (a tcgen05.mma of M = 128: TMEM lane = query row =
// thread of the softmax warps).  Six (or seven) warps in three roles, decoupled by mbarriers:
//   * warp 4, one thread: copies the pages of every 64-key tile of K and V with TMA
//     (cp.async.bulk.tensor, one box per page, 128-byte swizzle) into a three-stage ring;
//   * warp 5, one thread: issues S(t) = Q K(t)^T (four tcgen05.mma of k = 16, A = Q from tensor
//     memory, B = K from shared memory) into one of two 64-column TMEM buffers, one tile ahead
//     of the softmax, and O += P(t) V(t) (A = P from tensor memory, V as an MN-major B operand)
//     as soon as the weights of tile t are written; tcgen05.commit signals the softmax warps
//     and frees the ring stage (head size 128: a seventh warp issues the second product, so
//     that the two products' instructions go out side by side);
//   * warps 0-3: every thread puts its row of Q into tensor memory once, then for every tile
//     reads its row of S (tcgen05.ld 32x32b), masks (diagonal and window tiles only), keeps the
//     running maximum and sum -- a row is private to a thread, no shuffles -- rounds the weights
//     to bfloat16 and writes them, two to a column, over the row of S (tcgen05.st).
// The output accumulator stays in tensor memory for the whole key range.  The maximum that the
// weights are taken against follows the running maximum only when that has grown by more than
// 2^8; only then is the accumulator read, rescaled and written back.
// While the softmax of tile t runs, the tensor core computes S(t+1) and P(t-1) V(t-1), and the
// copies of tile t+2 are in flight; shared memory carries K and V only.  All waits on mbarriers
// are bounded; a block that waits too long records IE_ERR_TIMEOUT, frees its TMEM and leaves.
// The reference's counterpart is the FlashAttention varlen call over gathered keys and values
// (engine/model/layers.py:246-253).
#include "tma.cuh"
#include <math.h>

#ifndef IE_HD
#error "compile with -DIE_HD=<head size>"
#endif

#if IE_HD == 64 || IE_HD == 128

using namespace ie_tma;

namespace {
constexpr int HD = IE_HD;
constexpr int HALVES = HD / 64;           // 64-wide column halves of a K or V row (128 bytes, one swizzle atom)
constexpr int BM = 128;             // query rows per block
constexpr int KT = 64;              // keys per tile
constexpr int SOFTMAX_THREADS = 128;
// Head size 128: a thread gets a tcgen05.mma out about every 117 clocks whatever its size, and a
// tile's sixteen products would keep one thread busy longer than the softmax takes, so each of the
// two products has an issuing warp of its own.
constexpr bool SPLIT_ISSUE = HD == 128;
constexpr int THREADS = SPLIT_ISSUE ? 224 : 192;  // + the copy warp and the tensor-core warp(s)
constexpr int KV_STAGES = HD == 64 ? 3 : 4;   // head size 128: 132 KB of shared memory, one block per SM as its tensor memory asks
constexpr int KV_BYTES = KT * HD * 2;       // K (and as much V) of a stage: HALVES tiles of 64 keys x 64 dims, 8 KB each
constexpr int HALF_BYTES = KT * 128;
// block-table entries a block keeps in shared memory (a late query tile needs the request's whole table: 131,072
// tokens in pages of 16; 32 KB of the 80 KB a block of head size 64 takes, two blocks to an SM)
constexpr int MAX_TABLE = 8192;
// tensor memory: S (then P, packed) in columns 0..63 and 64..127, O in the next HD, Q (two dims to a
// column) in the next HD / 2: 224 columns for head size 64 (two blocks per SM), 320 for 128 (one)
constexpr int TMEM_COLS = HD == 64 ? 256 : 512;
constexpr int BLOCKS_PER_SM = HD == 64 ? 2 : 1;
constexpr float RESCALE_LAG = 8.0f;         // in powers of two

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Two 32-bit multiply-adds, or adds, in one instruction (the packed forms this architecture has):
// the softmax warps are bound by the instructions they issue, not by a pipe.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float, M = 128, N = 64; b_mn: B is MN-major.
__device__ __forceinline__ unsigned instr_desc(bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
}
// D (TMEM) = or += A B; A in tensor memory: lane = row, a 32-bit column = two consecutive k.
__device__ __forceinline__ void umma_ta(unsigned tmem_d, unsigned tmem_a, unsigned long long b, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// One row (this thread's TMEM lane) of 64 columns starting at `taddr`.
__device__ __forceinline__ void tmem_ld64(float (&v)[64], unsigned taddr) {
    unsigned* r = reinterpret_cast<unsigned*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
        "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32(float (&v)[32], unsigned taddr) {
    unsigned* r = reinterpret_cast<unsigned*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32(const float (&v)[32], unsigned taddr) {
    const unsigned* r = reinterpret_cast<const unsigned*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

#ifdef IE_TC5_TIMING
__device__ long long g_tc5_clocks[16];
#define TC5_T(i) do { if (timing) { long long now_ = clock64(); g_tc5_clocks[i] += now_ - mark_; mark_ = now_; } } while (0)
#else
#define TC5_T(i) do { } while (0)
#endif

struct __align__(8) Barriers {
    unsigned long long q_full, kv_full[KV_STAGES], kv_empty[KV_STAGES], s_done[2], p_ready[2], o_done;
    unsigned tmem_base;
    int failed;
    int is_last;
};

// The last block of a tile and head merges the shares of the tile's keys that `ksplit` blocks
// left in scratch, in their order: one thread per query row.  Kept out of line: inlined, its
// registers slowed the kernel's main path down.
template <int C>
__device__ __forceinline__ void merge_rows(const float* __restrict__ part_o, size_t first, int ksplit,
                                           bf16* __restrict__ out0, size_t row_stride, int rows,
                                           const float* __restrict__ factor_s, int tid) {
    constexpr int TPR = HD / 4;               // threads per row
    constexpr int ROWS_AT_ONCE = SOFTMAX_THREADS / TPR;
    constexpr int U = 16 / C;                 // row groups at a time
    int d4 = tid % TPR, r0 = tid / TPR;
#pragma unroll 1
    for (int rb = 0; rb < BM; rb += U * ROWS_AT_ONCE) {
        float4 acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z0 = 0; z0 < ksplit; z0 += C) {
            float4 v[U][C];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int j = 0; j < C; ++j) {
                    int row = rb + u * ROWS_AT_ONCE + r0;
                    bool in = z0 + j < ksplit;
                    size_t p = first + (size_t)(in ? z0 + j : 0) * BM + row;
                    v[u][j] = in ? __ldcg(reinterpret_cast<const float4*>(part_o + p * HD) + d4) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int j = 0; j < C; ++j)    // (in the shares' order)
                    if (z0 + j < ksplit) {
                        float f = factor_s[(z0 + j) * BM + rb + u * ROWS_AT_ONCE + r0];
                        acc[u].x += v[u][j].x * f; acc[u].y += v[u][j].y * f;
                        acc[u].z += v[u][j].z * f; acc[u].w += v[u][j].w * f;
                    }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            int row = rb + u * ROWS_AT_ONCE + r0;
            if (row < rows) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(acc[u].x, acc[u].y), hi = __floats2bfloat162_rn(acc[u].z, acc[u].w);
                *reinterpret_cast<uint2*>(out0 + (size_t)row * row_stride + d4 * 4) =
                    make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
            }
        }
    }
}

__device__ __noinline__ void merge_key_shares(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              size_t first, int ksplit, bf16* __restrict__ out0, size_t row_stride,
                                              int rows, float* __restrict__ factor_s, int tid) {
    // Called by the 128 softmax threads of the block that ends last.  `first`: the pair's first row in
    // scratch (share z's row r at first + z * BM + r); `out0`: the tile's first output row of this head.
    // 1. A thread per row: the shares' maxima and sums (eight shares' loads in flight at a time) give
    //    every share's factor exp2(m_z - m) / l for the row, left in shared memory.
    __threadfence();
    {
        size_t at = first + tid;
        float m_all = -INFINITY;
        for (int z0 = 0; z0 < ksplit; z0 += 8) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                t[j] = z0 + j < ksplit ? __ldcg(part_ml + (at + (size_t)(z0 + j) * BM) * 2) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) m_all = fmaxf(m_all, t[j]);
        }
        float m_safe = (m_all == -INFINITY) ? 0.f : m_all;
        float l_all = 0.f;
        for (int z0 = 0; z0 < ksplit; z0 += 8) {
            float tm[8], tl[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                size_t p = at + (size_t)(z0 + j < ksplit ? z0 + j : 0) * BM;
                tm[j] = z0 + j < ksplit ? __ldcg(part_ml + p * 2) : -INFINITY;
                tl[j] = z0 + j < ksplit ? __ldcg(part_ml + p * 2 + 1) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (z0 + j < ksplit) {   // (in the shares' order)
                    float f = exp2f(tm[j] - m_safe);
                    l_all += tl[j] * f;
                    factor_s[(z0 + j) * BM + tid] = f;
                }
        }
        float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
        for (int z = 0; z < ksplit; ++z) factor_s[z * BM + tid] *= inv;
    }
    named_barrier(2, SOFTMAX_THREADS);
    // 2. The rows' sums: a thread takes four dims of the rows tid / (HD / 4) + k * 128 / (HD / 4), so that
    //    a warp reads whole rows; sixteen loads in flight: C shares of 16 / C rows at a time.
    if (ksplit <= 2) merge_rows<2>(part_o, first, ksplit, out0, row_stride, rows, factor_s, tid);
    else if (ksplit <= 4) merge_rows<4>(part_o, first, ksplit, out0, row_stride, rows, factor_s, tid);
    else merge_rows<8>(part_o, first, ksplit, out0, row_stride, rows, factor_s, tid);
}

// SPLIT: the keys of a tile are shared among gridDim.z blocks (an instance of its own: the code
// for it cost the plain kernel 4 % on long prompts).
template <bool SPLIT>
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM)
attention_prefill_tc5_kernel(const bf16* __restrict__ q, const __grid_constant__ CUtensorMap k_map,
                             const __grid_constant__ CUtensorMap v_map, const int* __restrict__ tables,
                             int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                             bf16* __restrict__ out, int num_seqs, int nh, int nkv, int page_shift,
                             int total_pages, float scale_log2, int window, int paired, int ksplit,
                             float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ tickets,
                             int* err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* k_s = smem;                                  // stages x 8 KB
    unsigned char* v_s = k_s + KV_STAGES * KV_BYTES;
    int* table_s = reinterpret_cast<int*>(v_s + KV_STAGES * KV_BYTES);  // MAX_TABLE ints
    Barriers* bars = reinterpret_cast<Barriers*>(table_s + MAX_TABLE);
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int head = blockIdx.y, G = nh / nkv, kvh = head / G;
    ie_pdl_trigger();
    // (lengths and block tables are the step's inputs; queries, keys and values are the previous
    // kernel's output: the roles wait for it below, after the set-up)
    // Which request and which of its 128-token tiles are this block's?  Tile i of a request of n
    // tiles needs about i + 1 key tiles.  With few blocks (`paired`) a block takes the pair
    // (n - 1 - p, p), one after the other, so that every block of a request has the same amount
    // of work and all run at once; with many blocks each takes one tile, the heavy ones first.
    int item = paired ? blockIdx.x : gridDim.x - 1 - blockIdx.x;
    int seq = -1, q0 = 0, qlen = 0, tile_a = 0, tile_b = 0;
    for (int s = 0; s < num_seqs; ++s) {
        int a = cu_q[s], n = cu_q[s + 1] - a;
        int tiles = (n * G > 16) ? (n + BM - 1) / BM : 0;
        int items = paired ? (tiles + 1) / 2 : tiles;
        if (item < items) {
            seq = s; q0 = a; qlen = n;
            tile_a = paired ? tiles - 1 - item : item;
            tile_b = item;  // unpaired: the same tile, one part
            break;
        }
        item -= items;
    }
    if (seq < 0) return;
    int ctx = ctx_lens[seq];
    const int* table = tables + (size_t)seq * table_width;
    int first_qpos = ctx - qlen;
    struct Part { int t0, rows, qpos_lo, qpos_hi, key_begin, n_tiles; };
    auto make_part = [&](int tile) {
        Part p;
        p.t0 = tile * BM;
        p.rows = min(BM, qlen - p.t0);
        p.qpos_lo = first_qpos + p.t0;
        p.qpos_hi = p.qpos_lo + p.rows - 1;
        int lo = (window > 0 && p.qpos_lo - window + 1 > 0) ? p.qpos_lo - window + 1 : 0;
        p.key_begin = (lo / KT) * KT;
        p.n_tiles = (p.qpos_hi - p.key_begin) / KT + 1;
        if (SPLIT) {  // this block's share of the tile's keys (it may be empty)
            int first = (int)((long long)blockIdx.z * p.n_tiles / ksplit);
            int end = (int)((long long)(blockIdx.z + 1) * p.n_tiles / ksplit);
            p.key_begin += first * KT;
            p.n_tiles = end - first;
        }
        return p;
    };
    Part parts[2];
    int nparts = tile_b < tile_a ? 2 : 1;
    parts[0] = make_part(tile_a);
    parts[1] = make_part(nparts == 2 ? tile_b : tile_a);
    int page_size = 1 << page_shift;
    int pages_per_tile = KT >> page_shift;
    // block-table entries of both parts' key ranges, once
    int first_entry = min(parts[0].key_begin, parts[1].key_begin) >> page_shift;
    int last_entry = max(parts[0].key_begin + parts[0].n_tiles * KT, parts[1].key_begin + parts[1].n_tiles * KT) - 1;
    last_entry >>= page_shift;
    int n_entries = min(last_entry - first_entry + 1, MAX_TABLE);

    if (tid == 0) {
        mbar_init(&bars->q_full, SOFTMAX_THREADS);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&bars->kv_full[s], 1); mbar_init(&bars->kv_empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&bars->s_done[b], 1); mbar_init(&bars->p_ready[b], SOFTMAX_THREADS); }
        mbar_init(&bars->o_done, 1);
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < n_entries; i += THREADS) {
        int e = first_entry + i;
        int page = e < table_width ? table[e] : -1;
        // a page that is not there lies beyond the context: its keys are masked, any page's
        // (finite) contents will do
        table_s[i] = (page >= 0 && page < total_pages) ? page : 0;
    }
    if (warp == 0) {  // one warp allocates the block's TMEM columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    unsigned tmem = bars->tmem_base;
    unsigned tmem_o = tmem + 2 * KT, tmem_q = tmem + 2 * KT + HD;
    // In all three roles g counts the key tiles over both parts: ring stage g % 3, S buffer
    // g & 1 and the barriers' phases go on from the first part into the second.

    if (warp == 4) {
        // ---- copies: one thread ----
        ie_pdl_wait();
        if (lane == 0) {
            int g = 0;
            bool ok = true;
            for (int pi = 0; pi < nparts && ok; ++pi) {
                const Part& pt = parts[pi];
                for (int t = 0; t < pt.n_tiles; ++t, ++g) {
                    int stage = g % KV_STAGES;
                    if (g >= KV_STAGES && !mbar_wait_compact(&bars->kv_empty[stage], (g / KV_STAGES - 1) & 1)) { ok = false; break; }
                    mbar_expect_tx(&bars->kv_full[stage], 2 * KV_BYTES);
                    int entry = ((pt.key_begin + t * KT) >> page_shift) - first_entry;
                    for (int p = 0; p < pages_per_tile; ++p) {
                        int page = table_s[min(entry + p, MAX_TABLE - 1)];
                        int row = (page * nkv + kvh) << page_shift;
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) {  // 64 dims to a box
                            int at = stage * KV_BYTES + h * HALF_BYTES + p * page_size * 128;
                            tma_load_2d(k_s + at, &k_map, h * 64, row, &bars->kv_full[stage]);
                            tma_load_2d(v_s + at, &v_map, h * 64, row, &bars->kv_full[stage]);
                        }
                    }
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (!SPLIT_ISSUE && warp == 5) {
        // ---- tensor core: one thread issues both products (head size 64: the exponentials bound
        // the kernel, a second issuing warp only takes issue slots from the softmax warps) ----
        if (lane == 0) {
            unsigned idesc_qk = instr_desc(false), idesc_pv = instr_desc(true);
            bool ok = true;
            auto issue_s = [&](int g) {  // S = Q K^T of key tile g into S buffer g & 1
                int stage = g % KV_STAGES;
                if (!mbar_wait_compact(&bars->kv_full[stage], (g / KV_STAGES) & 1)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned ka = smem_u32(k_s + stage * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)  // 32 bytes further along k per step, 4 steps to a half
                    umma_ta(tmem + (g & 1) * KT, tmem_q + ks * 8, umma_desc_sw128(ka + (ks >> 2) * HALF_BYTES + (ks & 3) * 32),
                            idesc_qk, ks > 0);
                umma_commit(&bars->s_done[g & 1]);
                return true;
            };
            int g = 0;
            for (int pi = 0; pi < nparts && ok; ++pi) {
                int n_tiles = parts[pi].n_tiles;
                // the part's Q is in tensor memory (and the softmax warps are done with the
                // accumulator of the part before)
                ok = mbar_wait_compact(&bars->q_full, pi & 1) && (n_tiles == 0 || issue_s(g));
                for (int t = 0; t < n_tiles && ok; ++t, ++g) {
                    if (t + 1 < n_tiles) {
                        // its S buffer held the weights of tile g - 1: that product must have read them
                        if (g > 0 && !mbar_wait_compact(&bars->o_done, (g - 1) & 1)) { ok = false; break; }
                        ok = issue_s(g + 1);
                    }
                    if (!ok || !mbar_wait_compact(&bars->p_ready[g & 1], (g >> 1) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    int stage = g % KV_STAGES;
                    unsigned va = smem_u32(v_s + stage * KV_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)  // 64 output dims per product
#pragma unroll
                        for (int ks = 0; ks < KT / 16; ++ks)  // P: 8 columns of two keys each; V: 16 keys = 2048 bytes
                            umma_ta(tmem_o + h * 64, tmem + (g & 1) * KT + ks * 8,
                                    umma_desc_sw128(va + h * HALF_BYTES + ks * 2048), idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&bars->o_done);
                    umma_commit(&bars->kv_empty[stage]);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (SPLIT_ISSUE && warp == 5) {
        // ---- tensor core, first product: one thread issues S = Q K^T of every key tile ----
        // (a thread gets a tcgen05.mma out about every 117 clocks whatever its size, so the two
        // products of a tile are issued by a thread each)
        if (lane == 0) {
            unsigned idesc_qk = instr_desc(false);
            bool ok = true;
            int g = 0;
            for (int pi = 0; pi < nparts && ok; ++pi) {
                // the part's Q is in tensor memory
                ok = mbar_wait_compact(&bars->q_full, pi & 1);
                for (int t = 0; t < parts[pi].n_tiles && ok; ++t, ++g) {
                    // S buffer g & 1 held the weights of tile g - 2: that product must have read
                    // them.  (Waited for right after S(g - 1) went out, so the barrier cannot be
                    // more than one phase ahead.  For a part's first two tiles the wait for Q
                    // covers it: the softmax warps had waited for all products of the part before,
                    // and by now this barrier may be any number of phases ahead.)
                    if (t >= 2 && !mbar_wait_compact(&bars->o_done, (g - 2) & 1)) { ok = false; break; }
                    int stage = g % KV_STAGES;
                    if (!mbar_wait_compact(&bars->kv_full[stage], (g / KV_STAGES) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned ka = smem_u32(k_s + stage * KV_BYTES);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks)  // 32 bytes further along k per step, 4 steps to a half
                        umma_ta(tmem + (g & 1) * KT, tmem_q + ks * 8,
                                umma_desc_sw128(ka + (ks >> 2) * HALF_BYTES + (ks & 3) * 32), idesc_qk, ks > 0);
                    umma_commit(&bars->s_done[g & 1]);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else if (SPLIT_ISSUE && warp == 6) {
        // ---- tensor core, second product: one thread issues O += P V of every key tile ----
        if (lane == 0) {
            unsigned idesc_pv = instr_desc(true);
            bool ok = true;
            int g = 0;
            for (int pi = 0; pi < nparts && ok; ++pi) {
                for (int t = 0; t < parts[pi].n_tiles; ++t, ++g) {
                    int stage = g % KV_STAGES;
                    // (the softmax warps are done with the accumulator of the part before: they
                    // read it before they wrote this part's Q and its first weights)
                    if (!mbar_wait_compact(&bars->kv_full[stage], (g / KV_STAGES) & 1) ||
                        !mbar_wait_compact(&bars->p_ready[g & 1], (g >> 1) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned va = smem_u32(v_s + stage * KV_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)  // 64 output dims per product
#pragma unroll
                        for (int ks = 0; ks < KT / 16; ++ks)  // P: 8 columns of two keys each; V: 16 keys = 2048 bytes
                            umma_ta(tmem_o + h * 64, tmem + (g & 1) * KT + ks * 8,
                                    umma_desc_sw128(va + h * HALF_BYTES + ks * 2048), idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&bars->o_done);
                    umma_commit(&bars->kv_empty[stage]);
                }
            }
            if (!ok) bars->failed = 1;
        }
    } else {
        // ---- softmax: thread = query row = TMEM lane ----
        int row = tid;
        unsigned lane_addr = (unsigned)(warp * 32) << 16;  // this warp's 32 TMEM lanes
        bool ok = true;
        int g = 0;
        ie_pdl_wait();
#ifdef IE_TC5_TIMING
        bool timing = tid == 0 && blockIdx.x == gridDim.x / 2 && blockIdx.y == 0;
        long long mark_ = clock64();
#endif
        for (int pi = 0; pi < nparts && ok; ++pi) {
            const Part& pt = parts[pi];
            int n_tiles = pt.n_tiles, qpos_lo = pt.qpos_lo, qpos_hi = pt.qpos_hi;
            bool exists = row < pt.rows;
            int qpos = exists ? qpos_lo + row : -1;
            int qlo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
            // m: the maximum that the weights are taken against.  It follows the running maximum
            // only when that has grown by more than 2^RESCALE_LAG (for any row of the warp), so
            // that the accumulator in TMEM is rescaled on few tiles; weights stay below 2^RESCALE_LAG
            // and the quotient of accumulator and sum is the same.
            float m = -INFINITY, l = 0.f;
            {   // this row of Q, two features to a column, as the first product's A operand (the
                // products of the part before have all been waited for)
                const uint4* src = reinterpret_cast<const uint4*>(q + ((size_t)(q0 + pt.t0 + row) * nh + head) * HD);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) {
                    float qw[32];
                    uint4* q4 = reinterpret_cast<uint4*>(qw);
#pragma unroll
                    for (int c = 0; c < 8; ++c) q4[c] = exists ? src[h * 8 + c] : make_uint4(0u, 0u, 0u, 0u);
                    tmem_st32(qw, tmem_q + h * 32 + lane_addr);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(&bars->q_full);
            }
            for (int t = 0; t < n_tiles; ++t, ++g) {
                int key0 = pt.key_begin + t * KT;
                TC5_T(0);
                if (!mbar_wait_compact(&bars->s_done[g & 1], (g >> 1) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                TC5_T(1);
                float s[KT];
                tmem_ld64(s, tmem + (g & 1) * KT + lane_addr);
                TC5_T(2);
                // inner tiles (every key visible to every row of the block) need no mask
                bool inner = key0 + KT - 1 <= qpos_lo && (window <= 0 || key0 >= qpos_hi - window + 1);
                if (!inner) {
#pragma unroll
                    for (int j = 0; j < KT; ++j) {
                        int kpos = key0 + j;
                        s[j] = (kpos <= qpos && kpos >= qlo) ? s[j] : -INFINITY;
                    }
                }
                float mx[8];  // eight independent chains of three-way maxima
#pragma unroll
                for (int j = 0; j < 8; ++j) mx[j] = s[j];
#pragma unroll
                for (int j = 8; j + 16 <= KT; j += 16)
#pragma unroll
                    for (int i = 0; i < 8; ++i) mx[i] = max3(mx[i], s[j + i], s[j + 8 + i]);
#pragma unroll
                for (int j = 8 + (KT - 8) / 16 * 16; j < KT; ++j) mx[j & 7] = fmaxf(mx[j & 7], s[j]);
                float tile_max = fmaxf(max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), mx[6]), mx[7]);
                float m_cand = fmaxf(m, tile_max * scale_log2);
                bool rescale = __any_sync(0xffffffffu, m_cand > m + RESCALE_LAG);
                float alpha = 1.f;
                if (rescale) {
                    alpha = fast_exp2(m - ((m_cand == -INFINITY) ? 0.f : m_cand));
                    m = m_cand;
                    l *= alpha;
                }
                float m_safe = (m == -INFINITY) ? 0.f : m;
                TC5_T(3);
                // weights, rounded to bfloat16 and packed two to a column, over this row of S: the
                // second product's A operand
                float pw[32];
                unsigned* w = reinterpret_cast<unsigned*>(pw);
                float2 ls[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
                const float2 scale2 = make_float2(scale_log2, scale_log2), minus_m = make_float2(-m_safe, -m_safe);
#pragma unroll
                for (int c = 0; c < KT / 2; ++c) {
                    float2 x = fma2(make_float2(s[2 * c], s[2 * c + 1]), scale2, minus_m);
                    float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    ls[c & 3] = add2(ls[c & 3], p);
                    __nv_bfloat162 pk = __floats2bfloat162_rn(p.x, p.y);
                    w[c] = *reinterpret_cast<unsigned*>(&pk);
                }
                float2 lsum = add2(add2(ls[0], ls[1]), add2(ls[2], ls[3]));
                l += lsum.x + lsum.y;
                TC5_T(4);
                tmem_st32(pw, tmem + (g & 1) * KT + lane_addr);
                TC5_T(5);
                if (t > 0) {
                    // the previous tile's product has had this tile's softmax to finish; waiting for
                    // it here every tile also keeps this barrier's phase in step
                    if (!mbar_wait_compact(&bars->o_done, (g - 1) & 1)) { ok = false; break; }
                    if (rescale) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int half = 0; half < HD / 32; ++half) {
                            float acc[32];
                            tmem_ld32(acc, tmem_o + half * 32 + lane_addr);
#pragma unroll
                            for (int d = 0; d < 32; ++d) acc[d] *= alpha;
                            tmem_st32(acc, tmem_o + half * 32 + lane_addr);
                        }
                    }
                }
                TC5_T(6);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(&bars->p_ready[g & 1]);
                TC5_T(7);
#ifdef IE_TC5_TIMING
                if (timing) g_tc5_clocks[15] += 1;
#endif
            }
            if (ok && n_tiles > 0 && !mbar_wait_compact(&bars->o_done, (g - 1) & 1)) ok = false;
            bf16* orow = out + ((size_t)(q0 + pt.t0 + row) * nh + head) * HD;
            if (!SPLIT) {
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
                    for (int half = 0; half < HD / 32; ++half) {
                        float acc[32];
                        tmem_ld32(acc, tmem_o + half * 32 + lane_addr);
                        if (exists) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                unsigned w[4];
#pragma unroll
                                for (int h = 0; h < 4; ++h) {
                                    __nv_bfloat162 pk = __floats2bfloat162_rn(acc[c * 8 + 2 * h] * inv, acc[c * 8 + 2 * h + 1] * inv);
                                    w[h] = *reinterpret_cast<unsigned*>(&pk);
                                }
                                *reinterpret_cast<uint4*>(orow + half * 32 + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
            } else {
                // The tile's keys are shared among ksplit blocks: this one's row of the accumulator
                // (relative to its maximum m), m and the sum go to scratch; the block that finishes
                // last for this tile and head (ticket counter) merges the shares in their order.
                // All softmax threads pass the two barriers, whatever happened before.
                size_t pair = (size_t)blockIdx.x * nh + head;
                size_t at = (pair * ksplit + blockIdx.z) * BM + row;
                bool filled = ok && n_tiles > 0;  // (no keys for this share: an empty part)
                part_ml[at * 2] = filled ? m : -INFINITY;
                part_ml[at * 2 + 1] = filled ? l : 0.f;
                if (filled) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int half = 0; half < HD / 32; ++half) {
                    float acc[32];
                    if (filled) {
                        tmem_ld32(acc, tmem_o + half * 32 + lane_addr);
                    } else {
#pragma unroll
                        for (int d = 0; d < 32; ++d) acc[d] = 0.f;
                    }
                    float4* dst = reinterpret_cast<float4*>(part_o + at * HD + half * 32);
#pragma unroll
                    for (int c = 0; c < 8; ++c) dst[c] = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
                }
                __threadfence();
                named_barrier(2, SOFTMAX_THREADS);
                if (tid == 0) {
                    int ticket = atomicAdd(&tickets[pair], 1);
                    bars->is_last = ticket == ksplit - 1;
                    if (bars->is_last) tickets[pair] = 0;  // zero again for the next launch
                }
                named_barrier(2, SOFTMAX_THREADS);
                // (the ring of K and V tiles is free by now: the shares' factors go there)
                if (bars->is_last)
                    merge_key_shares(part_o, part_ml, pair * ksplit * BM, ksplit,
                                     out + ((size_t)(q0 + pt.t0) * nh + head) * HD, (size_t)nh * HD, pt.rows,
                                     reinterpret_cast<float*>(k_s), tid);
            }
        }
        if (!ok) bars->failed = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    if (tid == 0 && bars->failed) ie_report(err, IE_ERR_TIMEOUT, blockIdx.x, blockIdx.y);
}

constexpr size_t SMEM_BYTES = 2 * KV_STAGES * KV_BYTES + MAX_TABLE * 4 + sizeof(Barriers) + 1024;
}  // namespace

#ifdef IE_TC5_TIMING
IE_API int ie_tc5_timing(long long* out, int reset) {
    long long zero[16] = {0};
    cudaError_t e = cudaMemcpyFromSymbol(out, g_tc5_clocks, sizeof(zero));
    if (e == cudaSuccess && reset) e = cudaMemcpyToSymbol(g_tc5_clocks, zero, sizeof(zero));
    return (int)e;
}
#endif

// 1 if the tcgen05 prefill kernel can take this geometry: pages of 8..64 tokens, at most
// `MAX_TABLE` pages per 128-token tile's key range.
IE_API int ie_attention_prefill_tc5_ok(int page_size, int max_ctx) {
    if (encode_fn() == nullptr) return 0;
    if (page_size < 8 || page_size > KT || (page_size & (page_size - 1)) != 0) return 0;
    return ((max_ctx + KT - 1) / KT * KT + page_size - 1) / page_size <= MAX_TABLE ? 1 : 0;  // (whole key tiles)
}

// Floats of scratch for `ksplit` > 1: a partial result per (work item, head, share of the keys).
IE_API long long ie_attention_prefill_tc5_scratch_floats(int max_items, int nh, int ksplit) {
    if (ksplit <= 1) return 0;
    return (long long)max_items * nh * ksplit * BM * (HD + 2);
}

// `ksplit` > 1 (not with `paired`): the keys of every 128-token tile are shared among that many
// blocks, for steps with few tiles and long contexts; needs `scratch`
// (ie_attention_prefill_tc5_scratch_floats floats) and `tickets` (max_items * nh ints, zero before
// the first launch; a launch leaves them zero).
IE_API int ie_attention_prefill_tc5(const void* q, const void* k_cache, const void* v_cache, const int* tables,
                                    int table_width, const int* cu_q, const int* ctx_lens, void* out,
                                    int num_tokens, int num_seqs, int max_items, int paired, int nh, int nkv,
                                    int page_size, int total_pages, float scale, int window, int ksplit,
                                    float* scratch, int* tickets, int* err, void* stream) {
    if (num_seqs <= 0 || max_items <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || (page_size & (page_size - 1)) != 0 || page_size < 8 || page_size > KT ||
        ksplit < 1 || ksplit > 64 || (ksplit > 1 && (paired || scratch == nullptr || tickets == nullptr)))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    CUtensorMap km, vm;
    long long kv_rows = (long long)total_pages * nkv * page_size;
    if (!make_map_bf16(&km, k_cache, kv_rows, HD, page_size) ||
        !make_map_bf16(&vm, v_cache, kv_rows, HD, page_size))
        return (int)cudaErrorNotSupported;
    static IePerDevice configured_whole, configured_shared;
    cudaError_t e = ie_allow_smem(configured_whole, attention_prefill_tc5_kernel<false>, SMEM_BYTES);
    if (e == cudaSuccess) e = ie_allow_smem(configured_shared, attention_prefill_tc5_kernel<true>, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)max_items * nh * ksplit * BM * HD : nullptr;
    float scale_log2 = scale * 1.4426950408889634f;
    if (ksplit > 1)
        return ie_launch(attention_prefill_tc5_kernel<true>, dim3(max_items, nh, ksplit), dim3(THREADS), SMEM_BYTES,
                         (cudaStream_t)stream, (const bf16*)q, km, vm, tables, table_width, cu_q, ctx_lens, (bf16*)out,
                         num_seqs, nh, nkv, page_shift, total_pages, scale_log2, window, paired, ksplit, part_o, part_ml,
                         tickets, err);
    return ie_launch(attention_prefill_tc5_kernel<false>, dim3(max_items, nh), dim3(THREADS), SMEM_BYTES,
                     (cudaStream_t)stream, (const bf16*)q, km, vm, tables, table_width, cu_q, ctx_lens, (bf16*)out, num_seqs,
                     nh, nkv, page_shift, total_pages, scale_log2, window, paired, ksplit, part_o, part_ml, tickets, err);
}

#else  // other head sizes: the mma.sync kernels of attention_mma.cu serve them

IE_API int ie_attention_prefill_tc5_ok(int, int) { return 0; }
IE_API long long ie_attention_prefill_tc5_scratch_floats(int, int, int) { return 0; }
IE_API int ie_attention_prefill_tc5(const void*, const void*, const void*, const int*, int, const int*,
                                    const int*, void*, int, int, int, int, int, int, int, int, float, int, int,
                                    float*, int*, int*, void*) {
    return (int)cudaErrorNotSupported;
}

#endif
