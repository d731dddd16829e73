// Paged attention in bfloat16 on the tensor cores, one build per head size (-DIE_HD=64).
//
// Three kernels share the tile code below:
//   * decode: requests that bring few tokens (tokens x group size <= 16 rows: one decoded
//     token, or a portion of two or three) -- one block per (request, key/value head, split of
//     the context).  The group's query heads are rows of one 16-row matrix, so every key and
//     value is read once for the whole group; the context is split over blocks and over the
//     warps of a block (flash-decoding), and the block that finishes last merges the splits in
//     a fixed order;
//   * decode with the work dealt by length: the same for steps whose contexts differ much --
//     a fixed grid, every block works out from the lengths which key tiles are its own;
//   * prefill: longer portions -- one block per (128 query tokens, query head; 64 tokens above
//     head size 64), four warps of 32 or 16 rows each, walking the keys from the start of the window to the
//     last query position (bottom-right causal mask for portions that start mid-sequence).  Head
//     sizes 64 and 128 with pages of 8 tokens or more go to the tcgen05 kernel of
//     attention_tc5.cu instead.
// Keys and values come through the block table row by row (a row is a head's head_dim values
// of one token, contiguous), are staged in shared memory with cp.async (rings of three tiles,
// zero-filled outside the valid range) and read with ldmatrix; products are
// mma.sync.m16n8k16 with 32-bit accumulators.  Scores, the running maximum and sum are
// 32-bit; the weights are rounded to bfloat16 before they multiply the values, as in the
// reference's bfloat16 kernel (engine/kernels/paged_attention.py:125-136), whose counterparts
// these are (together with the FlashAttention varlen call, engine/model/layers.py:246-253).
// Window: a query at position p sees keys p - window + 1 .. p (window = 0: all).
#include "common.cuh"
#include "ie_no_alloc.h"
#include <math.h>
#include <stdio.h>

#ifndef IE_HD
#error "compile with -DIE_HD=<head size, a multiple of 16, at most 128>"
#endif

namespace {
constexpr int HD = IE_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head size must be a multiple of 16 up to 128");
constexpr int C = HD / 8;                 // 16-byte chunks per row
constexpr int KT_PREFILL = HD <= 64 ? 64 : 32;  // keys per tile, prefill kernel
constexpr int KT_DECODE = HD <= 64 ? 32 : 16;   // keys per tile and warp, decode kernel
constexpr int KS = HD / 16;               // 16-dim steps of q.k
constexpr int DT = HD / 8;                // 8-dim tiles of the output
constexpr bool SWZ = (C % 8 == 0);
constexpr int WARPS = 4;
constexpr int MAX_ROWS = 16;
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ int swz(int row, int c) { return SWZ ? (c ^ (row & 7)) : c; }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int bytes = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
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
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (flushes denormals; -inf gives 0): the softmax's exponentials
// are as many as its multiply-adds are few, so the slower exact exp2f would bound the kernel.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Staging keys key0 .. key0 + KT - 1 of one key/value head into shared-memory tiles takes two
// steps that callers keep a whole tile apart, because a dependent trip to memory costs about
// 1,600 cycles on this part and a block-table lookup in front of every copy would dominate:
//   fetch_pages  reads the block-table entries a thread's copies will need (into registers);
//   issue_kv     issues the 16-byte copies of K and V rows from those pages (cp.async).
// NTHREADS threads share the tile (`tid` among them).  Keys outside [lo, hi] are zero-filled.
template <int KT, int NTHREADS>
struct TilePages {
    static constexpr int ITERS = (KT * C + NTHREADS - 1) / NTHREADS;
    // A warp that stages a tile by itself, whole rows per instruction (the decode kernel): lane l
    // keeps the one block-table entry (key0 >> page_shift) + l, and the copies take theirs from
    // the lane that has it.  A tile never spans more than KT <= 32 entries.
    static constexpr bool BY_LANE = NTHREADS == 32 && 32 % C == 0 && KT <= 32;
    int page[BY_LANE ? 1 : ITERS];
};

template <int KT, int NTHREADS>
__device__ __forceinline__ void fetch_pages(TilePages<KT, NTHREADS>& pg, const int* __restrict__ table,
                                            int table_width, int key0, int lo, int hi, int page_shift,
                                            int tid) {
    if constexpr (TilePages<KT, NTHREADS>::BY_LANE) {
        int entry = (key0 >> page_shift) + tid;
        int first = entry << page_shift, last = first + (1 << page_shift) - 1;
        bool wanted = last >= max(key0, lo) && first <= min(key0 + KT - 1, hi) && entry < table_width;
        pg.page[0] = wanted ? table[entry] : -1;
    } else {
#pragma unroll
        for (int i = 0; i < TilePages<KT, NTHREADS>::ITERS; ++i) {
            int idx = i * NTHREADS + tid;
            int kpos = key0 + idx / C;
            int entry = kpos >> page_shift;
            bool wanted = idx < KT * C && kpos >= lo && kpos <= hi && entry < table_width;
            pg.page[i] = wanted ? table[entry] : -1;
        }
    }
}

// REPORT: a missing page inside [lo, hi] is an error (recorded).  Otherwise (the speculative
// first load, issued before the context length is known) it is zero-filled silently and the
// lowest such key position is returned for the caller to judge.
template <int KT, int NTHREADS, bool REPORT>
__device__ __forceinline__ int issue_kv(bf16* ktile, bf16* vtile, const TilePages<KT, NTHREADS>& pg,
                                        const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                        int key0, int lo, int hi, int kvh, int nkv, int page_shift,
                                        int total_pages, int tid, int* err) {
    if constexpr (REPORT && TilePages<KT, NTHREADS>::BY_LANE) {
        // A warp's own tile (the decode kernel): every instruction copies R whole rows, so the
        // shared-memory offsets are constants of the lane and the unrolled iteration, and the
        // global address is one 64-bit multiply-add per instruction.  Tiles that lie wholly
        // inside [lo, hi] (all but a request's first and last) skip the range checks.  (The
        // decode kernel is bound by the number of instructions it issues per tile.)
        constexpr int R = 32 / C;                 // rows per instruction
        constexpr int V = R >= 8 ? 1 : 8 / R;     // distinct (row & 7) patterns over iterations
        const int sub = tid / C, c = tid % C;
        const int page_mask = (1 << page_shift) - 1, entry0 = key0 >> page_shift;
        const unsigned ks = (unsigned)__cvta_generic_to_shared(ktile), vs = (unsigned)__cvta_generic_to_shared(vtile);
        const unsigned page_bytes = (unsigned)(HD * 2) << page_shift;   // one head's rows of a page
        const unsigned long long kb = (unsigned long long)k_cache, vb = (unsigned long long)v_cache;
        unsigned dst_lane[V];
#pragma unroll
        for (int v = 0; v < V; ++v) dst_lane[v] = (unsigned)((sub * C + swz(sub + v * R, c)) * 16);
        const bool inner = key0 >= lo && key0 + KT - 1 <= hi;  // the same for the whole warp
#pragma unroll
        for (int i = 0; i < KT / R; ++i) {
            int kpos = key0 + sub + i * R;
            int page = __shfl_sync(0xffffffffu, pg.page[0], (kpos >> page_shift) - entry0);
            bool in_range = inner || (kpos >= lo && kpos <= hi);
            bool valid = in_range && (unsigned)page < (unsigned)total_pages;
            if (in_range && !valid) ie_report(err, page < 0 ? IE_ERR_TABLE : IE_ERR_PAGE, page, kpos);
            unsigned long long off = valid ? (unsigned long long)(unsigned)(page * nkv + kvh) * page_bytes +
                                                 (unsigned)(((kpos & page_mask) * HD + c * 8) * 2)
                                           : 0ull;
            unsigned dst = (unsigned)(i * R * C * 16) + dst_lane[((i * R) & 7) / R % V];
            int bytes = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(ks + dst), "l"(kb + off), "r"(bytes));
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(vs + dst), "l"(vb + off), "r"(bytes));
        }
        return 0x7fffffff;
    }
    int page_mask = (1 << page_shift) - 1;
    int bad = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < TilePages<KT, NTHREADS>::ITERS; ++i) {
        int idx = i * NTHREADS + tid;
        if (idx >= KT * C) break;
        int row = idx / C, c = idx - row * C;
        int kpos = key0 + row;
        bool in_range = kpos >= lo && kpos <= hi;
        int page = pg.page[i];
        bool valid = in_range && page >= 0 && page < total_pages;
        if (in_range && !valid) {
            if (REPORT) ie_report(err, page < 0 ? IE_ERR_TABLE : IE_ERR_PAGE, page, kpos);
            else bad = min(bad, kpos);
        }
        size_t off = valid ? ((((size_t)page * nkv + kvh) << page_shift) + (kpos & page_mask)) * HD + c * 8 : 0;
        int dst = (row * C + swz(row, c)) * 8;
        cp_async16(ktile + dst, k_cache + off, valid);
        cp_async16(vtile + dst, v_cache + off, valid);
    }
    return bad;
}

// The state of one warp's 16 rows: running maximum (in log2 units), running sum, output.
struct RowState {
    float m[2], l[2];
    float o[DT][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    }
};

// Online softmax of one 16-row tile over one key tile: mask, running maximum and sum, rescale of
// the output so far; on return s holds the weights 2^(scale*s - m).
//   qpos, qlo : for the thread's two rows (lane / 4 and lane / 4 + 8): position of the query
//               and first key it may see; a row that does not exist has qpos < 0
//   key_hi    : last key of the range this call may use (split end)
template <int KT>
__device__ __forceinline__ void softmax_rows(RowState& st, float (&s)[KT / 8][4], int key0,
                                             const int (&qpos)[2], const int (&qlo)[2], int key_hi,
                                             float scale_log2, int lane) {
    constexpr int NT = KT / 8;
    float tile_max[2] = {-INFINITY, -INFINITY};
    int last = key0 + KT - 1;
    bool all_visible = last <= key_hi && last <= qpos[0] && last <= qpos[1] &&
                       key0 >= qlo[0] && key0 >= qlo[1];
    if (__all_sync(0xffffffffu, all_visible)) {  // an inner tile: nothing to mask
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int j = 0; j < 4; ++j) tile_max[j >> 1] = fmaxf(tile_max[j >> 1], s[n][j]);
        }
    } else {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int r = j >> 1;
                int kpos = key0 + n * 8 + (lane & 3) * 2 + (j & 1);
                bool valid = kpos <= qpos[r] && kpos >= qlo[r] && kpos <= key_hi;
                float v = valid ? s[n][j] : -INFINITY;
                s[n][j] = v;
                tile_max[r] = fmaxf(tile_max[r], v);
            }
        }
    }
    float alpha[2], m_safe[2];
    bool grew = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float t = tile_max[r];
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 1));
        t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 2));
        float m_new = fmaxf(st.m[r], t * scale_log2);  // the scale is positive: max commutes
        m_safe[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = fast_exp2(st.m[r] - m_safe[r]);  // 0 when nothing was seen before
        grew = grew || m_new > st.m[r];
        st.m[r] = m_new;
    }
    // the sum and the output so far shrink only when a row's maximum grew; on most tiles of a
    // long context none of the warp's rows does
    if (__any_sync(0xffffffffu, grew)) {
        st.l[0] *= alpha[0];
        st.l[1] *= alpha[1];
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            st.o[d][0] *= alpha[0]; st.o[d][1] *= alpha[0];
            st.o[d][2] *= alpha[1]; st.o[d][3] *= alpha[1];
        }
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float p = fast_exp2(fmaf(s[n][j], scale_log2, -m_safe[j >> 1]));  // -inf stays -inf -> 0
            s[n][j] = p;
            st.l[j >> 1] += p;
        }
    }
}

// One key tile for MT 16-row tiles of one warp: scores, softmax, weighted values.  The K and V
// fragments read from shared memory are used by all MT row tiles (with MT = 2 shared-memory
// traffic per multiply is halved, which is what bounds the prefill kernel otherwise).
//   qf : the warp's query rows as A fragments
template <int KT, int MT>
__device__ __forceinline__ void process_tile(RowState (&st)[MT], const unsigned (&qf)[MT][KS][4],
                                             const bf16* ktile, const bf16* vtile, int key0,
                                             const int (&qpos)[MT][2], const int (&qlo)[MT][2], int key_hi,
                                             float scale_log2, int lane) {
    constexpr int NT = KT / 8;  // 8-key score tiles per key tile
    float s[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int n = 0; n < NT; ++n) s[mt][n][0] = s[mt][n][1] = s[mt][n][2] = s[mt][n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            unsigned b[4];
            int row = n * 8 + (lane & 7) + ((lane >> 4) << 3);
            int c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b, ktile + (row * C + swz(row, c)) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16(s[mt][n], qf[mt][ks], b[0], b[1]);
                mma_bf16(s[mt][n + 1], qf[mt][ks], b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        softmax_rows<KT>(st[mt], s[mt], key0, qpos[mt], qlo[mt], key_hi, scale_log2, lane);
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
        unsigned a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
            a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
            a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
            a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
        }
#pragma unroll
        for (int d = 0; d < DT; d += 2) {
            unsigned b[4];
            int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            int c = d + (lane >> 4);
            ldmatrix_x4_trans(b, vtile + (row * C + swz(row, c)) * 8);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16(st[mt].o[d], a[mt], b[0], b[1]);
                mma_bf16(st[mt].o[d + 1], a[mt], b[2], b[3]);
            }
        }
    }
}

__device__ __forceinline__ void finish_rows(RowState& st) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
}

__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

// The rows of one (request, key/value head) pair in a decode block: the group's query heads
// for each of the request's tokens, row = token * G + head within the group.  Two layouts:
//   wide   (up to 16 rows): the rows are the 16 rows of the instruction, keys its 8 columns;
//   narrow (up to 8 rows):  the products are swapped.  Scores come out transposed, S^T = K Q^T
//          (16 keys are the instruction's rows, the query rows its 8 columns), and so does the
//          output, O^T = V^T P^T (16 dims x 8 rows); P^T reaches the second product through one
//          movmatrix per 8 keys.  A decoded token with a group of 4 fills 4 of 8 columns instead
//          of 4 of 16 rows: half the products and half the exponentials per key, which is what
//          bounds the kernel on long contexts (it issues instructions faster than memory
//          delivers keys only when there are few of them per key).
// Both give the same m, l and o per row up to the order of the 32-bit sums.
constexpr int NARROW_ROWS = 8;
template <bool NARROW> struct DecodeRows;

template <> struct DecodeRows<false> {
    RowState st[1];
    int qpos[1][2], qlo[1][2];
    unsigned qf[1][KS][4];

    __device__ __forceinline__ void load(const bf16* __restrict__ q, int q0, int rows, int G, int nh, int kvh,
                                         int first_qpos, int window, int lane) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int row = (lane >> 2) + r * 8;
            bool exists = row < rows;
            int tok = exists ? row / G : 0, g = exists ? row - tok * G : 0;
            // (a row that does not exist sees every key: its result is never stored, and the tiles
            // inside the context keep the path that masks nothing)
            qpos[0][r] = exists ? first_qpos + tok : 0x7fffffff;
            qlo[0][r] = (exists && window > 0 && qpos[0][r] - window + 1 > 0) ? qpos[0][r] - window + 1 : 0;
            const bf16* qrow = q + ((size_t)(q0 + tok) * nh + kvh * G + g) * HD;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                int d = ks * 16 + (lane & 3) * 2;
                qf[0][ks][r] = exists ? *reinterpret_cast<const unsigned*>(qrow + d) : 0u;
                qf[0][ks][r + 2] = exists ? *reinterpret_cast<const unsigned*>(qrow + d + 8) : 0u;
            }
        }
        st[0].init();
    }
    template <int KT>
    __device__ __forceinline__ void tile(const bf16* ktile, const bf16* vtile, int key0, int key_hi,
                                         float scale_log2, int lane) {
        process_tile<KT, 1>(st, qf, ktile, vtile, key0, qpos, qlo, key_hi, scale_log2, lane);
    }
    // m, l to sm_ml[warp][row][2] and o to sm_o[warp][row][HD]
    __device__ __forceinline__ void to_shared(float* sm_ml, float* sm_o, int warp, int lane) {
        finish_rows(st[0]);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int row = (lane >> 2) + r * 8;
            if ((lane & 3) == 0) {
                sm_ml[(warp * MAX_ROWS + row) * 2] = st[0].m[r];
                sm_ml[(warp * MAX_ROWS + row) * 2 + 1] = st[0].l[r];
            }
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                float* dst = sm_o + ((size_t)(warp * MAX_ROWS + row)) * HD + d * 8 + (lane & 3) * 2;
                dst[0] = st[0].o[d][r * 2];
                dst[1] = st[0].o[d][r * 2 + 1];
            }
        }
    }
};

template <> struct DecodeRows<true> {
    // this thread's two columns (query rows) are 2 * (lane & 3) and the next
    float m[2], l[2];        // running maximum (log2 units) and this thread's share of the sum
    float o[KS][4];          // O^T: 16-dim tiles; [0],[1]: dim lane / 4, [2],[3]: dim lane / 4 + 8
    int cpos[2], clo[2];     // the columns' query position and first visible key
    unsigned qb[KS][2];      // Q^T as B fragments: query row lane / 4, dims 2 * (lane & 3) ..

    __device__ __forceinline__ void load(const bf16* __restrict__ q, int q0, int rows, int G, int nh, int kvh,
                                         int first_qpos, int window, int lane) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            int col = (lane & 3) * 2 + c;
            bool exists = col < rows;
            cpos[c] = exists ? first_qpos + col / G : 0x7fffffff;  // see the wide layout
            clo[c] = (exists && window > 0 && cpos[c] - window + 1 > 0) ? cpos[c] - window + 1 : 0;
            m[c] = -INFINITY;
            l[c] = 0.f;
        }
        int col = lane >> 2;
        bool exists = col < rows;
        int tok = exists ? col / G : 0, g = exists ? col - tok * G : 0;
        const bf16* qrow = q + ((size_t)(q0 + tok) * nh + kvh * G + g) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            int d = ks * 16 + (lane & 3) * 2;
            qb[ks][0] = exists ? *reinterpret_cast<const unsigned*>(qrow + d) : 0u;
            qb[ks][1] = exists ? *reinterpret_cast<const unsigned*>(qrow + d + 8) : 0u;
            o[ks][0] = o[ks][1] = o[ks][2] = o[ks][3] = 0.f;
        }
    }

    template <int KT>
    __device__ __forceinline__ void tile(const bf16* ktile, const bf16* vtile, int key0, int key_hi,
                                         float scale_log2, int lane) {
        constexpr int MT = KT / 16;  // 16-key tiles of the scores
        float s[MT][4];              // [0],[1]: key lane / 4, [2],[3]: key lane / 4 + 8; columns as above
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
        {
            const int arow = (lane & 7) + (((lane >> 3) & 1) << 3), achunk = lane >> 4;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    unsigned a[4];
                    int row = mt * 16 + arow, c = ks * 2 + achunk;
                    ldmatrix_x4(a, ktile + (row * C + swz(row, c)) * 8);
                    mma_bf16(s[mt], a, qb[ks][0], qb[ks][1]);
                }
            }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
        int last = key0 + KT - 1;
        bool all_visible = last <= key_hi && last <= cpos[0] && last <= cpos[1] && key0 >= clo[0] && key0 >= clo[1];
        if (__all_sync(0xffffffffu, all_visible)) {  // an inner tile: nothing to mask
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                tile_max[0] = fmaxf(tile_max[0], fmaxf(s[mt][0], s[mt][2]));
                tile_max[1] = fmaxf(tile_max[1], fmaxf(s[mt][1], s[mt][3]));
            }
        } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int c = j & 1;
                    int kpos = key0 + mt * 16 + (lane >> 2) + ((j >> 1) << 3);
                    bool valid = kpos <= cpos[c] && kpos >= clo[c] && kpos <= key_hi;
                    float v = valid ? s[mt][j] : -INFINITY;
                    s[mt][j] = v;
                    tile_max[c] = fmaxf(tile_max[c], v);
                }
            }
        }
        float alpha[2], m_safe[2];
        bool grew = false;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float t = tile_max[c];  // over the keys of the tile: the lanes that share lane & 3
            t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 4));
            t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 8));
            t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, 16));
            float m_new = fmaxf(m[c], t * scale_log2);  // the scale is positive: max commutes
            m_safe[c] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[c] = fast_exp2(m[c] - m_safe[c]);  // 0 when nothing was seen before
            grew = grew || m_new > m[c];
            m[c] = m_new;
        }
        if (__any_sync(0xffffffffu, grew)) {
            l[0] *= alpha[0];
            l[1] *= alpha[1];
#pragma unroll
            for (int d = 0; d < KS; ++d) {
                o[d][0] *= alpha[0]; o[d][1] *= alpha[1];
                o[d][2] *= alpha[0]; o[d][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float p = fast_exp2(fmaf(s[mt][j], scale_log2, -m_safe[j & 1]));  // -inf stays -inf -> 0
                s[mt][j] = p;
                l[j & 1] += p;
            }
        }
        const int vrow = (lane & 7) + ((lane >> 4) << 3), vchunk = (lane >> 3) & 1;
#pragma unroll
        for (int kk = 0; kk < MT; ++kk) {
            // P^T for 16 keys as B fragments: the weights rounded to bfloat16, 8 x 8 blocks transposed
            unsigned b0 = movmatrix_trans(pack_bf16(s[kk][0], s[kk][1]));
            unsigned b1 = movmatrix_trans(pack_bf16(s[kk][2], s[kk][3]));
#pragma unroll
            for (int d = 0; d < KS; ++d) {
                unsigned a[4];  // V^T: 16 dims x 16 keys
                int row = kk * 16 + vrow, c = d * 2 + vchunk;
                ldmatrix_x4_trans(a, vtile + (row * C + swz(row, c)) * 8);
                mma_bf16(o[d], a, b0, b1);
            }
        }
    }

    __device__ __forceinline__ void to_shared(float* sm_ml, float* sm_o, int warp, int lane) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            l[c] += __shfl_xor_sync(0xffffffffu, l[c], 4);
            l[c] += __shfl_xor_sync(0xffffffffu, l[c], 8);
            l[c] += __shfl_xor_sync(0xffffffffu, l[c], 16);
            int col = (lane & 3) * 2 + c;
            if ((lane >> 2) == 0) {
                sm_ml[(warp * MAX_ROWS + col) * 2] = m[c];
                sm_ml[(warp * MAX_ROWS + col) * 2 + 1] = l[c];
            }
        }
#pragma unroll
        for (int d = 0; d < KS; ++d) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int col = (lane & 3) * 2 + (j & 1), dim = d * 16 + (lane >> 2) + ((j >> 1) << 3);
                sm_o[((size_t)(warp * MAX_ROWS + col)) * HD + dim] = o[d][j];
            }
        }
    }
};

// -------------------------------------------------------------------------------------------------
// Decode: few rows per request.  grid = (requests, kv heads, splits), 8 warps, one block per SM.
//
// A decode step is bound by latency, not by arithmetic: a dependent trip to memory costs about
// a microsecond on this part.  So the kernel keeps the chain of dependent loads short and the
// number of bytes in flight high:
//   * key tiles are dealt round-robin: tile j (keys lo + j*KT ...) goes to split j % S, and
//     within a split to warp (j / S) % 8.  Without a window lo is 0, so a warp knows its first
//     tiles before it knows the context length and fetches their block-table entries at once,
//     while the lengths are still on their way; later entries are fetched a tile ahead of use;
//   * every warp owns a ring of three (K, V) tiles in shared memory and keeps two tiles in
//     flight beyond the one it works on: 192 KB per SM, enough for one block per request and
//     key/value head to stream at the SM's full rate;
//   * with splits > 1 the block that finishes last merges the partial results (ticket counter),
//     always in the order 0, 1, 2, ...
// Partials for splits > 1: part_o[((seq * nkv + kvh) * splits + split) * 16 + row][HD],
// part_ml[... ][2] = (maximum in log2 units, sum).
// -------------------------------------------------------------------------------------------------
constexpr int DWARPS = 8;   // warps of a block that has an SM to itself (192 KB of tiles in flight)
constexpr int DWARPS_SHARED = 4;  // warps of a block when more blocks than SMs run: two blocks share an SM
constexpr int DSTAGES = 3;
template <int NWARPS>
__device__ __forceinline__ void decode_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(NWARPS * 32) : "memory"); }

// A warp's walk over its key tiles j0, j0 + stride, ... < n_tiles of one (request, key/value
// head) pair.  The copies of the first DSTAGES - 1 tiles are in flight (one group each) and
// `next` holds the block-table entries of tile j0 + (DSTAGES - 1) * stride: the copies of tile
// i+2 use entries fetched one tile earlier, and the entries of tile i+3 are fetched now, so no
// lookup is waited for.
template <bool NARROW>
__device__ __forceinline__ void decode_walk(DecodeRows<NARROW>& rs, TilePages<KT_DECODE, 32> next, bf16* ring,
                                            const int* __restrict__ table, int table_width,
                                            const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                            int j0, int stride, int n_tiles, int lo, int hi, int kvh, int nkv,
                                            int page_shift, int total_pages, float scale_log2, int lane, int* err) {
    constexpr int KT = KT_DECODE, TILE_ELEMS = KT * HD;
    int i = 0;
    for (int j = j0; j < n_tiles; j += stride, ++i) {
        int pre = j + (DSTAGES - 1) * stride;
        if (pre < n_tiles) {
            bf16* st_k = ring + (size_t)((i + DSTAGES - 1) % DSTAGES) * 2 * TILE_ELEMS;
            issue_kv<KT, 32, true>(st_k, st_k + TILE_ELEMS, next, k_cache, v_cache, lo + pre * KT, lo, hi,
                                   kvh, nkv, page_shift, total_pages, lane, err);
        }
        cp_async_commit();
        if (pre + stride < n_tiles)
            fetch_pages<KT, 32>(next, table, table_width, lo + (pre + stride) * KT, lo, hi, page_shift, lane);
        cp_async_wait<DSTAGES - 1>();
        __syncwarp();
        const bf16* cur = ring + (size_t)(i % DSTAGES) * 2 * TILE_ELEMS;
        rs.template tile<KT>(cur, cur + TILE_ELEMS, lo + j * KT, hi, scale_log2, lane);
        __syncwarp();
    }
    cp_async_wait<0>();
}

// The end of a decode block (its 8 x 32 compute threads call this together): the warps' partial
// results are merged through shared memory; with one split the block writes the output, with
// more it writes its partial result and the block that finishes last for this (request,
// key/value head) merges all splits, always in the order 0, 1, 2, ...  The ticket counter goes
// back to zero for the next launch.  Barrier 1 is used, so that other warps of the block need
// not take part.
// PAIR: the splits of a (request, key/value head) pair (2, 4 or 8 of them) are one thread-block
// cluster.  All leave their results in the shared memory of the first (the others through the
// cluster's window), and after a cluster barrier the first merges them in the order 0, 1, 2, ...
// and writes the output: no partial results through memory, no ticket.  `stage` is the first's
// [splits][16][HD + 2] floats beyond the tile rings (the rings may still be in use there while
// another block already writes).
__device__ __forceinline__ void pair_store(float* stage, float v) {
    unsigned local = (unsigned)__cvta_generic_to_shared(stage), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(local));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int NWARPS, bool PAIR = false, typename Rows>
__device__ __forceinline__ void decode_merge_store(Rows& rs, unsigned char* smem_raw, int* is_last, int warp,
                                                   int lane, int rows, int G, int q0, int seq, int kvh, int split,
                                                   int num_splits, int nh, int nkv, bf16* __restrict__ out,
                                                   float* __restrict__ part_o, float* __restrict__ part_ml,
                                                   int* __restrict__ tickets) {
    constexpr int WARPS = NWARPS;
    int tid = warp * 32 + lane;
    decode_barrier<NWARPS>();  // every warp is done with its tiles: the shared memory is reused below
    // [warp][row] m, l and [warp][row][HD] o in shared memory
    float* sm_ml = reinterpret_cast<float*>(smem_raw);            // [WARPS][16][2]
    float* sm_o = sm_ml + WARPS * MAX_ROWS * 2;                   // [WARPS][16][HD]
    float* pair_stage = reinterpret_cast<float*>(smem_raw + (size_t)WARPS * DSTAGES * 2 * KT_DECODE * HD * sizeof(bf16));
    (void)pair_stage;
    rs.to_shared(sm_ml, sm_o, warp, lane);
    decode_barrier<NWARPS>();
    for (int idx = tid; idx < rows * HD; idx += WARPS * 32) {
        int row = idx / HD, d = idx - row * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[(w * MAX_ROWS + row) * 2]);
        float m_safe = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            float f = exp2f(sm_ml[(w * MAX_ROWS + row) * 2] - m_safe);
            l += sm_ml[(w * MAX_ROWS + row) * 2 + 1] * f;
            o += sm_o[((size_t)(w * MAX_ROWS + row)) * HD + d] * f;
        }
        if (num_splits == 1) {
            int tok = row / G, g = row - tok * G;
            out[((size_t)(q0 + tok) * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else if (PAIR) {
            float* slot = pair_stage + ((size_t)split * MAX_ROWS + row) * (HD + 2);
            pair_store(slot + d, o);
            if (d == 0) { pair_store(slot + HD, m); pair_store(slot + HD + 1, l); }
        } else {
            size_t p = (((size_t)seq * nkv + kvh) * num_splits + split) * MAX_ROWS + row;
            part_o[p * HD + d] = o;
            if (d == 0) { part_ml[p * 2] = m; part_ml[p * 2 + 1] = l; }
        }
    }
    if (num_splits == 1) return;
    if (PAIR) {
        asm volatile("barrier.cluster.arrive.release;" ::: "memory");
        if (split != 0) return;  // its results are in the first block's shared memory
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
        for (int idx = tid; idx < rows * HD; idx += WARPS * 32) {
            int row = idx / HD, d = idx - row * HD;
            const float* slot = pair_stage + (size_t)row * (HD + 2);
            const size_t next = (size_t)MAX_ROWS * (HD + 2);
            float m = -INFINITY;
            for (int z = 0; z < num_splits; ++z) m = fmaxf(m, slot[z * next + HD]);
            float m_safe = (m == -INFINITY) ? 0.f : m;
            float l = 0.f, o = 0.f;
            for (int z = 0; z < num_splits; ++z) {
                float f = exp2f(slot[z * next + HD] - m_safe);
                l += slot[z * next + HD + 1] * f;
                o += slot[z * next + d] * f;
            }
            int tok = row / G, g = row - tok * G;
            out[((size_t)(q0 + tok) * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        }
        return;
    }
    __threadfence();
    decode_barrier<NWARPS>();
    if (tid == 0) {
        int ticket = atomicAdd(&tickets[seq * nkv + kvh], 1);
        *is_last = (ticket == num_splits - 1);
        if (*is_last) tickets[seq * nkv + kvh] = 0;
    }
    decode_barrier<NWARPS>();
    if (!*is_last) return;
    __threadfence();
    size_t base = ((size_t)seq * nkv + kvh) * num_splits * MAX_ROWS;
    for (int idx = tid; idx < rows * HD; idx += WARPS * 32) {
        int row = idx / HD, d = idx - row * HD;
        // the splits' partial results: loaded eight at a time, merged in the order 0, 1, 2, ...
        float m = -INFINITY;
        for (int s0 = 0; s0 < num_splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                t[j] = s0 + j < num_splits ? __ldcg(part_ml + (base + (size_t)(s0 + j) * MAX_ROWS + row) * 2) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, t[j]);
        }
        float m_safe = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, o = 0.f;
        for (int s0 = 0; s0 < num_splits; s0 += 8) {
            float tm[8], tl[8], to[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bool in = s0 + j < num_splits;
                size_t p = base + (size_t)(in ? s0 + j : 0) * MAX_ROWS + row;
                tm[j] = in ? __ldcg(part_ml + p * 2) : -INFINITY;
                tl[j] = in ? __ldcg(part_ml + p * 2 + 1) : 0.f;
                to[j] = in ? __ldcg(part_o + p * HD + d) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (s0 + j < num_splits) {
                    float f = exp2f(tm[j] - m_safe);
                    l += tl[j] * f;
                    o += to[j] * f;
                }
            }
        }
        int tok = row / G, g = row - tok * G;
        out[((size_t)(q0 + tok) * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}


template <int NWARPS, bool PAIR = false>
__global__ void __launch_bounds__(NWARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, const int* __restrict__ tables,
                        int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                        bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ tickets, int nh, int nkv, int page_shift, int total_pages,
                        float scale_log2, int window, int num_splits, int narrow_rows, const int* __restrict__ order,
                        int* err) {
    constexpr int KT = KT_DECODE, TILE_ELEMS = KT * HD, WARPS = NWARPS;
    __shared__ int is_last;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    // Blocks start in the order of their number: the heads of a request side by side, the requests
    // in the order the caller gives (`order`: the longest first, so that with more blocks than the
    // device runs at once the short ones fill the end) or as they are numbered.
    int kvh = blockIdx.x, seq = order ? order[blockIdx.y] : blockIdx.y, split = blockIdx.z;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int G = nh / nkv;
    const int* table = tables + (size_t)seq * table_width;
    bf16* ring = smem + (size_t)warp * DSTAGES * 2 * TILE_ELEMS;
    int stride = num_splits * WARPS;          // tiles between two tiles of the same warp
    int j0 = split + num_splits * warp;       // this warp's first tile

    // 1. lengths (on their way) and, without a window, the block-table entries of the first
    //    tiles at once: tile j of a request starts at key lo + j*KT and lo is 0
    //    (lengths and tables were copied in before the step's first kernel; the kernel right
    //    before this one wrote the newest keys and values, so those wait for it)
    typedef TilePages<KT, 32> Pages;
    ie_pdl_trigger();
    int q0 = cu_q[seq], q1 = cu_q[seq + 1], ctx = ctx_lens[seq];
    bool early = window <= 0;
    Pages pg[DSTAGES];
    if (early) {
#pragma unroll
        for (int s = 0; s < DSTAGES; ++s)
            fetch_pages<KT, 32>(pg[s], table, table_width, (j0 + s * stride) * KT, 0, 0x7fffffff, page_shift, lane);
    }
    int qlen = q1 - q0;
    int rows = qlen * G;
    int first_qpos = ctx - qlen, hi = ctx - 1;
    int lo = (window > 0 && first_qpos - window + 1 > 0) ? first_qpos - window + 1 : 0;
    int n_tiles = (hi - lo) / KT + 1;         // tiles of the whole request
    // 2. the first tiles' keys and values.  Tiles that lie wholly before this step's tokens
    //    were written by earlier steps: their copies start before the wait for the previous
    //    kernel and overlap it.  A warp whose first tiles reach this step's tokens (short
    //    contexts) starts its copies after the wait.
    bool ahead = early && qlen > 0 && rows <= MAX_ROWS;
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; ++s) {
        int j = j0 + s * stride;
        ahead = ahead && (j >= n_tiles || (j + 1) * KT <= first_qpos);
    }
    if (ahead) {
#pragma unroll
        for (int s = 0; s < DSTAGES - 1; ++s) {
            int j = j0 + s * stride;
            if (j < n_tiles) {
                bf16* st_k = ring + (size_t)s * 2 * TILE_ELEMS;
                issue_kv<KT, 32, true>(st_k, st_k + TILE_ELEMS, pg[s], k_cache, v_cache, lo + j * KT, lo, hi,
                                       kvh, nkv, page_shift, total_pages, lane, err);
            }
            cp_async_commit();
        }
    }
    ie_pdl_wait();
    if (rows > MAX_ROWS || qlen <= 0) return;  // the prefill kernel takes this request
    if (!early) {
#pragma unroll
        for (int s = 0; s < DSTAGES; ++s)
            fetch_pages<KT, 32>(pg[s], table, table_width, lo + (j0 + s * stride) * KT, lo, hi, page_shift, lane);
    }
    if (!ahead) {
#pragma unroll
        for (int s = 0; s < DSTAGES - 1; ++s) {
            int j = j0 + s * stride;
            if (j < n_tiles) {
                bf16* st_k = ring + (size_t)s * 2 * TILE_ELEMS;
                issue_kv<KT, 32, true>(st_k, st_k + TILE_ELEMS, pg[s], k_cache, v_cache, lo + j * KT, lo, hi,
                                       kvh, nkv, page_shift, total_pages, lane, err);
            }
            cp_async_commit();
        }
    }
    // 3. the queries (they needed cu_q) while those are in flight, 4. the ring, 5. the merge
    if (rows <= narrow_rows) {
        DecodeRows<true> rs;
        rs.load(q, q0, rows, G, nh, kvh, first_qpos, window, lane);
        decode_walk(rs, pg[DSTAGES - 1], ring, table, table_width, k_cache, v_cache, j0, stride, n_tiles, lo, hi, kvh,
                    nkv, page_shift, total_pages, scale_log2, lane, err);
        decode_merge_store<NWARPS, PAIR>(rs, smem_raw, &is_last, warp, lane, rows, G, q0, seq, kvh, split, num_splits,
                                         nh, nkv, out, part_o, part_ml, tickets);
    } else {
        DecodeRows<false> rs;
        rs.load(q, q0, rows, G, nh, kvh, first_qpos, window, lane);
        decode_walk(rs, pg[DSTAGES - 1], ring, table, table_width, k_cache, v_cache, j0, stride, n_tiles, lo, hi, kvh,
                    nkv, page_shift, total_pages, scale_log2, lane, err);
        decode_merge_store<NWARPS, PAIR>(rs, smem_raw, &is_last, warp, lane, rows, G, q0, seq, kvh, split, num_splits,
                                         nh, nkv, out, part_o, part_ml, tickets);
    }
}

// -------------------------------------------------------------------------------------------------
// Decode for batches whose contexts differ: the same tile code, the work dealt by length.
//
// The kernel above gives every (request, head) pair the same number of blocks, whatever the
// request's length: right when the contexts are alike, and it knows its tiles from its block
// number alone.  With one long context among short ones the long one's blocks hold the step up.
// Here a fixed one-dimensional grid (as many blocks as the device runs at once) deals the key
// tiles of all requests by their number; every block works the assignment out from the lengths
// (the step's inputs, there before the previous kernel ends), which costs one trip to memory
// more than the kernel above.  A pair that lies in several blocks is merged by the block that
// finishes last (ticket counter), in the order of the blocks.
// Partials: part_o[slot * 16 + row][HD], part_ml[slot * 16 + row][2] = (maximum in log2 units,
// sum); at most pairs + gridDim.x slots are used.
// -------------------------------------------------------------------------------------------------
constexpr int MAX_BALANCED_SEQS = 512;  // requests a balanced launch takes (their running sums sit in shared memory)

// The end of a pair's tiles in a decode block (all its threads call this together): the warps'
// partial results are merged through shared memory.  `whole`: the block held all tiles of the
// pair and writes the output.  Otherwise it writes its partial result to `slot`, and the block
// that finishes last of the pair's `parts` blocks merges their slots first_slot, first_slot + 1,
// ... in that order.  The ticket counter goes back to zero for the next launch.
template <int NWARPS, typename Rows>
__device__ __forceinline__ void decode_merge_slots(Rows& rs, unsigned char* smem_raw, int* is_last, int warp,
                                                   int lane, int rows, int G, int q0, int kvh, int nh, bool whole,
                                                   int slot, int first_slot, int parts, int* ticket,
                                                   bf16* __restrict__ out, float* __restrict__ part_o,
                                                   float* __restrict__ part_ml) {
    constexpr int WARPS = NWARPS;
    int tid = warp * 32 + lane;
    decode_barrier<NWARPS>();  // every warp is done with its tiles: the shared memory is reused below
    // [warp][row] m, l and [warp][row][HD] o in shared memory
    float* sm_ml = reinterpret_cast<float*>(smem_raw);            // [WARPS][16][2]
    float* sm_o = sm_ml + WARPS * MAX_ROWS * 2;                   // [WARPS][16][HD]
    rs.to_shared(sm_ml, sm_o, warp, lane);
    decode_barrier<NWARPS>();
    for (int idx = tid; idx < rows * HD; idx += WARPS * 32) {
        int row = idx / HD, d = idx - row * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[(w * MAX_ROWS + row) * 2]);
        float m_safe = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            float f = exp2f(sm_ml[(w * MAX_ROWS + row) * 2] - m_safe);
            l += sm_ml[(w * MAX_ROWS + row) * 2 + 1] * f;
            o += sm_o[((size_t)(w * MAX_ROWS + row)) * HD + d] * f;
        }
        if (whole) {
            int tok = row / G, g = row - tok * G;
            out[((size_t)(q0 + tok) * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            size_t p = (size_t)slot * MAX_ROWS + row;
            part_o[p * HD + d] = o;
            if (d == 0) { part_ml[p * 2] = m; part_ml[p * 2 + 1] = l; }
        }
    }
    if (whole) return;
    __threadfence();
    decode_barrier<NWARPS>();
    if (tid == 0) {
        int t = atomicAdd(ticket, 1);
        *is_last = (t == parts - 1);
        if (*is_last) *ticket = 0;
    }
    decode_barrier<NWARPS>();
    if (!*is_last) return;
    __threadfence();
    size_t base = (size_t)first_slot * MAX_ROWS;
    for (int idx = tid; idx < rows * HD; idx += WARPS * 32) {
        int row = idx / HD, d = idx - row * HD;
        // the blocks' partial results: loaded eight at a time, merged in the order of the blocks
        float m = -INFINITY;
        for (int s0 = 0; s0 < parts; s0 += 8) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                t[j] = s0 + j < parts ? __ldcg(part_ml + (base + (size_t)(s0 + j) * MAX_ROWS + row) * 2) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, t[j]);
        }
        float m_safe = (m == -INFINITY) ? 0.f : m;
        float l = 0.f, o = 0.f;
        for (int s0 = 0; s0 < parts; s0 += 8) {
            float tm[8], tl[8], to[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bool in = s0 + j < parts;
                size_t p = base + (size_t)(in ? s0 + j : 0) * MAX_ROWS + row;
                tm[j] = in ? __ldcg(part_ml + p * 2) : -INFINITY;
                tl[j] = in ? __ldcg(part_ml + p * 2 + 1) : 0.f;
                to[j] = in ? __ldcg(part_o + p * HD + d) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (s0 + j < parts) {
                    float f = exp2f(tm[j] - m_safe);
                    l += tl[j] * f;
                    o += to[j] * f;
                }
            }
        }
        int tok = row / G, g = row - tok * G;
        out[((size_t)(q0 + tok) * nh + kvh * G + g) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

// Key tiles of a request for the decode kernel (0: the prefill kernel takes it) and its key range.
struct DecodeSeq {
    int q0, qlen, ctx, lo, hi, n_tiles;
};
__device__ __forceinline__ DecodeSeq decode_seq(const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                                                int seq, int G, int window) {
    DecodeSeq d;
    d.q0 = cu_q[seq];
    d.qlen = cu_q[seq + 1] - d.q0;
    d.ctx = ctx_lens[seq];
    int first_qpos = d.ctx - d.qlen;
    d.hi = d.ctx - 1;
    d.lo = (window > 0 && first_qpos - window + 1 > 0) ? first_qpos - window + 1 : 0;
    bool mine = d.qlen > 0 && d.qlen * G <= MAX_ROWS && d.hi >= d.lo;
    d.n_tiles = mine ? (d.hi - d.lo) / KT_DECODE + 1 : 0;
    return d;
}

// Pieces a pair of n tiles is cut into when an even share of all tiles is `share`: the nearest
// whole number of shares, leaving every piece at least a tile per warp.
__device__ __forceinline__ int decode_pieces(int n, int share, int warps) {
    if (n <= 0) return 0;
    int k = (n + share / 2) / share;
    int most = n / warps;
    if (k > most) k = most;
    return k < 1 ? 1 : k;
}

template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
attention_decode_balanced_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                        const bf16* __restrict__ v_cache, const int* __restrict__ tables,
                        int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                        bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ tickets, int num_seqs, int nh, int nkv, int page_shift,
                        int total_pages, float scale_log2, int window, int narrow_rows, int* err) {
    constexpr int KT = KT_DECODE, TILE_ELEMS = KT * HD, WARPS = NWARPS;
    __shared__ int is_last;
    // balanced launches: tiles (of one head) and pieces (of all heads) of the requests before each request
    __shared__ int tiles_before[MAX_BALANCED_SEQS + 1];
    __shared__ int pieces_before[MAX_BALANCED_SEQS + 1];
    __shared__ int warp_sums[NWARPS];
    __shared__ int largest_piece_s;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int G = nh / nkv;
    bf16* ring = smem + (size_t)warp * DSTAGES * 2 * TILE_ELEMS;
    typedef TilePages<KT, 32> Pages;
    ie_pdl_trigger();

    // ---- how the tiles are dealt (lengths and tables were copied in before the step's first
    // kernel: nothing here waits for the kernel before this one).  The tile list: all tiles of
    // request 0's head 0, then its head 1, ..., then request 1's.  Two ways to deal it:
    //   pieces: every (request, head) pair's tiles are cut into k equal pieces, k so that a piece
    //     is about an even share of the list (never less than a tile per warp); pieces are
    //     numbered in list order and block b takes pieces b, b + gridDim.x, ...  A block has one
    //     pair to set up; the blocks' loads differ by as much as the pieces do;
    //   ranges: the list is cut into gridDim.x equal ranges, one per block; a range may end one
    //     pair and begin the next (two set-ups), the loads are equal.
    // Every block takes the same decision from the same lengths: ranges when the pieces would
    // leave the slowest block well behind an even share (ragged batches).
    int num_items, share = 0;
    bool by_range = false;
    {
        long long all_tiles;
        int num_pieces, largest_piece;
        if (num_seqs <= 32) {
            // a small batch: every warp works the sums out by itself, a request to a lane, and
            // no warp waits for another (the warps store the same values)
            int n = lane < num_seqs ? decode_seq(cu_q, ctx_lens, lane, G, window).n_tiles : 0;
            int total = n;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
            all_tiles = (long long)total * nkv;
            share = (int)((all_tiles + gridDim.x - 1) / gridDim.x);
            if (share < WARPS) share = WARPS;
            int k = decode_pieces(n, share, WARPS);
            int incl_t = n, incl_p = k * nkv;
            largest_piece = k > 0 ? (n + k - 1) / k : 0;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int vt = __shfl_up_sync(0xffffffffu, incl_t, off), vp = __shfl_up_sync(0xffffffffu, incl_p, off);
                if (lane >= off) { incl_t += vt; incl_p += vp; }
                largest_piece = max(largest_piece, __shfl_xor_sync(0xffffffffu, largest_piece, off));
            }
            num_pieces = __shfl_sync(0xffffffffu, incl_p, 31);
            if (lane < num_seqs) {
                tiles_before[lane + 1] = incl_t;
                pieces_before[lane + 1] = incl_p;
            }
            if (lane == 0) tiles_before[0] = pieces_before[0] = 0;
            __syncwarp();
        } else {
            int mine = 0;
            for (int s = threadIdx.x; s < num_seqs; s += WARPS * 32) {
                int n = decode_seq(cu_q, ctx_lens, s, G, window).n_tiles;
                tiles_before[s + 1] = n;
                mine += n;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, off);
            if (lane == 0) warp_sums[warp] = mine;
            __syncthreads();
            int total = 0;  // tiles of one head over all requests
#pragma unroll
            for (int w = 0; w < WARPS; ++w) total += warp_sums[w];
            all_tiles = (long long)total * nkv;
            share = (int)((all_tiles + gridDim.x - 1) / gridDim.x);
            if (share < WARPS) share = WARPS;
            if (warp == 0) {  // running sums of tiles and of pieces: a lane sums its stretch, the warp scans the lanes' sums
                int per = (num_seqs + 31) / 32, first = lane * per, sum_t = 0, sum_p = 0, largest = 0;
                for (int i = 0; i < per; ++i)
                    if (first + i < num_seqs) {
                        int n = tiles_before[first + i + 1], k = decode_pieces(n, share, WARPS);
                        sum_t += n;
                        sum_p += k * nkv;
                        if (k > 0) largest = max(largest, (n + k - 1) / k);
                    }
                int incl_t = sum_t, incl_p = sum_p;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    int vt = __shfl_up_sync(0xffffffffu, incl_t, off), vp = __shfl_up_sync(0xffffffffu, incl_p, off);
                    if (lane >= off) { incl_t += vt; incl_p += vp; }
                    largest = max(largest, __shfl_xor_sync(0xffffffffu, largest, off));
                }
                int run_t = incl_t - sum_t, run_p = incl_p - sum_p;
                for (int i = 0; i < per; ++i)
                    if (first + i < num_seqs) {
                        int n = tiles_before[first + i + 1];
                        run_t += n;
                        run_p += decode_pieces(n, share, WARPS) * nkv;
                        tiles_before[first + i + 1] = run_t;
                        pieces_before[first + i + 1] = run_p;
                    }
                if (lane == 0) {
                    tiles_before[0] = 0;
                    pieces_before[0] = 0;
                    largest_piece_s = largest;
                }
            }
            __syncthreads();
            num_pieces = pieces_before[num_seqs];
            largest_piece = largest_piece_s;
        }
        long long rounds = (num_pieces + (int)gridDim.x - 1) / (int)gridDim.x;
        // a pair's set-up costs a block about as much as six tiles per warp
        by_range = rounds * largest_piece > (long long)share + 6 * WARPS;
        num_items = by_range ? (int)min(all_tiles, (long long)0x7fffffff) : num_pieces;
    }

    bool waited = false;
    // items: tiles (ranges) or pieces; a block's first item, and how many it takes at a time
    long long item = by_range ? (long long)blockIdx.x * share : blockIdx.x;
    int left = by_range ? share : 1;   // ranges: tiles still to take from this block's range
    int seq = -1, kvh = 0, tile0 = 0;  // ranges: where the next tile of the range lies
    while (item < num_items && left > 0) {
        int part = 0, parts = 1, tile_end, first_slot = 0, slot = 0;
        DecodeSeq ds;
        if (by_range) {
            if (seq < 0) {
                // the request that holds tile `item`: the last one whose first tile is at or before it
                int lo_s = 0, hi_s = num_seqs - 1;
                while (lo_s < hi_s) {
                    int mid = (lo_s + hi_s + 1) >> 1;
                    if ((long long)tiles_before[mid] * nkv <= item) lo_s = mid; else hi_s = mid - 1;
                }
                seq = lo_s;
                int n = tiles_before[seq + 1] - tiles_before[seq];  // > 0: the tile lies inside it
                int r = (int)(item - (long long)tiles_before[seq] * nkv);
                kvh = r / n;
                tile0 = r - kvh * n;
            }
            ds = decode_seq(cu_q, ctx_lens, seq, G, window);
            if (ds.n_tiles == 0) {  // the prefill kernel's request: no tiles in the list
                ++seq; kvh = 0; tile0 = 0;
                if (seq >= num_seqs) break;
                continue;
            }
            tile_end = min(ds.n_tiles, tile0 + left);
            if (tile0 > 0 || tile_end < ds.n_tiles) {
                // the pair lies in several blocks: one slot each, numbered pair + block (unique:
                // later pairs lie in later blocks)
                long long pair_begin = (long long)tiles_before[seq] * nkv + (long long)kvh * ds.n_tiles;
                int first_block = (int)(pair_begin / share);
                parts = (int)((pair_begin + ds.n_tiles - 1) / share) - first_block + 1;
                first_slot = seq * nkv + kvh + first_block;
                slot = seq * nkv + kvh + (int)blockIdx.x;
            }
        } else {
            int piece = (int)item;
            int lo_s = 0, hi_s = num_seqs - 1;
            while (lo_s < hi_s) {
                int mid = (lo_s + hi_s + 1) >> 1;
                if (pieces_before[mid] <= piece) lo_s = mid; else hi_s = mid - 1;
            }
            seq = lo_s;
            parts = (pieces_before[seq + 1] - pieces_before[seq]) / nkv;  // > 0: the piece lies inside it
            int r = piece - pieces_before[seq];
            kvh = r / parts;
            part = r - kvh * parts;
            ds = decode_seq(cu_q, ctx_lens, seq, G, window);
            tile0 = (int)((long long)part * ds.n_tiles / parts);
            tile_end = (int)((long long)(part + 1) * ds.n_tiles / parts);
            first_slot = pieces_before[seq] + kvh * parts;  // the pair's pieces have consecutive numbers
            slot = first_slot + part;
        }
        bool whole = parts == 1;
        const int* table = tables + (size_t)seq * table_width;
        int q0 = ds.q0, qlen = ds.qlen, lo = ds.lo, hi = ds.hi;
        int rows = qlen * G, first_qpos = ds.ctx - qlen;
        int n_tiles = tile_end;                   // tiles of this pair the block works on end here
        int j0 = tile0 + warp, stride = WARPS;    // this warp's first tile, tiles between two of its tiles

        // 1. block-table entries of the first tiles
        Pages pg[DSTAGES];
#pragma unroll
        for (int s = 0; s < DSTAGES; ++s)
            fetch_pages<KT, 32>(pg[s], table, table_width, lo + (j0 + s * stride) * KT, lo, hi, page_shift, lane);
        // 2. the first tiles' keys and values.  Tiles that lie wholly before this step's tokens
        //    were written by earlier steps: their copies start before the wait for the previous
        //    kernel and overlap it.  A warp whose first tiles reach this step's tokens (short
        //    contexts) starts its copies after the wait.
        bool ahead = !waited;
#pragma unroll
        for (int s = 0; s < DSTAGES - 1; ++s) {
            int j = j0 + s * stride;
            ahead = ahead && (j >= n_tiles || lo + (j + 1) * KT <= first_qpos);
        }
        if (ahead) {
#pragma unroll
            for (int s = 0; s < DSTAGES - 1; ++s) {
                int j = j0 + s * stride;
                if (j < n_tiles) {
                    bf16* st_k = ring + (size_t)s * 2 * TILE_ELEMS;
                    issue_kv<KT, 32, true>(st_k, st_k + TILE_ELEMS, pg[s], k_cache, v_cache, lo + j * KT, lo, hi,
                                           kvh, nkv, page_shift, total_pages, lane, err);
                }
                cp_async_commit();
            }
        }
        if (!waited) {
            ie_pdl_wait();
            waited = true;
        } else {
            ahead = false;
        }
        if (!ahead) {
#pragma unroll
            for (int s = 0; s < DSTAGES - 1; ++s) {
                int j = j0 + s * stride;
                if (j < n_tiles) {
                    bf16* st_k = ring + (size_t)s * 2 * TILE_ELEMS;
                    issue_kv<KT, 32, true>(st_k, st_k + TILE_ELEMS, pg[s], k_cache, v_cache, lo + j * KT, lo, hi,
                                           kvh, nkv, page_shift, total_pages, lane, err);
                }
                cp_async_commit();
            }
        }
        // 3. the queries while those are in flight, 4. the ring, 5. merge the warps; write the
        //    output or this block's partial result
        if (rows <= narrow_rows) {
            DecodeRows<true> rs;
            rs.load(q, q0, rows, G, nh, kvh, first_qpos, window, lane);
            decode_walk(rs, pg[DSTAGES - 1], ring, table, table_width, k_cache, v_cache, j0, stride, n_tiles, lo, hi,
                        kvh, nkv, page_shift, total_pages, scale_log2, lane, err);
            decode_merge_slots<NWARPS>(rs, smem_raw, &is_last, warp, lane, rows, G, q0, kvh, nh, whole, slot,
                                       first_slot, parts, tickets + seq * nkv + kvh, out, part_o, part_ml);
        } else {
            DecodeRows<false> rs;
            rs.load(q, q0, rows, G, nh, kvh, first_qpos, window, lane);
            decode_walk(rs, pg[DSTAGES - 1], ring, table, table_width, k_cache, v_cache, j0, stride, n_tiles, lo, hi,
                        kvh, nkv, page_shift, total_pages, scale_log2, lane, err);
            decode_merge_slots<NWARPS>(rs, smem_raw, &is_last, warp, lane, rows, G, q0, kvh, nh, whole, slot,
                                       first_slot, parts, tickets + seq * nkv + kvh, out, part_o, part_ml);
        }
        decode_barrier<NWARPS>();  // the merge read shared memory that the next pair's copies overwrite
        if (by_range) {
            int took = tile_end - tile0;
            left -= took;
            item += took;
            tile0 = 0;
            if (++kvh == nkv) { kvh = 0; ++seq; }
            if (seq >= num_seqs) break;
        } else {
            item += gridDim.x;
        }
    }
    if (!waited) ie_pdl_wait();
}

// -------------------------------------------------------------------------------------------------
// Prefill: portions with more than 16 rows.  grid = (128-token tiles over all requests, heads);
// four warps of 32 rows (two 16-row tiles that share every K and V fragment).
// -------------------------------------------------------------------------------------------------
constexpr int PMT = HD <= 64 ? 2 : 1;  // 16-row tiles per warp (registers allow two up to head size 64)
constexpr int BM = WARPS * PMT * 16;   // query tokens per block

__global__ void __launch_bounds__(WARPS * 32)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, const int* __restrict__ tables,
                         int table_width, const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                         bf16* __restrict__ out, int num_seqs, int nh, int nkv, int page_shift,
                         int total_pages, float scale_log2, int window, int* err) {
    constexpr int KT = KT_PREFILL, TILE_ELEMS = KT * HD;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int head = blockIdx.y, G = nh / nkv, kvh = head / G;
    // which request and which query tile of it is this block's?
    ie_pdl_trigger();
    ie_pdl_wait();
    // late tiles of a portion see the most keys: they go first so the short ones fill the tail
    int tile = gridDim.x - 1 - blockIdx.x, seq = -1, t0 = 0, q0 = 0, qlen = 0;
    for (int s = 0; s < num_seqs; ++s) {
        int a = cu_q[s], n = cu_q[s + 1] - a;
        int tiles = (n * G > MAX_ROWS) ? (n + BM - 1) / BM : 0;
        if (tile < tiles) { seq = s; t0 = tile * BM; q0 = a; qlen = n; break; }
        tile -= tiles;
    }
    if (seq < 0) return;
    int ctx = ctx_lens[seq];
    const int* table = tables + (size_t)seq * table_width;
    int first_qpos = ctx - qlen;                 // position of the portion's first token
    int tile_rows = min(BM, qlen - t0);
    int cta_qpos_lo = first_qpos + t0, cta_qpos_hi = first_qpos + t0 + tile_rows - 1;
    int lo = (window > 0 && cta_qpos_lo - window + 1 > 0) ? cta_qpos_lo - window + 1 : 0;
    int key_begin = (lo / KT) * KT;              // tiles are aligned to absolute position 0
    int n_tiles = (cta_qpos_hi - key_begin) / KT + 1;

    constexpr int WROWS = PMT * 16;  // rows of one warp
    int qpos[PMT][2], qlo[PMT][2];
    unsigned qf[PMT][KS][4];
#pragma unroll
    for (int mt = 0; mt < PMT; ++mt) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int row = warp * WROWS + mt * 16 + (lane >> 2) + r * 8;
            bool exists = row < tile_rows;
            qpos[mt][r] = exists ? cta_qpos_lo + row : -1;
            qlo[mt][r] = (window > 0 && qpos[mt][r] - window + 1 > 0) ? qpos[mt][r] - window + 1 : 0;
            const bf16* qrow = q + ((size_t)(q0 + t0 + (exists ? row : 0)) * nh + head) * HD;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                int d = ks * 16 + (lane & 3) * 2;
                qf[mt][ks][r] = exists ? *reinterpret_cast<const unsigned*>(qrow + d) : 0u;
                qf[mt][ks][r + 2] = exists ? *reinterpret_cast<const unsigned*>(qrow + d + 8) : 0u;
            }
        }
    }
    int warp_hi = min(cta_qpos_lo + warp * WROWS + WROWS - 1, cta_qpos_hi);  // last position this warp's rows see
    int warp_lo_pos = cta_qpos_lo + warp * WROWS;
    int warp_lo = (window > 0 && warp_lo_pos - window + 1 > 0) ? warp_lo_pos - window + 1 : 0;
    bool warp_has_rows = warp * WROWS < tile_rows;

    RowState st[PMT];
#pragma unroll
    for (int mt = 0; mt < PMT; ++mt) st[mt].init();
    // Three stages of (K, V) tiles; the block-table entries of a tile are fetched one tile
    // before its copies are issued, so no lookup is waited for inside the loop.
    typedef TilePages<KT, WARPS * 32> Pages;
    constexpr int PSTAGES = 3;
    Pages pg[PSTAGES];
#pragma unroll
    for (int s = 0; s < PSTAGES; ++s)
        fetch_pages<KT, WARPS * 32>(pg[s], table, table_width, key_begin + s * KT, lo, cta_qpos_hi, page_shift, threadIdx.x);
#pragma unroll
    for (int s = 0; s < PSTAGES - 1; ++s) {
        if (s < n_tiles) {
            bf16* st_k = smem + (size_t)s * 2 * TILE_ELEMS;
            issue_kv<KT, WARPS * 32, true>(st_k, st_k + TILE_ELEMS, pg[s], k_cache, v_cache, key_begin + s * KT,
                                           lo, cta_qpos_hi, kvh, nkv, page_shift, total_pages, threadIdx.x, err);
        }
        cp_async_commit();
    }
    Pages next = pg[PSTAGES - 1];
    for (int t = 0; t < n_tiles; ++t) {
        int key0 = key_begin + t * KT;
        int pre = t + PSTAGES - 1;
        cp_async_wait<PSTAGES - 2>();  // tile t has landed (this thread's part)
        __syncthreads();               // ... everybody's part; and tile t-1 is no longer read
        if (pre < n_tiles) {
            bf16* st_k = smem + (size_t)(pre % PSTAGES) * 2 * TILE_ELEMS;
            issue_kv<KT, WARPS * 32, true>(st_k, st_k + TILE_ELEMS, next, k_cache, v_cache, key_begin + pre * KT,
                                           lo, cta_qpos_hi, kvh, nkv, page_shift, total_pages, threadIdx.x, err);
        }
        cp_async_commit();
        if (pre + 1 < n_tiles)
            fetch_pages<KT, WARPS * 32>(next, table, table_width, key_begin + (pre + 1) * KT, lo, cta_qpos_hi,
                                        page_shift, threadIdx.x);
        const bf16* cur = smem + (size_t)(t % PSTAGES) * 2 * TILE_ELEMS;
        if (warp_has_rows && key0 <= warp_hi && key0 + KT - 1 >= warp_lo)
            process_tile<KT, PMT>(st, qf, cur, cur + TILE_ELEMS, key0, qpos, qlo, cta_qpos_hi, scale_log2, lane);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int mt = 0; mt < PMT; ++mt) {
        finish_rows(st[mt]);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            int row = warp * WROWS + mt * 16 + (lane >> 2) + r * 8;
            if (row >= tile_rows) continue;
            float inv = st[mt].l[r] > 0.f ? 1.0f / st[mt].l[r] : 0.f;
            bf16* orow = out + ((size_t)(q0 + t0 + row) * nh + head) * HD;
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                __nv_bfloat162 v = __floats2bfloat162_rn(st[mt].o[d][r * 2] * inv, st[mt].o[d][r * 2 + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(orow + d * 8 + (lane & 3) * 2) = v;
            }
        }
    }
}

constexpr size_t decode_smem(int warps) {
    size_t tiles = (size_t)warps * DSTAGES * 2 * KT_DECODE * HD * sizeof(bf16);
    size_t merge = (size_t)warps * MAX_ROWS * (2 + HD) * sizeof(float);
    return tiles > merge ? tiles : merge;
}
constexpr size_t PREFILL_SMEM = (size_t)3 * 2 * KT_PREFILL * HD * sizeof(bf16);
}  // namespace

constexpr size_t PAIR_SLOT_BYTES = (size_t)MAX_ROWS * (HD + 2) * sizeof(float);
constexpr size_t MAX_DYNAMIC_SMEM = 227 * 1024;
// The largest number of splits (2, 4, 8) that merge as one cluster of blocks through shared
// memory; 0: every merge goes through memory.
inline int& decode_pair_enabled() {
    static int enabled = 8;
    return enabled;
}

// Requests with at most this many rows (tokens x group size) run the decode kernels' swapped
// products (DecodeRows<true>); 0: all run the 16-row layout.
inline int& decode_narrow_rows() {
    static int rows = NARROW_ROWS;
    return rows;
}

IE_API int ie_attention_head_dim() { return HD; }
IE_API void ie_set_decode_pair(int max_splits) { decode_pair_enabled() = max_splits; }
IE_API void ie_set_decode_narrow(int enabled) { decode_narrow_rows() = enabled ? NARROW_ROWS : 0; }

// Query tokens one block of the prefill kernel takes (callers count tiles with it).
IE_API int ie_attention_prefill_rows() { return BM; }
IE_API void ie_set_pdl(int enabled) { ie_pdl_enabled() = enabled ? 1 : 0; }

// Floats of scratch the decode kernel needs for `num_seqs` requests at `num_splits` splits:
// part_o first, then part_ml.
IE_API long long ie_attention_decode_scratch_floats(int num_seqs, int nkv, int num_splits) {
    if (num_splits <= 1) return 0;
    return (long long)num_seqs * nkv * num_splits * MAX_ROWS * (HD + 2);
}

namespace {
// How many clusters of `num_splits` decode blocks of NWARPS warps the current device runs at one
// time (a cluster's blocks need room in one group of SMs together, so fewer than SMs over
// num_splits): a grid with more clusters than that takes a second round.  0 if the splits do not
// merge as a cluster or the runtime cannot say.
template <int NWARPS>
int max_decode_clusters(int num_splits) {
    size_t smem = decode_smem(NWARPS) + (size_t)num_splits * PAIR_SLOT_BYTES;
    if (!(num_splits == 2 || num_splits == 4 || num_splits == 8) || smem > MAX_DYNAMIC_SMEM) return 0;
    auto kernel = attention_decode_kernel<NWARPS, true>;
    size_t limit = decode_smem(NWARPS) + (size_t)8 * PAIR_SLOT_BYTES;
    if (limit > MAX_DYNAMIC_SMEM) limit = MAX_DYNAMIC_SMEM;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, (unsigned)num_splits);
    cfg.blockDim = dim3(NWARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned)num_splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return clusters;
}

// The same, asked once per device and cluster size.
template <int NWARPS>
int decode_clusters_at_once(int num_splits) {
    static int known[IE_MAX_DEVICES][3] = {};  // 0: not asked yet, else the answer + 1
    int dev = -1, slot = num_splits == 2 ? 0 : num_splits == 4 ? 1 : 2;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= IE_MAX_DEVICES) return max_decode_clusters<NWARPS>(num_splits);
    if (known[dev][slot] == 0) known[dev][slot] = max_decode_clusters<NWARPS>(num_splits) + 1;
    return known[dev][slot] - 1;
}
}  // namespace

IE_API int ie_attention_decode_max_clusters(int num_splits) { return decode_clusters_at_once<DWARPS>(num_splits); }

namespace {
template <int NWARPS>
int launch_decode_as(const void* q, const void* k_cache, const void* v_cache, const int* tables, int table_width,
                     const int* cu_q, const int* ctx_lens, void* out, float* part_o, float* part_ml, int* tickets,
                     int num_seqs, int nh, int nkv, int page_shift, int total_pages, float scale, int window,
                     int num_splits, const int* order, int* err, cudaStream_t s) {
    dim3 grid(nkv, num_seqs, num_splits);
    size_t pair_smem = decode_smem(NWARPS) + (size_t)num_splits * PAIR_SLOT_BYTES;
    // the splits are a cluster that merges through shared memory, if all clusters run at one time
    // (where the runtime cannot say how many do, it is taken that they do)
    bool as_cluster = (num_splits == 2 || num_splits == 4 || num_splits == 8) && num_splits <= decode_pair_enabled() &&
                      pair_smem <= MAX_DYNAMIC_SMEM;
    if (as_cluster) {
        int fit = decode_clusters_at_once<NWARPS>(num_splits);
        as_cluster = fit <= 0 || (long long)num_seqs * nkv <= fit;
    }
    if (as_cluster) {
        static IePerDevice configured_pair;
        size_t smem = decode_smem(NWARPS) + (size_t)8 * PAIR_SLOT_BYTES;  // (what the function is set up for)
        if (smem > MAX_DYNAMIC_SMEM) smem = MAX_DYNAMIC_SMEM;
        cudaError_t e = ie_allow_smem(configured_pair, attention_decode_kernel<NWARPS, true>, smem);
        if (e != cudaSuccess) return (int)e;
        smem = pair_smem;
        return ie_launch_cluster(attention_decode_kernel<NWARPS, true>, grid, dim3(NWARPS * 32), smem, s,
                                 dim3(1, 1, (unsigned)num_splits),
                                 (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tables, table_width, cu_q,
                                 ctx_lens, (bf16*)out, part_o, part_ml, tickets, nh, nkv, page_shift, total_pages,
                                 scale * 1.4426950408889634f, window, num_splits, decode_narrow_rows(), order, err);
    }
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, attention_decode_kernel<NWARPS>, decode_smem(NWARPS));
    if (e != cudaSuccess) return (int)e;
    return ie_launch(attention_decode_kernel<NWARPS>, grid, dim3(NWARPS * 32), decode_smem(NWARPS), s,
                     (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tables, table_width, cu_q,
                     ctx_lens, (bf16*)out, part_o, part_ml, tickets, nh, nkv, page_shift, total_pages,
                     scale * 1.4426950408889634f, window, num_splits, decode_narrow_rows(), order, err);
}

// Blocks of `warps` warps an SM holds at one time (by their shared memory).
constexpr int blocks_per_sm(int warps) {
    size_t n = (MAX_DYNAMIC_SMEM + 1024) / (decode_smem(warps) + 1024);
    return n > 8 ? 8 : (int)n;
}

// With at most one block per SM a block takes the SM's whole shared memory for tiles in flight;
// with more blocks than SMs, blocks of half the size run two to an SM, so that one block's
// start-up and merge overlap the other's streaming.  The choice depends on the grid alone.
// `small_blocks` (the caller's choice): blocks of 3 or 2 warps, three or four to an SM at head size
// 64, so that a grid of more than two blocks per SM still runs in one round (40 requests x 8 heads
// of 1,024 tokens: 320 blocks, 25.8 us in two rounds of four-warp blocks, 17.9 us in one round of
// three-warp blocks; 64 requests: 27.3 us, 24.8 us in two-warp blocks).  Requests of very different
// lengths lose: the longest one's block has fewer warps to walk it.
int launch_decode(const void* q, const void* k_cache, const void* v_cache, const int* tables, int table_width,
                  const int* cu_q, const int* ctx_lens, void* out, float* part_o, float* part_ml, int* tickets,
                  int num_seqs, int nh, int nkv, int page_shift, int total_pages, float scale, int window,
                  int num_splits, const int* order, int small_blocks, int* err, cudaStream_t s) {
    int sms = ie_sm_count();
    long long blocks = (long long)num_seqs * nkv * num_splits;
    if (small_blocks == 3 && blocks > sms)
        return launch_decode_as<3>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o,
                                   part_ml, tickets, num_seqs, nh, nkv, page_shift, total_pages, scale,
                                   window, num_splits, order, err, s);
    if (small_blocks == 2 && blocks > sms)
        return launch_decode_as<2>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o,
                                   part_ml, tickets, num_seqs, nh, nkv, page_shift, total_pages, scale,
                                   window, num_splits, order, err, s);
    if (blocks > sms)
        return launch_decode_as<DWARPS_SHARED>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o,
                                               part_ml, tickets, num_seqs, nh, nkv, page_shift, total_pages, scale,
                                               window, num_splits, order, err, s);
    return launch_decode_as<DWARPS>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o, part_ml,
                                    tickets, num_seqs, nh, nkv, page_shift, total_pages, scale, window, num_splits,
                                    order, err, s);
}
}  // namespace

// Requests with (tokens x group size) <= 16 rows.  With num_splits > 1 the kernel needs
// `scratch` (ie_attention_decode_scratch_floats floats; contents do not matter) and `tickets`
// (num_seqs * nkv ints that are zero before the first launch; every launch leaves them zero
// again).  Both may be null when num_splits == 1.
IE_API int ie_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                               const int* tables, int table_width, const int* cu_q,
                               const int* ctx_lens, void* out, float* scratch, int* tickets,
                               int num_seqs, int nh, int nkv, int page_size, int total_pages,
                               float scale, int window, int num_splits, int* err, void* stream) {
    if (num_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || (page_size & (page_size - 1)) != 0 || num_splits < 1 ||
        (num_splits > 1 && (scratch == nullptr || tickets == nullptr)))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)num_seqs * nkv * num_splits * MAX_ROWS * HD : nullptr;
    return launch_decode(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o, part_ml, tickets,
                         num_seqs, nh, nkv, page_shift, total_pages, scale, window, num_splits, nullptr, 0, err,
                         (cudaStream_t)stream);
}

// How many decode blocks of `warps` warps an SM holds at one time.
IE_API int ie_attention_decode_blocks_per_sm(int warps) { return warps >= 1 && warps <= 8 ? blocks_per_sm(warps) : 0; }

// The same with the order in which the requests' blocks start: `order[i]` is the request that is
// i-th (every request once; the longest first pays when the step has more blocks than the device
// runs at once and contexts of different lengths), and with the choice of blocks of 3 or 2 warps
// (`small_blocks` 3, 2; 0: four or eight, by the grid) for grids of more blocks than SMs.
IE_API int ie_attention_decode_ordered(const void* q, const void* k_cache, const void* v_cache,
                                       const int* tables, int table_width, const int* cu_q,
                                       const int* ctx_lens, void* out, float* scratch, int* tickets,
                                       int num_seqs, int nh, int nkv, int page_size, int total_pages,
                                       float scale, int window, int num_splits, const int* order,
                                       int small_blocks, int* err, void* stream) {
    if (num_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || (page_size & (page_size - 1)) != 0 || num_splits < 1 ||
        (num_splits > 1 && (scratch == nullptr || tickets == nullptr)))
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)num_seqs * nkv * num_splits * MAX_ROWS * HD : nullptr;
    return launch_decode(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o, part_ml, tickets,
                         num_seqs, nh, nkv, page_shift, total_pages, scale, window, num_splits, order, small_blocks,
                         err, (cudaStream_t)stream);
}

namespace {
// Blocks of a balanced launch: what the device runs at once (blocks of four warps, two to an SM,
// when there are more pairs than SMs), no more than `max_blocks_per_pair` times the pairs.
int balanced_sms() { return ie_sm_count(); }
long long balanced_blocks(long long pairs, int max_blocks_per_pair) {
    int sms = balanced_sms();
    long long slots = pairs > sms ? 2LL * sms : sms;
    long long want = pairs * (max_blocks_per_pair < 1 ? 1 : max_blocks_per_pair);
    return want < slots ? want : slots;
}

template <int NWARPS>
int launch_balanced_as(const void* q, const void* k_cache, const void* v_cache, const int* tables, int table_width,
                       const int* cu_q, const int* ctx_lens, void* out, float* part_o, float* part_ml, int* tickets,
                       int num_seqs, int nh, int nkv, int page_shift, int total_pages, float scale, int window,
                       int blocks, int* err, cudaStream_t s) {
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, attention_decode_balanced_kernel<NWARPS>, decode_smem(NWARPS));
    if (e != cudaSuccess) return (int)e;
    return ie_launch(attention_decode_balanced_kernel<NWARPS>, dim3(blocks), dim3(NWARPS * 32), decode_smem(NWARPS), s,
                     (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tables, table_width, cu_q, ctx_lens,
                     (bf16*)out, part_o, part_ml, tickets, num_seqs, nh, nkv, page_shift, total_pages,
                     scale * 1.4426950408889634f, window, decode_narrow_rows(), err);
}
}  // namespace

// Requests a balanced launch takes at most.
IE_API int ie_attention_decode_balanced_max_seqs() { return MAX_BALANCED_SEQS; }

// Floats of scratch `ie_attention_decode_balanced` needs: a partial result for every (pair, block)
// that can occur.
IE_API long long ie_attention_decode_balanced_scratch_floats(int num_seqs, int nkv, int max_blocks_per_pair) {
    if (num_seqs <= 0 || nkv <= 0) return 0;
    long long pairs = (long long)num_seqs * nkv;
    return (pairs + balanced_blocks(pairs, max_blocks_per_pair)) * MAX_ROWS * (HD + 2);
}

// The decode attention of `ie_attention_decode` with the key tiles of all requests dealt evenly
// over the blocks: for batches whose contexts differ in length (at most
// ie_attention_decode_balanced_max_seqs requests).  `scratch`:
// ie_attention_decode_balanced_scratch_floats floats (contents do not matter); `tickets`:
// num_seqs * nkv ints that are zero before the first launch (every launch leaves them zero).
IE_API int ie_attention_decode_balanced(const void* q, const void* k_cache, const void* v_cache,
                                        const int* tables, int table_width, const int* cu_q,
                                        const int* ctx_lens, void* out, float* scratch, int* tickets,
                                        int num_seqs, int nh, int nkv, int page_size, int total_pages,
                                        float scale, int window, int max_blocks_per_pair, int* err, void* stream) {
    if (num_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || (page_size & (page_size - 1)) != 0 || num_seqs > MAX_BALANCED_SEQS ||
        scratch == nullptr || tickets == nullptr)
        return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    long long pairs = (long long)num_seqs * nkv;
    long long blocks = balanced_blocks(pairs, max_blocks_per_pair);
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)(pairs + blocks) * MAX_ROWS * HD;
    cudaStream_t s = (cudaStream_t)stream;
    if (pairs > balanced_sms())
        return launch_balanced_as<DWARPS_SHARED>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o,
                                                 part_ml, tickets, num_seqs, nh, nkv, page_shift, total_pages, scale,
                                                 window, (int)blocks, err, s);
    return launch_balanced_as<DWARPS>(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, part_o, part_ml,
                                      tickets, num_seqs, nh, nkv, page_shift, total_pages, scale, window, (int)blocks,
                                      err, s);
}

// Requests with more than 16 rows.  `max_tiles` bounds the number of query tiles over all
// such requests, each tile being ie_attention_prefill_rows() tokens.
IE_API int ie_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                                const int* tables, int table_width, const int* cu_q,
                                const int* ctx_lens, void* out, int num_seqs, int max_tiles,
                                int nh, int nkv, int page_size, int total_pages, float scale,
                                int window, int* err, void* stream) {
    if (num_seqs <= 0 || max_tiles <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || (page_size & (page_size - 1)) != 0) return (int)cudaErrorInvalidValue;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) ++page_shift;
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, attention_prefill_kernel, PREFILL_SMEM);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(max_tiles, nh);
    return ie_launch(attention_prefill_kernel, grid, dim3(WARPS * 32), PREFILL_SMEM, (cudaStream_t)stream,
                     (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, tables, table_width, cu_q,
                     ctx_lens, (bf16*)out, num_seqs, nh, nkv, page_shift, total_pages,
                     scale * 1.4426950408889634f, window, err);
}

// -------------------------------------------------------------------------------------------------
// The decode kernel for callers that cannot allocate device memory (declared in ie_no_alloc.h).
// The split partials live in a fixed array that is part of this library's device image.
// -------------------------------------------------------------------------------------------------
namespace {
// Scratch for the split partials of `ie_attention_decode_static`.  Every GPU that loads this
// library holds these 4 MiB until the process exits.
static __device__ __align__(256) float g_static_decode_scratch[IE_STATIC_DECODE_SCRATCH_FLOATS];
// Ticket counters of the split merge (one per request and key/value head).  They have to be
// zero when a launch starts; a launch leaves them zero, and every call clears them anyway.
static __device__ __align__(256) int g_static_decode_tickets[IE_STATIC_DECODE_MAX_TICKETS];

constexpr int MAX_DEVICES = 64;
// In host code the array's name is only a handle; the device address is looked up once per
// device with cudaGetSymbolAddress and kept here.
float* g_static_scratch_ptr[MAX_DEVICES] = {nullptr};
int* g_static_tickets_ptr[MAX_DEVICES] = {nullptr};

int fail(char* msg, int msg_len, int code, const char* text) {
    if (msg != nullptr && msg_len > 0) snprintf(msg, (size_t)msg_len, "%s", text);
    return code;
}
}  // namespace

IE_API long long ie_attention_decode_static_capacity_floats() { return IE_STATIC_DECODE_SCRATCH_FLOATS; }

IE_API int ie_attention_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                      const int* tables, int table_width, const int* cu_q,
                                      const int* ctx_lens, void* out, int num_seqs, int nh, int nkv,
                                      int page_size, int total_pages, float scale, int window,
                                      int num_splits, int* err, void* stream, char* msg, int msg_len) {
    if (msg != nullptr && msg_len > 0) msg[0] = 0;
    if (num_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv != 0 || num_splits < 1)
        return fail(msg, msg_len, (int)cudaErrorInvalidValue, "ie_attention_decode_static: bad head counts or split count");
    long long need = ie_attention_decode_scratch_floats(num_seqs, nkv, num_splits);
    if (need > IE_STATIC_DECODE_SCRATCH_FLOATS || (num_splits > 1 && (long long)num_seqs * nkv > IE_STATIC_DECODE_MAX_TICKETS)) {
        char text[512];
        snprintf(text, sizeof(text),
                 "ie_attention_decode_static: %d requests x %d key/value heads x %d splits need %lld "
                 "floats of scratch, the built-in array holds %lld (and %d ticket counters); use fewer "
                 "splits or smaller batches, or call ie_attention_decode with scratch of your own",
                 num_seqs, nkv, num_splits, need, (long long)IE_STATIC_DECODE_SCRATCH_FLOATS,
                 (int)IE_STATIC_DECODE_MAX_TICKETS);
        return fail(msg, msg_len, IE_STATIC_SCRATCH_TOO_SMALL, text);
    }
    float* scratch = nullptr;
    int* tickets = nullptr;
    if (num_splits > 1) {
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return fail(msg, msg_len, (int)e, "ie_attention_decode_static: cudaGetDevice failed");
        if (dev < 0 || dev >= MAX_DEVICES)
            return fail(msg, msg_len, (int)cudaErrorInvalidDevice, "ie_attention_decode_static: device index out of range");
        if (g_static_scratch_ptr[dev] == nullptr) {
            // First call on this device (it is the current one): ask the runtime where this
            // device's copy of the array lives.  Not an allocation; do it before any capture.
            float* ptr = nullptr;
            e = cudaGetSymbolAddress((void**)&ptr, g_static_decode_scratch);
            if (e != cudaSuccess || ptr == nullptr)
                return fail(msg, msg_len, e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol,
                            "ie_attention_decode_static: cudaGetSymbolAddress failed for the scratch array");
            int* tptr = nullptr;
            e = cudaGetSymbolAddress((void**)&tptr, g_static_decode_tickets);
            if (e != cudaSuccess || tptr == nullptr)
                return fail(msg, msg_len, e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol,
                            "ie_attention_decode_static: cudaGetSymbolAddress failed for the ticket array");
            g_static_scratch_ptr[dev] = ptr;
            g_static_tickets_ptr[dev] = tptr;
        }
        scratch = g_static_scratch_ptr[dev];
        tickets = g_static_tickets_ptr[dev];
        // the tickets must start at zero; the partials need no clearing (written before read)
        e = cudaMemsetAsync(tickets, 0, (size_t)num_seqs * nkv * sizeof(int), (cudaStream_t)stream);
        if (e != cudaSuccess) return fail(msg, msg_len, (int)e, "ie_attention_decode_static: clearing the tickets failed");
    }
    int rc = ie_attention_decode(q, k_cache, v_cache, tables, table_width, cu_q, ctx_lens, out, scratch,
                                 tickets, num_seqs, nh, nkv, page_size, total_pages, scale, window, num_splits,
                                 err, stream);
    if (rc != 0) return fail(msg, msg_len, rc, "ie_attention_decode_static: the kernel launch failed");
    return 0;
}
