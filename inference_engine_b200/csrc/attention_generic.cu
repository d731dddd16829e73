// Paged attention for any mix of prompt portions and decoded tokens, any head size that is
// a multiple of 8 up to 256, any number of heads and groups, 32-bit or bfloat16 cache.
//
// One warp per (token, query head).  The query at absolute position p of its request sees
// the keys at positions lo .. p of the same request (lo = 0, or p - window + 1 with a
// window), found through the request's block table.  Keys are walked in tiles of 32 aligned
// to absolute position 0; scores, the running maximum, the running sum and the weighted sum
// of values are 32-bit, with the same order of operations whatever else is in the step: a
// position's result depends on its own request's data only.  This is the attention of the
// engine's 32-bit path, and the fallback of the bfloat16 path for head sizes its
// tensor-core kernels do not take.  Counterparts in the reference:
// engine/kernels/paged_attention.py:44-87 (decode rows) and the gather + SDPA path
// engine/model/layers.py:215-225 (prompt portions).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_ACC = 8;  // head_dim <= 256

__device__ __forceinline__ float dot_row(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 4) {
        float4 kv = *reinterpret_cast<const float4*>(k + d);
        s = fmaf(q[d], kv.x, s); s = fmaf(q[d + 1], kv.y, s);
        s = fmaf(q[d + 2], kv.z, s); s = fmaf(q[d + 3], kv.w, s);
    }
    return s;
}
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k, int hd) {
    float s = 0.f;
    for (int d = 0; d < hd; d += 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(k + d);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h2[i]);
            s = fmaf(q[d + 2 * i], f.x, s);
            s = fmaf(q[d + 2 * i + 1], f.y, s);
        }
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_tables,
                               int table_width, const int* __restrict__ seq_of_token,
                               const int* __restrict__ positions, T* __restrict__ out,
                               int nh, int nkv, int hd, int page_size, int total_pages,
                               float scale, int window, int* err) {
    extern __shared__ float q_smem[];  // [WARPS][hd]
    ie_pdl_trigger();
    ie_pdl_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int head = blockIdx.x * WARPS + warp;
    int token = blockIdx.y;
    if (head >= nh) return;  // whole warp leaves together; no block-wide barrier below
    int kvh = head / (nh / nkv);
    int seq = seq_of_token[token], pos = positions[token];
    const int* table = block_tables + (size_t)seq * table_width;
    float* qs = q_smem + warp * hd;
    const T* qrow = q + ((size_t)token * nh + head) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = ie_load(qrow + d);
    __syncwarp();

    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) acc[i] = 0.f;
    int nacc = (hd + 31) / 32;

    for (int t0 = (lo / 32) * 32; t0 <= pos; t0 += 32) {
        int kpos = t0 + lane;
        bool valid = kpos >= lo && kpos <= pos;
        long long row = -1;
        float s = -INFINITY;
        if (valid) {
            int page = table[kpos / page_size];
            if (page < 0 || page >= total_pages) {
                ie_report(err, page < 0 ? IE_ERR_TABLE : IE_ERR_PAGE, page, token);
                valid = false;
            } else {
                row = ((long long)page * nkv + kvh) * page_size + (kpos % page_size);
                s = dot_row(qs, k_cache + row * hd, hd) * scale;
            }
        }
        float m_new = fmaxf(m, warp_max(s));
        float p = valid ? expf(s - m_new) : 0.f;
        float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_ACC; ++i) acc[i] *= alpha;
        int count = min(32, pos - t0 + 1);
        for (int j = 0; j < count; ++j) {
            float pj = __shfl_sync(0xffffffffu, p, j);
            long long rj = __shfl_sync(0xffffffffu, row, j);
            if (rj < 0) continue;  // uniform across the warp
            const T* vrow = v_cache + rj * hd;
#pragma unroll
            for (int i = 0; i < MAX_ACC; ++i) {
                int d = lane + 32 * i;
                if (i < nacc && d < hd) acc[i] = fmaf(pj, ie_load(vrow + d), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + ((size_t)token * nh + head) * hd;
    float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) {
        int d = lane + 32 * i;
        if (i < nacc && d < hd) ie_store(orow + d, acc[i] * inv);
    }
}
}  // namespace

IE_API int ie_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                      int dtype, const int* block_tables, int table_width,
                                      const int* seq_of_token, const int* positions, void* out,
                                      int num_tokens, int nh, int nkv, int hd, int page_size,
                                      int total_pages, float scale, int window, int* err,
                                      void* stream) {
    if (num_tokens <= 0) return 0;
    if (hd % 8 != 0 || hd > 32 * MAX_ACC || nkv <= 0 || nh % nkv != 0) return (int)cudaErrorInvalidValue;
    dim3 grid((nh + WARPS - 1) / WARPS, num_tokens);
    size_t smem = (size_t)WARPS * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        paged_attention_generic_kernel<<<grid, WARPS * 32, smem, s>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
            block_tables, table_width, seq_of_token, positions, (__nv_bfloat16*)out,
            nh, nkv, hd, page_size, total_pages, scale, window, err);
    else
        paged_attention_generic_kernel<<<grid, WARPS * 32, smem, s>>>(
            (const float*)q, (const float*)k_cache, (const float*)v_cache,
            block_tables, table_width, seq_of_token, positions, (float*)out,
            nh, nkv, hd, page_size, total_pages, scale, window, err);
    return IE_LAUNCH_CHECK();
}
