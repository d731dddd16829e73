// Embedding gather, RMS norm with fused residual add, rotary encoding fused with the write
// of keys and values into cache pages, and SiLU-and-multiply.  All arithmetic is 32-bit;
// results are rounded once to the output's dtype.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Embedding: out[n, :] = float(table[ids[n], :])          (engine/model/llama.py:25,61)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, int* err) {
    int row = blockIdx.x;
    int id = ids[row];
    bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) ie_report(err, IE_ERR_TOKEN_ID, id, row);
    const T* src = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? ie_load(src + i) : 0.f;
}

IE_API int ie_embedding(const void* table, int table_dtype, const int* ids, float* out,
                        int num_tokens, int hidden, int vocab, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_dtype == IE_BF16)
        embedding_kernel<<<num_tokens, threads, 0, s>>>((const __nv_bfloat16*)table, ids, out, hidden, vocab, err);
    else
        embedding_kernel<<<num_tokens, threads, 0, s>>>((const float*)table, ids, out, hidden, vocab, err);
    return IE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// RMS norm with residual add                               (engine/model/layers.py:41-43)
//   rows == nullptr:  h[r] += delta[r] (if delta);  out[r] = w * (h[r] * rsqrt(mean(h[r]^2) + eps))
//   rows != nullptr:  x = h[rows[r]] + delta[rows[r]];  out[r] = norm(x); h is not modified.
// One block per row.  The sum of squares of a row is added in an order that depends only on
// the row's width and the block size, never on the other rows of the step.
// ---------------------------------------------------------------------------------------------
template <typename OutT, int THREADS>
__global__ void rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta,
                               const float* __restrict__ weight, float eps, OutT* __restrict__ out,
                               const int* __restrict__ rows, int hidden) {
    __shared__ float partial[THREADS / 32];
    __shared__ float inv_rms;
    int r = blockIdx.x;
    size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float* hrow = h + src;
    const float* drow = delta ? delta + src : nullptr;
    bool write_back = (rows == nullptr) && (delta != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += THREADS) {
        float x = hrow[i];
        if (drow) x += drow[i];
        if (write_back) hrow[i] = x;
        ss += x * x;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) total += partial[w];
        inv_rms = 1.0f / sqrtf(total / (float)hidden + eps);
    }
    __syncthreads();
    float scale = inv_rms;
    OutT* orow = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += THREADS) {
        float x = hrow[i];
        if (drow && !write_back) x += drow[i];
        ie_store(orow + i, weight[i] * (x * scale));
    }
}

IE_API int ie_rmsnorm(float* h, const float* delta, const float* weight, float eps, void* out,
                      int out_dtype, const int* rows, int num_rows, int hidden, void* stream) {
    if (num_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16)
        rmsnorm_kernel<__nv_bfloat16, 256><<<num_rows, 256, 0, s>>>(h, delta, weight, eps, (__nv_bfloat16*)out, rows, hidden);
    else
        rmsnorm_kernel<float, 256><<<num_rows, 256, 0, s>>>(h, delta, weight, eps, (float*)out, rows, hidden);
    return IE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Rotary encoding + cache write            (engine/model/layers.py:82-93, paged_cache.py:42-45)
//   qkv  : [N, (nh + 2 nkv) * hd] 32-bit, the fused projection's output
//   table: [P, 2, rd/2] cos and sin of position * inv_freq (32-bit); rd = rotary_dim <= hd
//   q_out: [N, nh * hd]; k_cache, v_cache: [pages, nkv, page_size, hd]
//   out[d] = x[d] cos[d] - x[d + rd/2] sin[d]          for d <  rd/2
//          = x[d] cos[d - rd/2] + x[d - rd/2] sin[d - rd/2]   for rd/2 <= d < rd
//          = x[d]                                        for d >= rd  (and all of v)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ table, int rotary_dim, int table_rows,
                                     T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, const int* __restrict__ slot_mapping,
                                     int nh, int nkv, int hd, int page_size, int total_pages, int* err) {
    int n = blockIdx.x;
    int heads = nh + 2 * nkv;
    int half = rotary_dim / 2;
    int pos = positions[n];
    bool rotate = table != nullptr && rotary_dim > 0;
    if (rotate && (pos < 0 || pos >= table_rows)) {
        if (threadIdx.x == 0) ie_report(err, IE_ERR_POSITION, pos, n);
        rotate = false;
    }
    const float* cs = rotate ? table + (size_t)pos * rotary_dim : nullptr;  // cos[half] then sin[half]
    const float* x = qkv + (size_t)n * heads * hd;
    int slot = slot_mapping ? slot_mapping[n] : -1;
    int page = slot >= 0 ? slot / page_size : -1, off = slot >= 0 ? slot % page_size : 0;
    bool write_kv = slot_mapping != nullptr;
    if (write_kv && (page < 0 || page >= total_pages)) {
        if (threadIdx.x == 0) ie_report(err, IE_ERR_PAGE, slot, n);
        write_kv = false;
    }
    int limit = write_kv ? heads * hd : nh * hd;
    for (int e = threadIdx.x; e < limit; e += blockDim.x) {
        int head = e / hd, d = e - head * hd;
        float v = x[e];
        if (rotate && head < nh + nkv && d < rotary_dim) {
            if (d < half) v = v * cs[d] - x[e + half] * cs[half + d];
            else          v = v * cs[d - half] + x[e - half] * cs[d];
        }
        if (head < nh) {
            ie_store(q_out + (size_t)n * nh * hd + e, v);
        } else if (head < nh + nkv) {
            int kh = head - nh;
            ie_store(k_cache + (((size_t)page * nkv + kh) * page_size + off) * hd + d, v);
        } else {
            int kh = head - nh - nkv;
            ie_store(v_cache + (((size_t)page * nkv + kh) * page_size + off) * hd + d, v);
        }
    }
}

IE_API int ie_rope_kv_write(const float* qkv, const int* positions, const float* table,
                            int rotary_dim, int table_rows, void* q_out, void* k_cache,
                            void* v_cache, int dtype, const int* slot_mapping, int num_tokens,
                            int nh, int nkv, int hd, int page_size, int total_pages, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = (nh + 2 * nkv) * hd >= 1024 ? 256 : 128;
    if (dtype == IE_BF16)
        rope_kv_write_kernel<<<num_tokens, threads, 0, s>>>(qkv, positions, table, rotary_dim, table_rows,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping,
            nh, nkv, hd, page_size, total_pages, err);
    else
        rope_kv_write_kernel<<<num_tokens, threads, 0, s>>>(qkv, positions, table, rotary_dim, table_rows,
            (float*)q_out, (float*)k_cache, (float*)v_cache, slot_mapping,
            nh, nkv, hd, page_size, total_pages, err);
    return IE_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// SiLU-and-multiply: out[n, i] = silu(gu[n, i]) * gu[n, I + i], silu(g) = g / (1 + exp(-g))
// (engine/model/layers.py:277-281; engine/kernels/fused.py:82-90 evaluates it in 32-bit too)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter,
                                size_t total) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        size_t row = idx / inter;
        int i = (int)(idx - row * inter);
        float g = ie_load(gate_up + row * 2 * inter + i);
        float u = ie_load(gate_up + row * 2 * inter + inter + i);
        ie_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

IE_API int ie_silu_mul(const void* gate_up, void* out, int dtype, int num_rows, int inter,
                       void* stream) {
    size_t total = (size_t)num_rows * inter;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = 256;
    size_t want = (total + threads - 1) / threads;
    int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (dtype == IE_BF16)
        silu_mul_kernel<<<blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else
        silu_mul_kernel<<<blocks, threads, 0, s>>>((const float*)gate_up, (float*)out, inter, total);
    return IE_LAUNCH_CHECK();
}
