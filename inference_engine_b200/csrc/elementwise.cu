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
    ie_pdl_trigger();
    ie_pdl_wait();
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
        return ie_launch(embedding_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, s,
                         (const __nv_bfloat16*)table, ids, out, hidden, vocab, err);
    return ie_launch(embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, s, (const float*)table, ids,
                     out, hidden, vocab, err);
}

// ---------------------------------------------------------------------------------------------
// RMS norm with residual add                               (engine/model/layers.py:41-43)
//   rows == nullptr:  h[r] += delta[r] (if delta);  out[r] = w * (h[r] * rsqrt(mean(h[r]^2) + eps))
//   rows != nullptr:  x = h[rows[r]] + delta[rows[r]];  out[r] = norm(x); h is not modified.
// One block per row.  The sum of squares of a row is added in an order that depends only on
// the row's width and the block size, never on the other rows of the step.
// ---------------------------------------------------------------------------------------------
template <typename OutT, int THREADS>
__global__ void rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int num_partials,
                               size_t partial_stride, const float* __restrict__ weight, float eps,
                               OutT* __restrict__ out, const int* __restrict__ rows, int hidden) {
    __shared__ float partial[THREADS / 32];
    __shared__ float inv_rms;
    ie_pdl_trigger();
    ie_pdl_wait();
    int r = blockIdx.x;
    size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float* hrow = h + src;
    const float* drow = delta ? delta + src : nullptr;
    bool write_back = (rows == nullptr) && (delta != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += THREADS) {
        float x = hrow[i];
        if (drow) for (int p = 0; p < num_partials; ++p) x += drow[p * partial_stride + i];
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
        if (drow && !write_back) for (int p = 0; p < num_partials; ++p) x += drow[p * partial_stride + i];
        ie_store(orow + i, weight[i] * (x * scale));
    }
}

__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
    *reinterpret_cast<uint2*>(p) = u;
}

// The same result for rows whose width is a multiple of 4 and at most THREADS * 4 * VPT: every
// thread keeps its part of the row in registers, so the row is read once and all loads are in
// flight together (a decode step's few rows are bound by latency, not bandwidth).  The order
// in which a row's squares are added depends only on the row's width.
// PCH: how many parts of `delta` are loaded at a time (1 when it is a single array: a prefill
// step's thousands of rows want the registers for occupancy instead).
template <typename OutT, int THREADS, int VPT, int PCH>
__global__ void __launch_bounds__(THREADS)
rmsnorm_vec_kernel(float* __restrict__ h, const float* __restrict__ delta, int num_partials,
                   size_t partial_stride, const float* __restrict__ weight, float eps,
                   OutT* __restrict__ out, const int* __restrict__ rows, int hidden) {
    __shared__ float partial[THREADS / 32];
    __shared__ float inv_rms;
    ie_pdl_trigger();
    int r = blockIdx.x;
    float4 x[VPT], wt[VPT];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {  // the norm's weights: nobody writes them, no need to wait
        int i = (v * THREADS + threadIdx.x) * 4;
        wt[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < hidden) wt[v] = *reinterpret_cast<const float4*>(weight + i);
    }
    ie_pdl_wait();
    size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    bool write_back = (rows == nullptr) && (delta != nullptr);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        int i = (v * THREADS + threadIdx.x) * 4;
        x[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < hidden) x[v] = *reinterpret_cast<const float4*>(h + src + i);
    }
    if (delta) {
        // The parts are added in order, but their loads are issued several parts at a time:
        // one part after the other, every part would cost a trip to memory.
        for (int p0 = 0; p0 < num_partials; p0 += PCH) {
            float4 d[PCH][VPT];
#pragma unroll
            for (int j = 0; j < PCH; ++j)
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    int i = (v * THREADS + threadIdx.x) * 4;
                    d[j][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p0 + j < num_partials && i < hidden)
                        d[j][v] = *reinterpret_cast<const float4*>(delta + (p0 + j) * partial_stride + src + i);
                }
#pragma unroll
            for (int j = 0; j < PCH; ++j)
                if (p0 + j < num_partials) {
#pragma unroll
                    for (int v = 0; v < VPT; ++v) {
                        x[v].x += d[j][v].x; x[v].y += d[j][v].y; x[v].z += d[j][v].z; x[v].w += d[j][v].w;
                    }
                }
        }
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        int i = (v * THREADS + threadIdx.x) * 4;
        if (i < hidden) {
            if (write_back) *reinterpret_cast<float4*>(h + src + i) = x[v];
            ss += x[v].x * x[v].x; ss += x[v].y * x[v].y; ss += x[v].z * x[v].z; ss += x[v].w * x[v].w;
        }
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
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        int i = (v * THREADS + threadIdx.x) * 4;
        if (i < hidden) {
            float4 w = wt[v];
            float4 o = make_float4(w.x * (x[v].x * scale), w.y * (x[v].y * scale),
                                   w.z * (x[v].z * scale), w.w * (x[v].w * scale));
            store4(out + (size_t)r * hidden + i, o);
        }
    }
}

template <typename OutT>
static int launch_rmsnorm(float* h, const float* delta, int num_partials, size_t partial_stride,
                          const float* weight, float eps, OutT* out, const int* rows, int num_rows,
                          int hidden, cudaStream_t s) {
#define IE_NORM_ARGS s, h, delta, num_partials, partial_stride, weight, eps, out, rows, hidden
    bool multi = delta != nullptr && num_partials > 1;
    if (hidden % 4 == 0 && hidden <= 128 * 4 * 2)
        return multi ? ie_launch(rmsnorm_vec_kernel<OutT, 128, 2, 8>, dim3(num_rows), dim3(128), 0, IE_NORM_ARGS)
                     : ie_launch(rmsnorm_vec_kernel<OutT, 128, 2, 1>, dim3(num_rows), dim3(128), 0, IE_NORM_ARGS);
    if (hidden % 4 == 0 && hidden <= 256 * 4 * 2)
        return multi ? ie_launch(rmsnorm_vec_kernel<OutT, 256, 2, 8>, dim3(num_rows), dim3(256), 0, IE_NORM_ARGS)
                     : ie_launch(rmsnorm_vec_kernel<OutT, 256, 2, 1>, dim3(num_rows), dim3(256), 0, IE_NORM_ARGS);
    if (hidden % 4 == 0 && hidden <= 512 * 4 * 4)
        return multi ? ie_launch(rmsnorm_vec_kernel<OutT, 512, 4, 4>, dim3(num_rows), dim3(512), 0, IE_NORM_ARGS)
                     : ie_launch(rmsnorm_vec_kernel<OutT, 512, 4, 1>, dim3(num_rows), dim3(512), 0, IE_NORM_ARGS);
#undef IE_NORM_ARGS
    return ie_launch(rmsnorm_kernel<OutT, 256>, dim3(num_rows), dim3(256), 0, s, h, delta, num_partials, partial_stride, weight, eps, out, rows, hidden);
}

// `delta` may be the sum of `num_partials` arrays `partial_stride` floats apart (the parts of
// a matrix product that was split along its inner dimension); they are added in order.
IE_API int ie_rmsnorm(float* h, const float* delta, int num_partials, long long partial_stride,
                      const float* weight, float eps, void* out, int out_dtype, const int* rows,
                      int num_rows, int hidden, void* stream) {
    if (num_rows <= 0) return 0;
    if (delta != nullptr && num_partials < 1) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == IE_BF16)
        return launch_rmsnorm(h, delta, num_partials, (size_t)partial_stride, weight, eps, (__nv_bfloat16*)out, rows, num_rows, hidden, s);
    return launch_rmsnorm(h, delta, num_partials, (size_t)partial_stride, weight, eps, (float*)out, rows, num_rows, hidden, s);
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
// `qkv` may be the sum of `num_partials` arrays, added in order (see the vector kernel below).
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, int num_partials, size_t partial_stride,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ table, int rotary_dim, int table_rows,
                                     T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, const int* __restrict__ slot_mapping,
                                     int nh, int nkv, int hd, int page_size, int total_pages, int* err) {
    ie_pdl_trigger();
    ie_pdl_wait();
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
    auto value = [&](int e) {
        float sum = x[e];
        for (int p = 1; p < num_partials; ++p) sum += x[(size_t)p * partial_stride + e];
        return sum;
    };
    for (int e = threadIdx.x; e < limit; e += blockDim.x) {
        int head = e / hd, d = e - head * hd;
        float v = value(e);
        if (rotate && head < nh + nkv && d < rotary_dim) {
            if (d < half) v = v * cs[d] - value(e + half) * cs[half + d];
            else          v = v * cs[d - half] + value(e - half) * cs[d];
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

// The same for rotary_dim == head_dim (or no rotation) and head_dim a multiple of 8: a thread
// takes four neighbouring dims of a head's low half and the four that pair with them in the
// high half, so all its loads are independent 16-byte loads.  `qkv` may be the sum of
// `num_partials` arrays (the parts of a matrix product split along its inner dimension).
template <typename T, int PCH>
__global__ void __launch_bounds__(128)
rope_kv_write_vec_kernel(const float* __restrict__ qkv, int num_partials, size_t partial_stride,
                         const int* __restrict__ positions, const float* __restrict__ table,
                         int table_rows, T* __restrict__ q_out, T* __restrict__ k_cache,
                         T* __restrict__ v_cache, const int* __restrict__ slot_mapping,
                         int nh, int nkv, int hd, int page_size, int total_pages, int* err) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int n = blockIdx.x;
    int half = hd / 2, per_head = hd / 8;
    int heads = slot_mapping ? nh + 2 * nkv : nh;
    int item = blockIdx.y * blockDim.x + threadIdx.x;
    if (item >= heads * per_head) return;
    int head = item / per_head, d = (item - head * per_head) * 4;
    int pos = positions[n];
    bool rotate = table != nullptr && head < nh + nkv;
    if (rotate && (pos < 0 || pos >= table_rows)) {
        ie_report(err, IE_ERR_POSITION, pos, n);
        rotate = false;
    }
    size_t base = (size_t)n * (nh + 2 * nkv) * hd + (size_t)head * hd + d;
    float4 lo = *reinterpret_cast<const float4*>(qkv + base);
    float4 hi = *reinterpret_cast<const float4*>(qkv + base + half);
    // further parts: added in order, loaded PCH at a time (one after the other, every part
    // would cost a trip to memory)
    for (int p0 = 1; p0 < num_partials; p0 += PCH) {
        float4 a[PCH], b[PCH];
#pragma unroll
        for (int j = 0; j < PCH; ++j) {
            a[j] = b[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p0 + j < num_partials) {
                a[j] = *reinterpret_cast<const float4*>(qkv + (p0 + j) * partial_stride + base);
                b[j] = *reinterpret_cast<const float4*>(qkv + (p0 + j) * partial_stride + base + half);
            }
        }
#pragma unroll
        for (int j = 0; j < PCH; ++j)
            if (p0 + j < num_partials) {
                lo.x += a[j].x; lo.y += a[j].y; lo.z += a[j].z; lo.w += a[j].w;
                hi.x += b[j].x; hi.y += b[j].y; hi.z += b[j].z; hi.w += b[j].w;
            }
    }
    if (rotate) {
        float4 c = *reinterpret_cast<const float4*>(table + (size_t)pos * hd + d);
        float4 sn = *reinterpret_cast<const float4*>(table + (size_t)pos * hd + half + d);
        float4 olo = make_float4(lo.x * c.x - hi.x * sn.x, lo.y * c.y - hi.y * sn.y,
                                 lo.z * c.z - hi.z * sn.z, lo.w * c.w - hi.w * sn.w);
        float4 ohi = make_float4(hi.x * c.x + lo.x * sn.x, hi.y * c.y + lo.y * sn.y,
                                 hi.z * c.z + lo.z * sn.z, hi.w * c.w + lo.w * sn.w);
        lo = olo; hi = ohi;
    }
    T* dst;
    if (head < nh) {
        dst = q_out + (size_t)n * nh * hd + (size_t)head * hd + d;
    } else {
        int slot = slot_mapping[n];
        int page = slot >= 0 ? slot / page_size : -1, off = slot >= 0 ? slot % page_size : 0;
        if (page < 0 || page >= total_pages) {
            if (d == 0) ie_report(err, IE_ERR_PAGE, slot, n);
            return;
        }
        bool is_k = head < nh + nkv;
        int kh = is_k ? head - nh : head - nh - nkv;
        dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kh) * page_size + off) * hd + d;
    }
    store4(dst, lo);
    store4(dst + half, hi);
}

template <typename T>
static int launch_rope(const float* qkv, int num_partials, size_t partial_stride, const int* positions,
                       const float* table, int rotary_dim, int table_rows, T* q_out, T* k_cache,
                       T* v_cache, const int* slot_mapping, int num_tokens, int nh, int nkv, int hd,
                       int page_size, int total_pages, int* err, cudaStream_t s) {
    bool rotates = table != nullptr && rotary_dim > 0;
    if (hd % 8 == 0 && (!rotates || rotary_dim == hd)) {
        int heads = slot_mapping ? nh + 2 * nkv : nh;
        dim3 grid(num_tokens, (heads * (hd / 8) + 127) / 128);
        if (num_partials > 1)
            return ie_launch(rope_kv_write_vec_kernel<T, 8>, grid, dim3(128), 0, s, qkv, num_partials, partial_stride,
                             positions, rotates ? table : (const float*)nullptr, table_rows, q_out, k_cache,
                             v_cache, slot_mapping, nh, nkv, hd, page_size, total_pages, err);
        return ie_launch(rope_kv_write_vec_kernel<T, 1>, grid, dim3(128), 0, s, qkv, num_partials, partial_stride,
                         positions, rotates ? table : (const float*)nullptr, table_rows, q_out, k_cache, v_cache,
                         slot_mapping, nh, nkv, hd, page_size, total_pages, err);
    } else {
        int threads = (nh + 2 * nkv) * hd >= 1024 ? 256 : 128;
        return ie_launch(rope_kv_write_kernel<T>, dim3(num_tokens), dim3(threads), 0, s, qkv, num_partials,
                         partial_stride, positions, table,
                         rotary_dim, table_rows, q_out, k_cache, v_cache, slot_mapping, nh, nkv, hd, page_size,
                         total_pages, err);
    }
}

// 1: kernels are launched with the programmatic-serialization attribute (the default); 0: plain launches.
IE_API void ie_set_pdl(int enabled) { ie_pdl_enabled() = enabled ? 1 : 0; }

IE_API int ie_rope_kv_write(const float* qkv, int num_partials, long long partial_stride,
                            const int* positions, const float* table, int rotary_dim, int table_rows,
                            void* q_out, void* k_cache, void* v_cache, int dtype,
                            const int* slot_mapping, int num_tokens, int nh, int nkv, int hd,
                            int page_size, int total_pages, int* err, void* stream) {
    if (num_tokens <= 0) return 0;
    if (num_partials < 1) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == IE_BF16)
        return launch_rope(qkv, num_partials, (size_t)partial_stride, positions, table, rotary_dim, table_rows,
                           (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                           slot_mapping, num_tokens, nh, nkv, hd, page_size, total_pages, err, s);
    return launch_rope(qkv, num_partials, (size_t)partial_stride, positions, table, rotary_dim, table_rows,
                       (float*)q_out, (float*)k_cache, (float*)v_cache,
                       slot_mapping, num_tokens, nh, nkv, hd, page_size, total_pages, err, s);
}

// ---------------------------------------------------------------------------------------------
// SiLU-and-multiply: out[n, i] = silu(gu[n, i]) * gu[n, I + i], silu(g) = g / (1 + exp(-g))
// (engine/model/layers.py:277-281; engine/kernels/fused.py:82-90 evaluates it in 32-bit too)
// ---------------------------------------------------------------------------------------------
// Where gate i and up i sit in a row of `gate_up`: the gates in the first half and the ups in the
// second (il == 0), or alternating in blocks of `il` values (il gates, their il ups, the next
// il gates, ...), the layout in which a matrix-product kernel finds a gate and its up in one tile.
__device__ __forceinline__ int gate_column(int i, int il) { return il ? (i / il) * 2 * il + i % il : i; }

template <typename T, typename InT>
__global__ void silu_mul_kernel(const InT* __restrict__ gate_up, int num_partials, size_t partial_stride,
                                T* __restrict__ out, int inter, size_t total, int il) {
    ie_pdl_trigger();
    ie_pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        size_t row = idx / inter;
        int i = (int)(idx - row * inter);
        int gc = gate_column(i, il), uc = gc + (il ? il : inter);
        float g = 0.f, u = 0.f;
        for (int p = 0; p < num_partials; ++p) {
            g += ie_load(gate_up + p * partial_stride + row * 2 * inter + gc);
            u += ie_load(gate_up + p * partial_stride + row * 2 * inter + uc);
        }
        ie_store(out + idx, g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 in and out, one array, width a multiple of 8: 16-byte loads and stores, two of each
// per thread in flight (a prefill step moves a hundred megabytes through this kernel), the row
// from the grid (no division), and the special-function unit's reciprocal and exponential: their
// error, a few units in the last place of a 32-bit value, vanishes in the rounding to bfloat16.
constexpr int SILU_VECS = 2;  // 8-value vectors per thread
__global__ void __launch_bounds__(256)
silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter, int il) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int per_row = inter / 8;
    size_t row = blockIdx.y;
    const __nv_bfloat16* g_row = gate_up + row * 2 * inter;
    int v0 = blockIdx.x * (256 * SILU_VECS) + threadIdx.x;
    uint4 graw[SILU_VECS], uraw[SILU_VECS];
#pragma unroll
    for (int k = 0; k < SILU_VECS; ++k) {
        int v = v0 + k * 256;
        if (v < per_row) {  // (il is a multiple of 8: a vector never straddles a block)
            int gc = gate_column(v * 8, il);
            graw[k] = *reinterpret_cast<const uint4*>(g_row + gc);
            uraw[k] = *reinterpret_cast<const uint4*>(g_row + gc + (il ? il : inter));
        }
    }
#pragma unroll
    for (int k = 0; k < SILU_VECS; ++k) {
        int v = v0 + k * 256;
        if (v >= per_row) continue;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw[k]);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw[k]);
        uint4 oraw;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 gf = __bfloat1622float2(g2[j]), uf = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x,
                                          __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y);
        }
        *reinterpret_cast<uint4*>(out + row * inter + (size_t)v * 8) = oraw;
    }
}

// `gate_up` has the output's dtype, or is 32-bit (in_dtype), possibly the sum of `num_partials`
// arrays `partial_stride` elements apart.  `interleave`: 0, or the size of the blocks in which
// gates and ups alternate (a multiple of 8 that divides `inter`).
IE_API int ie_silu_mul(const void* gate_up, int in_dtype, int num_partials, long long partial_stride,
                       void* out, int dtype, int num_rows, int inter, int interleave, void* stream) {
    size_t total = (size_t)num_rows * inter;
    if (total == 0) return 0;
    if (num_partials < 1 || (in_dtype != dtype && in_dtype != IE_F32)) return (int)cudaErrorInvalidValue;
    if (interleave < 0 || (interleave > 0 && (interleave % 8 != 0 || inter % interleave != 0)))
        return (int)cudaErrorInvalidValue;
    int il = interleave;
    cudaStream_t s = (cudaStream_t)stream;
    int threads = 256;
    size_t want = (total + threads - 1) / threads;
    int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    size_t ps = (size_t)partial_stride;
    if (dtype == IE_BF16 && in_dtype == IE_BF16 && num_partials == 1 && inter % 8 == 0 && num_rows <= 65535) {
        int per_block = 256 * SILU_VECS;
        return ie_launch(silu_mul_bf16x8_kernel, dim3((unsigned)((inter / 8 + per_block - 1) / per_block), (unsigned)num_rows),
                         dim3(256), 0, s, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, il);
    }
    if (dtype == IE_BF16 && in_dtype == IE_BF16)
        return ie_launch(silu_mul_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, s,
                         (const __nv_bfloat16*)gate_up, num_partials, ps, (__nv_bfloat16*)out, inter, total, il);
    if (dtype == IE_BF16)
        return ie_launch(silu_mul_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(threads), 0, s,
                         (const float*)gate_up, num_partials, ps, (__nv_bfloat16*)out, inter, total, il);
    return ie_launch(silu_mul_kernel<float, float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up,
                     num_partials, ps, (float*)out, inter, total, il);
}
