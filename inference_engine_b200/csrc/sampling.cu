// Next-token choice on the device: greedy argmax and temperature sampling, with optional
// top-k / top-p / min-p cut-offs and a repetition penalty.  A row of logits is shared among the
// eight blocks of a thread-block cluster (a vocabulary of a hundred thousand is too much for one
// SM: 70 us for a plain draw, 230 us with top-k and top-p); every block works on its slice and the
// blocks exchange maxima, sums and histograms through each other's shared memory (one cluster
// barrier per exchange), always added in the order of the blocks.  The number of blocks per row is
// fixed, so a row's arithmetic does not depend on how many rows the step has.
//
// Order of operations as in engine/runtime/sampler.py:10-45: repetition penalty, then (not
// greedy) divide by the temperature, top-k, top-p, min-p, softmax, draw.  The draw is a
// Gumbel-max over the kept tokens: argmax_i (z_i + g_i) with g_i = -log(-log(u_i)) picks i
// with probability softmax(z)_i, so no normalisation pass is needed.  u_i comes from the
// counter-based Philox4x32-10 generator keyed by the request's seed and indexed by (how many
// tokens the request has produced, i): a request's tokens do not depend on which other
// requests share the step or on its row in the batch (the property tests/test_engine.py:132-136
// of the reference asks for; the reference gets it from one torch.Generator per request).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        unsigned hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
        unsigned hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
        c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
        k.x += 0x9E3779B9u; k.y += 0xBB67AE85u;
    }
    return c;
}

// Token i of a row takes word i % 4 of the generator's call i / 4 (counter: call, draw; key: seed).
__device__ __forceinline__ uint4 random_words(unsigned long long seed, unsigned long long draw, unsigned call) {
    return philox4x32_10(make_uint4(call, (unsigned)draw, (unsigned)(draw >> 32), 0u),
                         make_uint2((unsigned)seed, (unsigned)(seed >> 32)));
}
// 23 random bits plus a half: every value is exact in 32-bit and strictly inside (0, 1)
__device__ __forceinline__ float uniform_of(unsigned word) {
    return ((float)(word >> 9) + 0.5f) * (1.0f / 8388608.0f);
}

struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ Best block_best(Best b, Best* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = b;
    __syncthreads();
    Best r = scratch[0];
    for (int w = 1; w < THREADS / 32; ++w) r = better(r, scratch[w]);
    return r;
}
__device__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < THREADS / 32; ++w) r += scratch[w];
    return r;
}

// ---- exchange among the blocks of a row's cluster ----------------------------------------------
constexpr int CLUSTER = 8;  // blocks per row
// A slot per block of the cluster, in every block's shared memory, twice: an exchange writes the
// set the one before it did not use, so a block may start the next exchange while another still
// reads this one (an exchange's barrier is passed only when every block is done reading the
// exchange before it).
struct Exchange {
    Best best[2][CLUSTER];
    float sum[2][CLUSTER];
    float hist[2][CLUSTER][256];
    float total[256];  // the blocks' histograms added up
    int turn;          // which set the next exchange writes
};
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `local` (in this block's shared memory) in block `rank`'s.
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
    unsigned a = (unsigned)__cvta_generic_to_shared(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void peer_store(const float* local, unsigned rank, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer_address(local, rank)), "f"(v) : "memory");
}
__device__ __forceinline__ void peer_store(const int* local, unsigned rank, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(peer_address(local, rank)), "r"(v) : "memory");
}
// The best of all blocks' `b` (every thread of every block gets it).
__device__ Best cluster_best(Best b, Best* scratch, Exchange* ex) {
    b = block_best(b, scratch);
    int turn = ex->turn;
    unsigned me = cluster_rank();
    if (threadIdx.x < CLUSTER) {
        peer_store(&ex->best[turn][me].v, threadIdx.x, b.v);
        peer_store(&ex->best[turn][me].i, threadIdx.x, b.i);
    }
    cluster_sync();
    Best r = ex->best[turn][0];
    for (int k = 1; k < CLUSTER; ++k) r = better(r, ex->best[turn][k]);
    __syncthreads();
    if (threadIdx.x == 0) ex->turn = turn ^ 1;
    __syncthreads();
    return r;
}
// The sum of all blocks' `v`, added in the order of the blocks.
__device__ float cluster_sum(float v, float* scratch, Exchange* ex) {
    v = block_sum(v, scratch);
    int turn = ex->turn;
    unsigned me = cluster_rank();
    if (threadIdx.x < CLUSTER) peer_store(&ex->sum[turn][me], threadIdx.x, v);
    cluster_sync();
    float r = 0.f;
    for (int k = 0; k < CLUSTER; ++k) r += ex->sum[turn][k];
    __syncthreads();
    if (threadIdx.x == 0) ex->turn = turn ^ 1;
    __syncthreads();
    return r;
}

// Monotone map of a float onto unsigned ints (larger float -> larger key).
__device__ __forceinline__ unsigned float_key(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Penalised, temperature-scaled logit i of the row (engine/runtime/sampler.py:48-56).
__device__ __forceinline__ float scaled_logit(const float* row, int i, float inv_temp, float penalty,
                                              const unsigned* seen_bits) {
    float z = row[i];
    if (seen_bits && (seen_bits[i >> 5] >> (i & 31) & 1u)) z = z > 0.f ? z / penalty : z * penalty;
    return z * inv_temp;
}

// Calls f(z, i) for the penalised, temperature-scaled logit of every token i of the row that is
// this thread's.  A block walks a row of a hundred thousand logits alone, so what counts is how
// many loads a thread has in flight: 16-byte loads, two per turn, when the row allows them (width
// a multiple of 4), single ones otherwise.
// This block's tokens are lo .. hi - 1 (lo a multiple of 4).
template <typename F>
__device__ __forceinline__ void for_each_scaled(const float* row, int lo, int hi, int vocab, float inv_temp,
                                                float penalty, const unsigned* seen_bits, F&& f) {
    auto scaled = [&](float z, int i) {
        if (seen_bits && (seen_bits[i >> 5] >> (i & 31) & 1u)) z = z > 0.f ? z / penalty : z * penalty;
        return z * inv_temp;
    };
    if ((vocab & 3) == 0 && (reinterpret_cast<size_t>(row) & 15) == 0) {  // (then hi is a multiple of 4 too)
        const float4* row4 = reinterpret_cast<const float4*>(row);
        int n4 = hi >> 2;
        for (int j = (lo >> 2) + threadIdx.x; j < n4; j += 2 * THREADS) {
            int j2 = j + THREADS;
            float4 a = row4[j];
            float4 b = j2 < n4 ? row4[j2] : make_float4(0.f, 0.f, 0.f, 0.f);
            f(scaled(a.x, 4 * j), 4 * j);
            f(scaled(a.y, 4 * j + 1), 4 * j + 1);
            f(scaled(a.z, 4 * j + 2), 4 * j + 2);
            f(scaled(a.w, 4 * j + 3), 4 * j + 3);
            if (j2 < n4) {
                f(scaled(b.x, 4 * j2), 4 * j2);
                f(scaled(b.y, 4 * j2 + 1), 4 * j2 + 1);
                f(scaled(b.z, 4 * j2 + 2), 4 * j2 + 2);
                f(scaled(b.w, 4 * j2 + 3), 4 * j2 + 3);
            }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += THREADS) f(scaled(row[i], i), i);
    }
}

// The largest threshold t (as a key) such that stat({z >= t}) >= target, found by a radix
// descent over the 32 key bits, 8 bits a level.  mode 0: stat = count (top-k);
// mode 1: stat = sum of exp(z - zmax) (top-p, target = top_p * total mass).
__device__ unsigned radix_threshold(const float* row, int lo, int hi, int vocab, float inv_temp, float penalty,
                                    const unsigned* seen_bits, float keep_min, int mode, float target,
                                    float zmax, float* hist /*[THREADS / 32][256]*/, float* scratch, Exchange* ex) {
    unsigned prefix = 0;
    float above = 0.f;  // stat of everything strictly above the current bucket range
    for (int level = 3; level >= 0; --level) {
        // a histogram per warp: the tokens of a row crowd into a few dozen buckets, and with one
        // histogram for the block its adds queued up behind each other (200 us a level)
        for (int b = threadIdx.x; b < (THREADS / 32) * 256; b += THREADS) hist[b] = 0.f;
        float* mine = hist + (threadIdx.x >> 5) * 256;
        __syncthreads();
        unsigned shift = level * 8;
        unsigned mask_hi = level == 3 ? 0u : (0xffffffffu << (shift + 8));
        // Neighbouring logits mostly fall into the same bucket (at the top level nearly all of a
        // row share two or three): a thread adds up its run of equal buckets in a register and
        // touches shared memory only when the bucket changes.  (One atomic per token made this
        // loop twenty times slower: a hundred thousand adds to the same few words.)
        int run_bucket = -1;
        float run_sum = 0.f;
        for_each_scaled(row, lo, hi, vocab, inv_temp, penalty, seen_bits, [&](float z, int) {
            if (z < keep_min) return;
            unsigned key = float_key(z);
            if ((key & mask_hi) != (prefix & mask_hi)) return;
            int bucket = (int)((key >> shift) & 255u);
            float w = mode == 0 ? 1.f : expf(z - zmax);
            if (bucket == run_bucket) {
                run_sum += w;
            } else {
                if (run_bucket >= 0) atomicAdd(&mine[run_bucket], run_sum);
                run_bucket = bucket;
                run_sum = w;
            }
        });
        if (run_bucket >= 0) atomicAdd(&mine[run_bucket], run_sum);
        __syncthreads();
        int turn = ex->turn;
        if (threadIdx.x < 256) {
            // the warps' histograms summed (in warp order), handed to every block of the cluster
            float total = 0.f;
            for (int w = 0; w < THREADS / 32; ++w) total += hist[w * 256 + threadIdx.x];
            unsigned me = cluster_rank();
            for (unsigned k = 0; k < CLUSTER; ++k) peer_store(&ex->hist[turn][me][threadIdx.x], k, total);
        }
        cluster_sync();
        if (threadIdx.x < 256) {  // ... and the blocks' histograms (in block order): the same in every block
            float total = 0.f;
            for (int k = 0; k < CLUSTER; ++k) total += ex->hist[turn][k][threadIdx.x];
            ex->total[threadIdx.x] = total;
        }
        __syncthreads();
        // thread 0 walks the buckets from the top
        if (threadIdx.x == 0) {
            ex->turn = turn ^ 1;
            float run = above;
            int b = 255;
            for (; b > 0; --b) {
                if (run + ex->total[b] >= target) break;
                run += ex->total[b];
            }
            scratch[0] = run;
            scratch[1] = (float)b;
        }
        __syncthreads();
        above = scratch[0];
        prefix |= ((unsigned)scratch[1]) << shift;
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ penalty,
              const unsigned* __restrict__ seen_bits, int seen_words,
              const long long* __restrict__ seeds, const long long* __restrict__ draws,
              int* __restrict__ out_tokens, float* __restrict__ out_logprob) {
    __shared__ Best best_scratch[THREADS / 32];
    __shared__ float sum_scratch[THREADS / 32];
    __shared__ float small[2];
    extern __shared__ __align__(16) unsigned char dynamic[];  // the warps' histograms, the exchange slots
    float* hist = reinterpret_cast<float*>(dynamic);          // [THREADS / 32][256]
    Exchange* ex = reinterpret_cast<Exchange*>(hist + (THREADS / 32) * 256);
    ie_pdl_trigger();
    ie_pdl_wait();
    if (threadIdx.x == 0) ex->turn = 0;
    cluster_sync();  // every block of the cluster runs (its shared memory may be written) and has its turn set
    int r = blockIdx.x / CLUSTER;
    // this block's slice of the row: CLUSTER slices of a multiple of four tokens
    int len = ((vocab + CLUSTER - 1) / CLUSTER + 3) & ~3;
    int lo = min((int)cluster_rank() * len, vocab), hi = min(lo + len, vocab);
    const float* row = logits + (size_t)r * vocab;
    float temp = temperature ? temperature[r] : 0.f;
    float pen = penalty ? penalty[r] : 1.f;
    const unsigned* seen = (seen_bits && pen != 1.f) ? seen_bits + (size_t)r * seen_words : nullptr;
    bool greedy = !(temp > 0.f);
    float inv_temp = greedy ? 1.f : 1.f / temp;

    int k = (!greedy && top_k) ? top_k[r] : 0;
    float p = (!greedy && top_p) ? top_p[r] : 1.f;
    float mp = (!greedy && min_p) ? min_p[r] : 0.f;

    // Pass 1: the maximum of the scaled logits: the greedy answer, and what the cut-offs are
    // taken against.  A row that is drawn from all tokens needs neither.
    float zmax = 0.f;
    int choice = 0;
    if (greedy || (k > 0 && k < vocab) || p < 1.f || mp > 0.f) {
        Best b{-INFINITY, 0x7fffffff};
        for_each_scaled(row, lo, hi, vocab, inv_temp, pen, seen, [&](float z, int i) { b = better(b, Best{z, i}); });
        b = cluster_best(b, best_scratch, ex);
        zmax = b.v;
        choice = b.i;
    }
    float keep_min = -INFINITY;  // tokens with a scaled logit below this are cut off

    if (!greedy) {
        if (k > 0 && k < vocab) {
            unsigned key = radix_threshold(row, lo, hi, vocab, inv_temp, pen, seen, keep_min, 0, (float)k,
                                           zmax, hist, small, ex);
            keep_min = fmaxf(keep_min, key_float(key));
        }
        if (p < 1.f) {
            float mass = 0.f;
            for_each_scaled(row, lo, hi, vocab, inv_temp, pen, seen, [&](float z, int) {
                if (z >= keep_min) mass += expf(z - zmax);
            });
            mass = cluster_sum(mass, sum_scratch, ex);
            // Keep the smallest set of top tokens whose mass reaches top_p
            // (engine/runtime/sampler.py:59-68, with its 1e-6 slack).
            unsigned key = radix_threshold(row, lo, hi, vocab, inv_temp, pen, seen, keep_min, 1,
                                           fmaxf(p - 1e-6f, 0.f) * mass, zmax, hist, small, ex);
            keep_min = fmaxf(keep_min, key_float(key));
        }
        if (mp > 0.f) {
            // Drop tokens whose probability is below min_p times the largest probability:
            // exp(z - zmax) < min_p  <=>  z < zmax + log(min_p)   (sampler.py:39-42)
            keep_min = fmaxf(keep_min, zmax + logf(mp));
        }
        unsigned long long seed = (unsigned long long)seeds[r];
        unsigned long long draw = (unsigned long long)draws[r];
        Best g{-INFINITY, 0x7fffffff};
        // four tokens to a thread and turn: they share one call of the generator (token i takes
        // word i % 4 of call i / 4), which is most of this loop's arithmetic
        for (int i4 = lo + threadIdx.x * 4; i4 < hi; i4 += THREADS * 4) {
            float z[4];
            bool kept = false;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                z[j] = i4 + j < hi ? scaled_logit(row, i4 + j, inv_temp, pen, seen) : -INFINITY;
                kept = kept || (z[j] >= keep_min && z[j] > -INFINITY);
            }
            if (!kept) continue;
            uint4 rnd = random_words(seed, draw, (unsigned)i4 >> 2);
            unsigned words[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (i4 + j >= hi || z[j] < keep_min) continue;
                g = better(g, Best{z[j] - logf(-logf(uniform_of(words[j]))), i4 + j});
            }
        }
        g = cluster_best(g, best_scratch, ex);
        choice = g.i;
    }
    if (out_logprob) {
        // log-probability of the chosen token under the model's own distribution, before
        // temperature and cut-offs (engine/runtime/engine.py:283-298).
        Best raw{-INFINITY, 0};
        for_each_scaled(row, lo, hi, vocab, 1.f, 1.f, nullptr, [&](float z, int i) { raw = better(raw, Best{z, i}); });
        raw = cluster_best(raw, best_scratch, ex);
        float s = 0.f;
        for_each_scaled(row, lo, hi, vocab, 1.f, 1.f, nullptr, [&](float z, int) { s += expf(z - raw.v); });
        s = cluster_sum(s, sum_scratch, ex);
        if (threadIdx.x == 0 && cluster_rank() == 0) out_logprob[r] = row[choice] - raw.v - logf(s);
    }
    if (threadIdx.x == 0 && cluster_rank() == 0) out_tokens[r] = choice;
    cluster_sync();  // no block leaves while another may still write into its shared memory
}

// Greedy choice for many rows at once: every row is cut into `chunks` pieces that different
// blocks scan, then one warp per row picks the best piece (lowest index on ties, as above).
__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const float* __restrict__ logits, int vocab, int chunks, float* __restrict__ part_v,
                    int* __restrict__ part_i) {
    __shared__ Best scratch[8];
    ie_pdl_trigger();
    ie_pdl_wait();
    int r = blockIdx.x, c = blockIdx.y;
    int len = (vocab + chunks - 1) / chunks;
    int lo = c * len, hi = min(vocab, lo + len);
    const float* row = logits + (size_t)r * vocab;
    Best b{-INFINITY, 0x7fffffff};
    int i = lo + threadIdx.x;
    for (; i + 3 * 256 < hi; i += 4 * 256) {  // four independent loads in flight per thread
        float v0 = row[i], v1 = row[i + 256], v2 = row[i + 512], v3 = row[i + 768];
        b = better(b, Best{v0, i}); b = better(b, Best{v1, i + 256});
        b = better(b, Best{v2, i + 512}); b = better(b, Best{v3, i + 768});
    }
    for (; i < hi; i += 256) b = better(b, Best{row[i], i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
    }
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        Best best = scratch[0];
        for (int w = 1; w < 8; ++w) best = better(best, scratch[w]);
        part_v[(size_t)r * chunks + c] = best.v;
        part_i[(size_t)r * chunks + c] = best.i;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int chunks, int* __restrict__ out_tokens) {
    ie_pdl_trigger();
    ie_pdl_wait();
    int r = blockIdx.x;
    Best b{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < chunks; c += 32)
        b = better(b, Best{part_v[(size_t)r * chunks + c], part_i[(size_t)r * chunks + c]});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
        b = better(b, other);
    }
    if (threadIdx.x == 0) out_tokens[r] = b.i;
}
}  // namespace

// Greedy tokens for all rows.  `scratch` holds 2 * num_rows * chunks 32-bit words.
IE_API int ie_argmax(const float* logits, int num_rows, int vocab, int chunks, void* scratch,
                     int* out_tokens, void* stream) {
    if (num_rows <= 0) return 0;
    if (chunks < 1 || scratch == nullptr) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    float* part_v = (float*)scratch;
    int* part_i = (int*)scratch + (size_t)num_rows * chunks;
    int rc = ie_launch(argmax_chunk_kernel, dim3(num_rows, chunks), dim3(256), 0, s, logits, vocab, chunks,
                       part_v, part_i);
    if (rc != 0) return rc;
    return ie_launch(argmax_final_kernel, dim3(num_rows), dim3(32), 0, s, (const float*)part_v,
                     (const int*)part_i, chunks, out_tokens);
}

// All per-row arrays but `logits` and `out_tokens` may be null (greedy, nothing cut off).
IE_API int ie_sample(const float* logits, int num_rows, int vocab, const float* temperature,
                     const int* top_k, const float* top_p, const float* min_p,
                     const float* penalty, const unsigned* seen_bits, int seen_words,
                     const long long* seeds, const long long* draws, int* out_tokens,
                     float* out_logprob, void* stream) {
    if (num_rows <= 0) return 0;
    if (temperature != nullptr && (seeds == nullptr || draws == nullptr)) return (int)cudaErrorInvalidValue;
    constexpr size_t smem = (size_t)(THREADS / 32) * 256 * sizeof(float) + sizeof(Exchange);
    static IePerDevice configured;
    cudaError_t e = ie_allow_smem(configured, sample_kernel, smem);
    if (e != cudaSuccess) return (int)e;
    return ie_launch_cluster(sample_kernel, dim3((unsigned)num_rows * CLUSTER), dim3(THREADS), smem, (cudaStream_t)stream,
                             dim3(CLUSTER, 1, 1), logits, vocab, temperature, top_k, top_p, min_p, penalty, seen_bits,
                             seen_words, seeds, draws, out_tokens, out_logprob);
}
