// Device-side sampling over fp32 logits [R, V]: argmax, and temperature / top-k / top-p
// draws, one thread block per row, so no logits leave the GPU.
//
// Semantics follow the reference's host sampler (src/compute/Sampling.cpp:119-264):
//   * temperature <= 0 or top_k == 1 is greedy; greedy is the first strict maximum,
//     i.e. the lowest index among equal maxima (:14-27; kernels/cuda/llm/argmax_rows.cu).
//   * otherwise p_i = exp(l_i/T - max/T); candidates are ordered by logit descending;
//     top-k keeps the k best; top-p keeps the smallest prefix whose share of the kept
//     mass reaches p; one uniform u picks the first candidate whose cumulative
//     probability exceeds u.
//   * optional before that: soft-cap cap*tanh(l/cap) (:38-44), then repetition /
//     frequency / presence penalties over a window of recent tokens (:66-117).
// Differences, by design: the order is found with a radix select instead of a sort;
// probabilities are summed as 40-bit fixed-point integers so that the result does not
// depend on the order in which threads add them; equal logits are ordered by index, and
// a top-k or top-p cut that falls inside a run of equal logits keeps the whole run (the
// reference's sort leaves that order unspecified).  The uniform number comes from a
// counter-based generator keyed by (seed, draw index) per request, so a request's stream
// does not depend on what else is in the batch.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define FIXED_ONE 1099511627776.0f  // 2^40

__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// splitmix64 finaliser over (seed, counter): a stateless stream of 64-bit numbers
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t seed, uint64_t counter) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (counter + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct ArgmaxPair {
    float v;
    int i;
};

__device__ __forceinline__ ArgmaxPair better(ArgmaxPair a, ArgmaxPair b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ int block_argmax(const float* __restrict__ row, int V, float* max_out) {
    __shared__ ArgmaxPair red[32];
    ArgmaxPair best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v || (v == best.v && i < best.i)) best = ArgmaxPair{v, i};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgmaxPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgmaxPair b = (lane < (int)(blockDim.x >> 5)) ? red[lane] : ArgmaxPair{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgmaxPair other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
            b = better(b, other);
        }
        if (lane == 0) red[0] = b;
    }
    __syncthreads();
    const ArgmaxPair r = red[0];
    if (max_out) *max_out = r.v;
    // a row of NaN or -inf only: every comparison failed, fall back to index 0
    return r.i == 0x7fffffff ? 0 : r.i;
}

__global__ void argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V) {
    pdl_wait();
    pdl_trigger();
    const float* row = logits + (size_t)blockIdx.x * V;
    const int idx = block_argmax(row, V, nullptr);
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

MM_EXPORT int mm_argmax_rows(const void* logits, void* out, int R, int V, void* stream) {
    MM_REQUIRE(R >= 0 && V > 0, "argmax: bad sizes");
    if (R == 0) return MM_OK;
    mm_launch_pdl(argmax_rows_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, (const float*)logits, (int32_t*)out, V);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// Two stages for wide rows: P blocks per row find (max, lowest index) of their slice, then one
// block per row reduces the P pairs.  `part` holds R*P pairs of (float value, int index).
__global__ void argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ part_val,
                                      int32_t* __restrict__ part_idx, int V, int P) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.y, p = blockIdx.x;
    const int chunk = (V + P - 1) / P;
    const int begin = p * chunk, end = min(V, begin + chunk);
    const float* row = logits + (size_t)r * V;
    __shared__ ArgmaxPair red[32];
    ArgmaxPair best{-INFINITY, 0x7fffffff};
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v || (v == best.v && i < best.i)) best = ArgmaxPair{v, i};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgmaxPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgmaxPair b = (lane < (int)(blockDim.x >> 5)) ? red[lane] : ArgmaxPair{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgmaxPair other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
            b = better(b, other);
        }
        if (lane == 0) {
            part_val[(size_t)r * P + p] = b.v;
            part_idx[(size_t)r * P + p] = b.i;
        }
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int32_t* __restrict__ part_idx,
                                    int32_t* __restrict__ out, int P) {
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, lane = threadIdx.x;
    ArgmaxPair best{-INFINITY, 0x7fffffff};
    for (int p = lane; p < P; p += 32) best = better(best, ArgmaxPair{part_val[(size_t)r * P + p], part_idx[(size_t)r * P + p]});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgmaxPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (lane == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

MM_EXPORT int mm_argmax_rows_split(const void* logits, void* out, void* part_val, void* part_idx, int R, int V, int P,
                                   void* stream) {
    MM_REQUIRE(R >= 0 && V > 0 && P >= 1 && P <= 1024 && R <= 65535, "argmax: bad sizes");
    if (R == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    mm_launch_pdl(argmax_partial_kernel, dim3(P, R), dim3(256), 0, s, (const float*)logits, (float*)part_val, (int32_t*)part_idx, V, P);
    MM_CHECK_LAUNCH();
    mm_launch_pdl(argmax_final_kernel, dim3(R), dim3(32), 0, s, (const float*)part_val, (const int32_t*)part_idx, (int32_t*)out, P);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---- radix select over weighted candidates -----------------------------------
// Candidates are the elements with key >= floor_key.  In the order (key descending,
// index ascending) find the first element whose cumulative weight exceeds `target`.
// Weight is 1 when `by_count`, else the fixed-point probability.  Returns the key of
// that element and, in *tie_rank, how many equal-key elements precede it.
struct SelectResult {
    uint32_t key;
    unsigned long long tie_rank;
    unsigned long long weight_of_key;  // weight of one element with that key
};

__device__ __forceinline__ unsigned long long weight_of(float logit, float inv_t, float max_scaled) {
    const float p = expf(logit * inv_t - max_scaled);
    return (unsigned long long)(p * FIXED_ONE);
}

__device__ SelectResult radix_select(const float* __restrict__ row, int V, float inv_t, float max_scaled,
                                     uint32_t floor_key, bool by_count, unsigned long long target,
                                     unsigned long long* hist /* [256] shared */, uint32_t* bcast /* [2] shared */,
                                     unsigned long long* carry /* shared */) {
    uint32_t prefix = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            const uint32_t key = order_key(v);
            if (key < floor_key) continue;
            if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
            const unsigned long long w = by_count ? 1ull : weight_of(v, inv_t, max_scaled);
            if (w) atomicAdd(&hist[(key >> shift) & 0xffu], w);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long cum = 0, rem = 0;
            int chosen = -1;
            for (int b = 255; b >= 0; --b) {
                if (hist[b] && target < cum + hist[b]) {
                    chosen = b;
                    break;
                }
                cum += hist[b];
            }
            if (chosen >= 0) {
                rem = target - cum;
            } else {
                // target at or beyond the total (rounding at the tail): the last candidate
                chosen = 0;
                for (int b = 0; b < 256; ++b)
                    if (hist[b]) {
                        chosen = b;
                        rem = hist[b] - 1ull;
                        break;
                    }
            }
            bcast[0] = (uint32_t)chosen;
            *carry = rem;
        }
        __syncthreads();
        prefix = (prefix << 8) | bcast[0];
        target = *carry;
        __syncthreads();
    }
    SelectResult r;
    r.key = prefix;
    // all elements with this key have the same logit, hence the same weight
    float key_val;
    {
        const uint32_t u = (prefix & 0x80000000u) ? (prefix & 0x7fffffffu) : ~prefix;
        key_val = __uint_as_float(u);
    }
    r.weight_of_key = by_count ? 1ull : weight_of(key_val, inv_t, max_scaled);
    r.tie_rank = r.weight_of_key ? target / r.weight_of_key : 0ull;
    return r;
}

// index of the (rank)-th element (by ascending index) whose key equals `key`
__device__ int nth_with_key(const float* __restrict__ row, int V, uint32_t key, unsigned long long rank,
                            int* counts /* [blockDim.x] shared */, int* result /* shared */) {
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int begin = threadIdx.x * chunk;
    const int end = min(V, begin + chunk);
    int c = 0;
    for (int i = begin; i < end; ++i) c += (order_key(row[i]) == key);
    counts[threadIdx.x] = c;
    if (threadIdx.x == 0) *result = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        // serial scan over at most 1024 partial counts
        unsigned long long before = 0;
        int owner = -1;
        long long total = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) total += counts[t];
        if (total > 0 && rank >= (unsigned long long)total) rank = (unsigned long long)total - 1;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (rank < before + (unsigned long long)counts[t]) {
                owner = t;
                break;
            }
            before += counts[t];
        }
        counts[0] = owner;
        // reuse *result to carry the remaining rank (fits an int: V < 2^31)
        *result = (int)(rank - before);
    }
    __syncthreads();
    const int owner = counts[0];
    const int rem = *result;
    __syncthreads();
    if ((int)threadIdx.x == owner) {
        int seen = 0;
        for (int i = begin; i < end; ++i) {
            if (order_key(row[i]) == key) {
                if (seen == rem) {
                    *result = i;
                    break;
                }
                ++seen;
            }
        }
    }
    __syncthreads();
    return *result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V,
                   const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                   const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
                   const unsigned long long* __restrict__ counters) {
    __shared__ unsigned long long hist[256];
    __shared__ uint32_t bcast[2];
    __shared__ int counts[SAMPLE_THREADS];
    __shared__ int result;
    __shared__ unsigned long long total_sh;
    __shared__ unsigned long long carry_sh;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const float T = temperature[r];
    const int k = top_k[r];
    const float P = top_p[r];
    float max_logit;
    const int best = block_argmax(row, V, &max_logit);
    if (T <= 0.0f || k == 1) {
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    const float inv_t = 1.0f / T;
    const float max_scaled = max_logit * inv_t;

    // top-k: everything at or above the k-th largest logit stays
    uint32_t floor_key = 0;
    if (k > 0 && k < V) {
        const SelectResult s = radix_select(row, V, inv_t, max_scaled, 0u, true, (unsigned long long)(k - 1), hist, bcast, &carry_sh);
        floor_key = s.key;
    }
    // mass of the kept set
    auto kept_mass = [&](uint32_t fk) -> unsigned long long {
        unsigned long long local = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (order_key(v) >= fk) local += weight_of(v, inv_t, max_scaled);
        }
        if (threadIdx.x == 0) total_sh = 0ull;
        __syncthreads();
        if (local) atomicAdd(&total_sh, local);
        __syncthreads();
        const unsigned long long t = total_sh;
        __syncthreads();
        return t;
    };
    unsigned long long total = kept_mass(floor_key);
    if (total == 0ull) {  // numerical underflow: the reference falls back to the best candidate
        if (threadIdx.x == 0) out[r] = best;
        return;
    }
    // top-p: the smallest prefix whose cumulative share reaches P
    if (P > 0.0f && P < 1.0f) {
        unsigned long long need = (unsigned long long)ceil((double)P * (double)total);
        if (need < 1ull) need = 1ull;
        if (need > total) need = total;
        const SelectResult s = radix_select(row, V, inv_t, max_scaled, floor_key, false, need - 1ull, hist, bcast, &carry_sh);
        if (s.key > floor_key) floor_key = s.key;
        total = kept_mass(floor_key);
    }
    // the draw
    const uint64_t bits = mix64(seeds[r], counters[r]);
    const float u = (float)(bits >> 40) * (1.0f / 16777216.0f);  // 24 bits → [0,1)
    unsigned long long target = (unsigned long long)((double)u * (double)total);
    if (target >= total) target = total - 1ull;
    const SelectResult s = radix_select(row, V, inv_t, max_scaled, floor_key, false, target, hist, bcast, &carry_sh);
    const int idx = nth_with_key(row, V, s.key, s.tie_rank, counts, &result);
    if (threadIdx.x == 0) out[r] = idx >= 0 ? idx : best;
}

MM_EXPORT int mm_sample_rows(const void* logits, void* out, int R, int V, const void* temperature, const void* top_k,
                             const void* top_p, const void* seeds, const void* counters, void* stream) {
    MM_REQUIRE(R >= 0 && V > 0, "sample: bad sizes");
    if (R == 0) return MM_OK;
    sample_rows_kernel<<<R, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(
        (const float*)logits, (int32_t*)out, V, (const float*)temperature, (const int32_t*)top_k, (const float*)top_p,
        (const unsigned long long*)seeds, (const unsigned long long*)counters);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---- soft-cap and penalties, in place on the logits ---------------------------
// recent: int32 [R, W] (entries < 0 are padding).  For each distinct recent token t with
// count c: l = l > 0 ? l / rep : l * rep; l -= freq * c; l -= pres.
__global__ void penalties_kernel(float* __restrict__ logits, int V, const int32_t* __restrict__ recent, int W,
                                 const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres, const float* __restrict__ softcap) {
    const int r = blockIdx.x;
    float* row = logits + (size_t)r * V;
    const float cap = softcap ? softcap[r] : 0.0f;
    if (cap > 0.0f) {
        const float inv = 1.0f / cap;
        for (int i = threadIdx.x; i < V; i += blockDim.x) row[i] = cap * tanhf(row[i] * inv);
        __syncthreads();
    }
    if (recent == nullptr || W <= 0) return;
    const float rp = rep[r], fp = freq[r], pp = pres[r];
    if (rp == 1.0f && fp == 0.0f && pp == 0.0f) return;
    const int32_t* win = recent + (size_t)r * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const int t = win[i];
        if (t < 0 || t >= V) continue;
        int count = 0;
        bool first = true;
        for (int j = 0; j < W; ++j) {
            if (win[j] == t) {
                ++count;
                if (j < i) first = false;
            }
        }
        if (!first) continue;
        float l = row[t];
        if (rp != 1.0f) l = (l > 0.0f) ? (l / rp) : (l * rp);
        if (fp != 0.0f) l -= fp * (float)count;
        if (pp != 0.0f) l -= pp;
        row[t] = l;
    }
}

MM_EXPORT int mm_apply_penalties(void* logits, int R, int V, const void* recent, int W, const void* rep,
                                 const void* freq, const void* pres, const void* softcap, void* stream) {
    MM_REQUIRE(R >= 0 && V > 0 && W >= 0, "penalties: bad sizes");
    if (R == 0) return MM_OK;
    penalties_kernel<<<R, 256, 0, (cudaStream_t)stream>>>((float*)logits, V, (const int32_t*)recent, W, (const float*)rep,
                                                          (const float*)freq, (const float*)pres, (const float*)softcap);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// uniform number of (seed, counter), exported so the host-side plain sampler draws the same stream
MM_EXPORT float mm_uniform_from(unsigned long long seed, unsigned long long counter) {
    return (float)(mix64(seed, counter) >> 40) * (1.0f / 16777216.0f);
}
