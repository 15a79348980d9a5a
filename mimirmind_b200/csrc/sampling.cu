// Device-side sampling over fp32 logits [R, V]: argmax, and temperature / top-k / top-p
// draws (one thread-block cluster per row, the CTAs of a cluster share the row), so no logits
// leave the GPU.
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
    const float* row = logits + (size_t)blockIdx.x * V;
    const int idx = block_argmax(row, V, nullptr);
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

MM_EXPORT int mm_argmax_rows(const void* logits, void* out, int R, int V, void* stream) {
    MM_REQUIRE(R >= 0 && V > 0, "argmax: bad sizes");
    if (R == 0) return MM_OK;
    mm_launch(argmax_rows_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, (const float*)logits, (int32_t*)out, V);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// Two stages for wide rows: P blocks per row find (max, lowest index) of their slice, then one
// block per row reduces the P pairs.  `part` holds R*P pairs of (float value, int index).
__global__ void argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ part_val,
                                      int32_t* __restrict__ part_idx, int V, int P) {
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
    mm_launch(argmax_partial_kernel, dim3(P, R), dim3(256), 0, s, (const float*)logits, (float*)part_val, (int32_t*)part_idx, V, P);
    MM_CHECK_LAUNCH();
    mm_launch(argmax_final_kernel, dim3(R), dim3(32), 0, s, (const float*)part_val, (const int32_t*)part_idx, (int32_t*)out, P);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---- sampling: one thread-block cluster per row -------------------------------------------------------------
// The CTAs of a cluster take contiguous slices of the row.  Whatever the whole row decides (its maximum, the mass
// of the kept set, the histogram of a radix pass, how many elements carry the chosen key) is computed per CTA,
// published in shared memory, and read by every CTA of the cluster from its peers through distributed shared
// memory after one cluster barrier; all CTAs then hold the same numbers and take the same branch.  Publications
// alternate between two buffers, so one barrier per exchange is enough: a CTA can run at most one exchange ahead of
// a peer that is still reading.  Histograms are per warp (64-bit shared-memory adds collide within a warp only).
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
#define SAMPLE_MAX_CLUSTER 8

struct SampleShared {
    unsigned long long whist[SAMPLE_WARPS][256];   // per-warp histograms of a radix pass
    unsigned long long pub[2][256 + 4];            // what this CTA publishes: a histogram, or scalars in [256..]
    unsigned long long tot[256];                   // the cluster's histogram
    unsigned long long warp_part[SAMPLE_WARPS];
    unsigned long long carry;
    uint32_t chosen;
    int counts[SAMPLE_THREADS];
    int result;
};

struct ClusterCtx {
    SampleShared* sh;
    const float* vals;                             // this CTA's slice: its copy in shared memory, or the row itself
    int vals_begin;                                // index of vals[0] in the row
    uint32_t rank, n_ranks;
    uint32_t round;                                // exchanges so far: selects the publication buffer
};

__device__ __forceinline__ void sample_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;\n" ::: "memory");
}
// The same word of every CTA of the cluster: the loads go out together (a loop that adds each value as it arrives would
// wait for one remote load after the other).  v[r] for r >= n_ranks is 0.
__device__ __forceinline__ void ld_all_peers_u64(const unsigned long long* local, uint32_t n_ranks, unsigned long long* v) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t remote[SAMPLE_MAX_CLUSTER];
#pragma unroll
    for (uint32_t r = 0; r < SAMPLE_MAX_CLUSTER; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote[r]) : "r"(addr), "r"(r < n_ranks ? r : 0u));
#pragma unroll
    for (uint32_t r = 0; r < SAMPLE_MAX_CLUSTER; ++r) {
        v[r] = 0ull;
        if (r < n_ranks) asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(v[r]) : "r"(remote[r]));
    }
}
__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    return v;
}

// The CTA's value (held by thread 0 after a block reduction through warp_part) is published; returns the sum
// (or the maximum) over the cluster, the same in every thread of every CTA.
__device__ unsigned long long cluster_combine(ClusterCtx& c, unsigned long long mine, bool take_max) {
    SampleShared* sh = c.sh;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    mine = take_max ? warp_max_u64(mine) : warp_sum_u64(mine);
    if (lane == 0) sh->warp_part[warp] = mine;
    __syncthreads();
    const uint32_t b = c.round & 1;
    if (warp == 0) {
        unsigned long long v = lane < SAMPLE_WARPS ? sh->warp_part[lane] : 0ull;
        v = take_max ? warp_max_u64(v) : warp_sum_u64(v);
        if (lane == 0) sh->pub[b][256] = v;
    }
    __syncthreads();
    sample_cluster_sync();
    unsigned long long all = 0ull, v[SAMPLE_MAX_CLUSTER];
    ld_all_peers_u64(&sh->pub[b][256], c.n_ranks, v);
#pragma unroll
    for (uint32_t r = 0; r < SAMPLE_MAX_CLUSTER; ++r) all = take_max ? (v[r] > all ? v[r] : all) : all + v[r];
    ++c.round;
    return all;
}

__device__ __forceinline__ unsigned long long weight_of(float logit, float inv_t, float max_scaled) {
    const float p = expf(logit * inv_t - max_scaled);
    return (unsigned long long)(p * FIXED_ONE);
}

// Candidates are the elements with key >= floor_key.  In the order (key descending, index ascending) find the
// first element whose cumulative weight exceeds `target`.  Weight is 1 when `by_count`, else the fixed-point
// probability.  Returns the key of that element and how many equal-key elements precede it.
struct SelectResult {
    uint32_t key;
    unsigned long long tie_rank;
};

__device__ SelectResult radix_select(ClusterCtx& c, const float* __restrict__ row, int begin, int end, float inv_t,
                                     float max_scaled, uint32_t floor_key, bool by_count, unsigned long long target) {
    SampleShared* sh = c.sh;
    const int warp = threadIdx.x >> 5;
    uint32_t prefix = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = threadIdx.x; i < SAMPLE_WARPS * 256; i += SAMPLE_THREADS) (&sh->whist[0][0])[i] = 0ull;
        __syncthreads();
        for (int i = begin + (int)threadIdx.x; i < end; i += 4 * SAMPLE_THREADS) {
            float v[4];                                          // four loads in flight when the slice is in global memory
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = i + u * SAMPLE_THREADS;
                v[u] = j < end ? c.vals[j - c.vals_begin] : __int_as_float(0x7fc00000);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i + u * SAMPLE_THREADS >= end) continue;
                const uint32_t key = order_key(v[u]);
                if (key < floor_key) continue;
                if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
                const unsigned long long w = by_count ? 1ull : weight_of(v[u], inv_t, max_scaled);
                if (w) atomicAdd(&sh->whist[warp][(key >> shift) & 0xffu], w);
            }
        }
        __syncthreads();
        const uint32_t b = c.round & 1;
        if (threadIdx.x < 256) {
            unsigned long long sum = 0ull;
#pragma unroll 8
            for (int w = 0; w < SAMPLE_WARPS; ++w) sum += sh->whist[w][threadIdx.x];
            sh->pub[b][threadIdx.x] = sum;
        }
        __syncthreads();
        sample_cluster_sync();
        if (threadIdx.x < 256) {
            unsigned long long sum = 0ull, v[SAMPLE_MAX_CLUSTER];
            ld_all_peers_u64(&sh->pub[b][threadIdx.x], c.n_ranks, v);
#pragma unroll
            for (uint32_t r = 0; r < SAMPLE_MAX_CLUSTER; ++r) sum += v[r];
            sh->tot[threadIdx.x] = sum;
        }
        ++c.round;
        __syncthreads();
        if (warp == 0) {
            // bins in descending order, eight per lane: lane L holds bins 255 - 8L .. 248 - 8L; the weight of all
            // bins before a lane's comes from a shuffle scan
            const int lane = threadIdx.x & 31;
            unsigned long long h[8], mine = 0ull;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                h[j] = sh->tot[255 - 8 * lane - j];
                mine += h[j];
            }
            unsigned long long incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            unsigned long long cum = incl - mine;
            int chosen = -1;
            unsigned long long rem = 0ull;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (chosen < 0 && h[j] && target < cum + h[j]) {
                    chosen = 255 - 8 * lane - j;
                    rem = target - cum;
                }
                cum += h[j];
            }
            const uint32_t found = __ballot_sync(0xffffffffu, chosen >= 0);
            if (found) {
                if (lane == __ffs(found) - 1) {                  // the first lane in descending bin order
                    sh->chosen = (uint32_t)chosen;
                    sh->carry = rem;
                }
            } else if (lane == 0) {
                // target at or beyond the total (rounding at the tail): the last candidate
                int last = 0;
                unsigned long long left = 0ull;
                for (int bin = 0; bin < 256; ++bin)
                    if (sh->tot[bin]) {
                        last = bin;
                        left = sh->tot[bin] - 1ull;
                        break;
                    }
                sh->chosen = (uint32_t)last;
                sh->carry = left;
            }
        }
        __syncthreads();
        prefix = (prefix << 8) | sh->chosen;
        target = sh->carry;
        __syncthreads();
    }
    SelectResult r;
    r.key = prefix;
    // all elements with this key have the same logit, hence the same weight
    const uint32_t u = (prefix & 0x80000000u) ? (prefix & 0x7fffffffu) : ~prefix;
    const unsigned long long w = by_count ? 1ull : weight_of(__uint_as_float(u), inv_t, max_scaled);
    r.tie_rank = w ? target / w : 0ull;
    return r;
}

// Index of the (rank)-th element, by ascending index, whose key equals `key`; written to out_token by the thread
// that owns it.  Returns nothing: if no element has the key, rank 0's thread 0 writes `fallback`.
__device__ void write_nth_with_key(ClusterCtx& c, const float* __restrict__ row, int begin, int end, uint32_t key,
                                   unsigned long long rank, int fallback, int32_t* out_token) {
    SampleShared* sh = c.sh;
    const int len = end - begin;
    const int sub = (len + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = begin + min(len, (int)threadIdx.x * sub), hi = begin + min(len, ((int)threadIdx.x + 1) * sub);
    int cnt = 0;
    for (int i = lo; i < hi; ++i) cnt += (order_key(c.vals[i - c.vals_begin]) == key);
    sh->counts[threadIdx.x] = cnt;
    // every CTA publishes how many it holds (cluster_combine would only give the sum: the prefix needs each)
    const unsigned long long mine = warp_sum_u64((unsigned long long)cnt);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) sh->warp_part[warp] = mine;
    __syncthreads();
    const uint32_t b = c.round & 1;
    if (threadIdx.x == 0) {
        unsigned long long v = 0ull;
        for (int w = 0; w < SAMPLE_WARPS; ++w) v += sh->warp_part[w];
        sh->pub[b][256] = v;
    }
    __syncthreads();
    sample_cluster_sync();
    unsigned long long before = 0ull, total = 0ull, v[SAMPLE_MAX_CLUSTER];
    ld_all_peers_u64(&sh->pub[b][256], c.n_ranks, v);
#pragma unroll
    for (uint32_t r = 0; r < SAMPLE_MAX_CLUSTER; ++r) {
        if (r < c.rank) before += v[r];
        total += v[r];
    }
    ++c.round;
    if (total == 0ull) {
        if (c.rank == 0 && threadIdx.x == 0) *out_token = fallback;
        return;
    }
    if (rank >= total) rank = total - 1ull;
    const unsigned long long here = sh->pub[b][256];
    if (rank < before || rank >= before + here) return;           // another CTA's slice holds it
    rank -= before;
    if (threadIdx.x == 0) {
        unsigned long long seen = 0ull;
        int owner = 0;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            if (rank < seen + (unsigned long long)sh->counts[t]) {
                owner = t;
                break;
            }
            seen += (unsigned long long)sh->counts[t];
        }
        sh->chosen = (uint32_t)owner;
        sh->result = (int)(rank - seen);
    }
    __syncthreads();
    if (threadIdx.x == sh->chosen) {
        int seen = 0;
        const int rem = sh->result;
        for (int i = lo; i < hi; ++i)
            if (order_key(c.vals[i - c.vals_begin]) == key) {
                if (seen == rem) {
                    *out_token = i;
                    break;
                }
                ++seen;
            }
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out, int V,
                   const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                   const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
                   const unsigned long long* __restrict__ counters, int cache_floats) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    ClusterCtx c;
    c.sh = reinterpret_cast<SampleShared*>(sample_smem);
    c.rank = blockIdx.x;                                           // the cluster spans x
    c.n_ranks = gridDim.x;
    c.round = 0;
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * V;
    const float T = temperature[r];
    const int k = top_k[r];
    const float P = top_p[r];
    const int chunk = (V + (int)c.n_ranks - 1) / (int)c.n_ranks;
    const int begin = min(V, (int)c.rank * chunk), end = min(V, begin + chunk);

    // maximum and its lowest index: (order key, ~index) packed so that the larger number is the better pair;
    // NaN takes no part; a row without any number gives index 0
    // The slice is read from global memory once, four loads in flight per thread, and kept in shared memory if it
    // fits (`cache_floats` > 0): the passes below then read it from there.
    float* cache = reinterpret_cast<float*>(sample_smem + sizeof(SampleShared));
    const bool cached = cache_floats >= end - begin;
    unsigned long long best = 0ull;
    for (int i = begin + (int)threadIdx.x; i < end; i += 4 * SAMPLE_THREADS) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = i + u * SAMPLE_THREADS;
            v[u] = j < end ? row[j] : __int_as_float(0x7fc00000);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = i + u * SAMPLE_THREADS;
            if (j >= end) continue;
            if (cached) cache[j - begin] = v[u];
            if (v[u] != v[u]) continue;
            const unsigned long long packed = ((unsigned long long)order_key(v[u]) << 32) | (uint32_t)(~(uint32_t)j);
            best = packed > best ? packed : best;
        }
    }
    c.vals = cached ? cache : row;
    c.vals_begin = cached ? begin : 0;
    best = cluster_combine(c, best, true);
    const int best_index = best ? (int)(~(uint32_t)(best & 0xffffffffull)) : 0;
    // (every path below ends with a cluster barrier: no CTA may exit while a peer still reads its shared memory)
    if (T <= 0.0f || k == 1 || best == 0ull) {
        if (c.rank == 0 && threadIdx.x == 0) out[r] = best_index;
        sample_cluster_sync();
        return;
    }
    float max_logit;
    {
        const uint32_t key = (uint32_t)(best >> 32);
        max_logit = __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
    }
    const float inv_t = 1.0f / T;
    const float max_scaled = max_logit * inv_t;

    // top-k: everything at or above the k-th largest logit stays
    uint32_t floor_key = 0;
    if (k > 0 && k < V) floor_key = radix_select(c, row, begin, end, inv_t, max_scaled, 0u, true, (unsigned long long)(k - 1)).key;
    auto kept_mass = [&](uint32_t fk) -> unsigned long long {
        unsigned long long local = 0;
        for (int i = begin + (int)threadIdx.x; i < end; i += 4 * SAMPLE_THREADS) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = i + u * SAMPLE_THREADS;
                v[u] = j < end ? c.vals[j - c.vals_begin] : __int_as_float(0x7fc00000);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + u * SAMPLE_THREADS < end && order_key(v[u]) >= fk) local += weight_of(v[u], inv_t, max_scaled);
        }
        return cluster_combine(c, local, false);
    };
    unsigned long long total = kept_mass(floor_key);
    if (total == 0ull) {  // numerical underflow: the reference falls back to the best candidate
        if (c.rank == 0 && threadIdx.x == 0) out[r] = best_index;
        sample_cluster_sync();
        return;
    }
    // top-p: the smallest prefix whose cumulative share reaches P
    if (P > 0.0f && P < 1.0f) {
        unsigned long long need = (unsigned long long)ceil((double)P * (double)total);
        if (need < 1ull) need = 1ull;
        if (need > total) need = total;
        const SelectResult s = radix_select(c, row, begin, end, inv_t, max_scaled, floor_key, false, need - 1ull);
        if (s.key > floor_key) floor_key = s.key;
        total = kept_mass(floor_key);
    }
    // the draw
    const uint64_t bits = mix64(seeds[r], counters[r]);
    const float u = (float)(bits >> 40) * (1.0f / 16777216.0f);  // 24 bits → [0,1)
    unsigned long long target = (unsigned long long)((double)u * (double)total);
    if (target >= total) target = total - 1ull;
    const SelectResult s = radix_select(c, row, begin, end, inv_t, max_scaled, floor_key, false, target);
    write_nth_with_key(c, row, begin, end, s.key, s.tie_rank, best_index, &out[r]);
    sample_cluster_sync();
}

MM_EXPORT int mm_sample_rows(const void* logits, void* out, int R, int V, const void* temperature, const void* top_k,
                             const void* top_p, const void* seeds, const void* counters, void* stream) {
    MM_REQUIRE(R >= 0 && R <= 65535 && V > 0, "sample: bad sizes");
    if (R == 0) return MM_OK;
    // a wide row is shared by a cluster of CTAs (a power of two: other sizes place badly); a narrow one is one CTA's
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int ranks = 1;
    while (ranks < SAMPLE_MAX_CLUSTER && V / (ranks * 2) >= 4096 && (ranks == 1 || R * ranks * 2 <= 2 * sms)) ranks *= 2;   // one wave of two CTAs per SM
    // a copy of the CTA's slice in shared memory if it fits beside the histograms
    const int chunk = (V + ranks - 1) / ranks;
    const size_t room = 200 * 1024 - sizeof(SampleShared);
    // (with the copy only one CTA fits on an SM: worth it while every CTA of the launch has an SM of its own)
    const int cache_floats = ((size_t)chunk * sizeof(float) <= room && R * ranks <= sms) ? chunk : 0;
    const size_t smem = sizeof(SampleShared) + (size_t)cache_floats * sizeof(float);
    static size_t ceiling = 0;
    if (smem > ceiling) {
        if (cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("sample: cannot reserve shared memory");
            return MM_ERR_LAUNCH;
        }
        ceiling = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ranks, R);
    cfg.blockDim = dim3(SAMPLE_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ranks > 1 ? 1 : 0;
    cudaLaunchKernelEx(&cfg, sample_rows_kernel, (const float*)logits, (int32_t*)out, V, (const float*)temperature,
                       (const int32_t*)top_k, (const float*)top_p, (const unsigned long long*)seeds,
                       (const unsigned long long*)counters, cache_floats);
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

// recent: int32 [R, W] rings of the last widths[r] tokens of each row (entries beyond the width, or not yet filled,
// are -1); lengths[r] counts the row's tokens so far.  Puts tokens[r] at lengths[r] % widths[r] and advances the count:
// the window of a captured decode step follows the sequence without the host.
__global__ void window_push_kernel(int32_t* __restrict__ recent, int W, const int32_t* __restrict__ widths,
                                   long long* __restrict__ lengths, const int32_t* __restrict__ tokens, int R) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    const int w = widths[r] < W ? widths[r] : W;
    if (w > 0) recent[(size_t)r * W + (int)(lengths[r] % w)] = tokens[r];
    lengths[r] += 1;
}

MM_EXPORT int mm_window_push(void* recent, int R, int W, const void* widths, void* lengths, const void* tokens, void* stream) {
    MM_REQUIRE(R >= 0 && W >= 1, "window_push: bad sizes");
    if (R == 0) return MM_OK;
    window_push_kernel<<<(R + 127) / 128, 128, 0, (cudaStream_t)stream>>>((int32_t*)recent, W, (const int32_t*)widths,
                                                                         (long long*)lengths, (const int32_t*)tokens, R);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// After a decode step: every request's position moves on by one, its draw counter too (null: no counters), and the
// sampled tokens become the next step's inputs (null: the caller feeds them).
__global__ void advance_step_kernel(int32_t* __restrict__ positions, long long* __restrict__ counters, int32_t* __restrict__ next_ids,
                                    const int32_t* __restrict__ tokens, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    positions[i] += 1;
    if (counters != nullptr) counters[i] += 1;
    if (next_ids != nullptr) next_ids[i] = tokens[i];
}

MM_EXPORT int mm_advance_step(void* positions, void* counters, void* next_ids, const void* tokens, int n, void* stream) {
    MM_REQUIRE(n >= 0 && positions != nullptr && (next_ids == nullptr || tokens != nullptr), "advance_step: bad arguments");
    if (n == 0) return MM_OK;
    advance_step_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((int32_t*)positions, (long long*)counters, (int32_t*)next_ids,
                                                                          (const int32_t*)tokens, n);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// uniform number of (seed, counter), exported so the host-side plain sampler draws the same stream
MM_EXPORT float mm_uniform_from(unsigned long long seed, unsigned long long counter) {
    return (float)(mix64(seed, counter) >> 40) * (1.0f / 16777216.0f);
}
