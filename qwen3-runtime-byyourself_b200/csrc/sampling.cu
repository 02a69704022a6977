// Token choice on the GPU: greedy argmax, and temperature / top-k / top-p sampling.
//
// The reference chooses greedily on the GPU (src/ops/argmax.cu:34-100: lowest id among
// equals, NaN counts as -inf, optional valid prefix) but samples on the CPU after
// copying the logits to the host (src/generation/sampler.cpp:137-247).  Here both stay
// on the device, one block per row, and only the chosen ids leave it.
//
// Sampling keeps the reference's order and meaning: score = logit / temperature; top-k
// keeps every candidate whose score reaches the k-th best (ties beyond k stay);
// candidates are ordered by score, lower id first among equals; weight = exp(score -
// max); top-p keeps the shortest prefix whose weight reaches top_p of the total; the
// draw takes r = u * kept weight and the first candidate whose cumulative weight
// exceeds r.  Instead of sorting, the kernel finds each boundary by radix selection
// over the order-preserving bit pattern of the logits: equal logits have equal
// weights, so a boundary inside a run of equals is plain arithmetic.  Weights are
// summed as 64-bit fixed point (2^-40 units), which makes the sums independent of the
// order of the additions; a weight below 2^-41 counts as zero.
//
// The uniform number is not the reference's shared mt19937_64 stream (which makes a
// sequence's tokens depend on what else is in the batch): it is a hash of (seed,
// sequence id, step), so every sequence has a stream of its own.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int THREADS = 512;
constexpr double FIX_ONE = 1099511627776.0;  // 2^40

__device__ __forceinline__ uint32_t float_key(float x) {
    if (x == 0.0f) x = 0.0f;  // -0 and +0 are equal scores
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ uint64_t fixed_weight(float logit, double temperature, double max_score) {
    const double w = exp((double)logit / temperature - max_score);
    return (uint64_t)(w * FIX_ONE + 0.5);
}

constexpr int ARGMAX_BLOCKS = 8;   // blocks (one cluster) that share a row

// A row is split over the blocks of a cluster; each finds the best of its share, and the block of
// rank 0 picks among the shares through distributed shared memory.
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int64_t stride, int valid, int* __restrict__ out) {
    __shared__ float best_v[THREADS / 32];
    __shared__ int best_i[THREADS / 32];
    __shared__ float share_v;
    __shared__ int share_i;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x / ARGMAX_BLOCKS, rank = blockIdx.x % ARGMAX_BLOCKS;
    const float* x = logits + (int64_t)row * stride;
    // shares of whole float4 packets, so that every share starts as aligned as the row does
    const int per = (((valid + ARGMAX_BLOCKS - 1) / ARGMAX_BLOCKS) + 3) & ~3;
    const int lo = min(valid, rank * per), hi = min(valid, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (isnan(v)) v = -INFINITY;
        if (v > bv || bi == 0x7fffffff) { bv = v; bi = i; }
    };
    // a thread sees its indices in ascending order, so "greater, or the first" keeps the lowest id
    int done = lo;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const int n4 = (hi - lo) >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x + lo);
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += THREADS) {
            const float4 v = x4[i];
            const int at = lo + 4 * i;
            take(v.x, at); take(v.y, at + 1); take(v.z, at + 2); take(v.w, at + 3);
        }
        done = lo + (n4 << 2);
    }
    for (int i = done + threadIdx.x; i < hi; i += THREADS) take(x[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        share_v = bv;
        share_i = bi;
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (rank == 0 && threadIdx.x == 0) {
        const uint32_t addr_v = (uint32_t)__cvta_generic_to_shared(&share_v), addr_i = (uint32_t)__cvta_generic_to_shared(&share_i);
        for (uint32_t r = 1; r < (uint32_t)ARGMAX_BLOCKS; ++r) {         // an empty share holds (-inf, 0x7fffffff)
            uint32_t remote_v, remote_i;
            float ov;
            int oi;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_v) : "r"(addr_v), "r"(r));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_i) : "r"(addr_i), "r"(r));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(ov) : "r"(remote_v) : "memory");
            asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(oi) : "r"(remote_i) : "memory");
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        out[row] = bi;
    }
    // nobody leaves while its share may still be read
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct Selected {
    uint32_t key;      // bit pattern of the boundary logit
    uint64_t before;   // weight (or count) of everything ordered before the run of `key`
    uint64_t inside;   // weight (or count) of the run of `key`
};

constexpr int S_THREADS = 1024;   // threads of a block of the sampling kernel
constexpr int S_BLOCKS_MAX = 8;   // most blocks (one cluster) that share a row
constexpr int SHORT_LIST = 1024;  // candidates that are sorted in shared memory instead of selected by radix
constexpr int PRIVATE_BYTES = 32 * 1024;   // private histograms of the warps (dynamic shared memory)

__device__ __forceinline__ void cluster_sync() {
    __syncwarp();                   // the barrier wants the warp converged
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The value of a shared-memory variable of this kernel in the block of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t remote_u32(const void* local, uint32_t rank) {
    uint32_t addr, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long remote_u64(const void* local, uint32_t rank) {
    uint32_t addr;
    unsigned long long v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// What a block tells the others of its cluster.
struct Share {
    float max_logit;
    int bad;
    uint32_t bound;
    int listed;                     // candidates in this block's list (SHORT_LIST + 1: too many)
    unsigned long long weight;      // total weight of this block's candidates
    int equals;                     // logits of this block equal to the drawn key
};

// Finds the key at which the cumulative sum, taken from the highest key downwards, first reaches
// `threshold` (1 <= threshold <= sum over all candidates), over the logits of the whole row: every
// block histograms its own share [lo, hi) and the histograms are added over the cluster.  WEIGHTED:
// sums fixed-point weights of the candidates (key >= floor_key); otherwise counts all.
// Most logits share their high bits, so one histogram for the block would be thousands of atomics
// on one address: every warp (every pair of warps for the 64-bit sums) counts into a histogram of
// its own in `priv`, and the histograms are added up afterwards.  `local_hist` is [2][256]: the
// passes alternate between the halves, so one cluster barrier a pass is enough.
template <bool WEIGHTED>
__device__ Selected radix_select(const float* __restrict__ x, int lo, int hi, uint64_t threshold, uint32_t floor_key,
                                 double temperature, double max_score, unsigned long long* local_hist,
                                 unsigned long long* hist, uint64_t* bcast, void* priv, int& pass, int n_blocks) {
    using Word = typename std::conditional<WEIGHTED, unsigned long long, unsigned int>::type;
    constexpr int COPIES = PRIVATE_BYTES / (256 * (int)sizeof(Word));      // 32 or 16
    Word* mine = reinterpret_cast<Word*>(priv) + ((threadIdx.x >> 5) % COPIES) * 256;
    uint32_t prefix = 0, mask = 0;
    uint64_t before = 0, inside = 0;
    for (int shift = 24; shift >= 0; shift -= 8, ++pass) {
        unsigned long long* mine_hist = local_hist + (pass & 1) * 256;
        for (int b = threadIdx.x; b < COPIES * 256; b += S_THREADS) reinterpret_cast<Word*>(priv)[b] = 0;
        __syncthreads();
        for (int i = lo + threadIdx.x; i < hi; i += S_THREADS) {
            const float v = x[i];
            const uint32_t key = float_key(v);
            if ((key & mask) != prefix || key < floor_key) continue;
            const Word add = WEIGHTED ? (Word)fixed_weight(v, temperature, max_score) : (Word)1;
            if (add) atomicAdd(&mine[(key >> shift) & 255u], add);
        }
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += S_THREADS) {
            unsigned long long sum = 0ull;
#pragma unroll 4
            for (int c = 0; c < COPIES; ++c) sum += reinterpret_cast<Word*>(priv)[c * 256 + b];
            mine_hist[b] = sum;
        }
        cluster_sync();                                                  // every block's histogram of this pass stands
        for (int b = threadIdx.x; b < 256; b += S_THREADS) {
            unsigned long long sum = 0ull;
            for (uint32_t r = 0; r < (uint32_t)n_blocks; ++r) sum += remote_u64(&mine_hist[b], r);
            hist[b] = sum;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int chosen = -1, last_nonzero = 0;
            uint64_t run = before;
            for (int b = 255; b >= 0; --b) {
                const uint64_t h = hist[b];
                if (h == 0) continue;
                last_nonzero = b;
                if (run + h >= threshold) { chosen = b; break; }
                run += h;
            }
            if (chosen < 0) {  // threshold above the total: settle on the last run
                chosen = last_nonzero;
                run -= hist[chosen];
            }
            bcast[0] = (uint64_t)chosen;
            bcast[1] = run;
            bcast[2] = hist[chosen];
        }
        __syncthreads();
        prefix |= (uint32_t)bcast[0] << shift;
        mask |= 255u << shift;
        before = bcast[1];
        inside = bcast[2];
        __syncthreads();
    }
    return Selected{prefix, before, inside};
}

// The uniform number of a row: a hash of (seed, sequence id, step), 53 bits.
__device__ __forceinline__ double uniform_of(uint64_t seed, int64_t seq_id, int step) {
    const uint64_t h = splitmix64(splitmix64(seed ^ splitmix64((uint64_t)seq_id)) + (uint64_t)step);
    return (double)(h >> 11) * (1.0 / 9007199254740992.0);
}

// One cluster of `n_blocks` blocks per row; a block reads its share [lo, hi) of the row.  Every block
// takes the same decisions from the same exchanged numbers, so all of them reach the same cluster
// barriers; the block of rank 0 finishes the short list.
__global__ void __launch_bounds__(S_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t stride, int valid, float temperature_f, int top_k, float top_p,
              uint64_t seed, const int64_t* __restrict__ seq_ids, const int* __restrict__ steps, int step_all,
              int* __restrict__ out, int n_blocks) {
    extern __shared__ __align__(16) unsigned char private_histograms[];   // PRIVATE_BYTES
    __shared__ unsigned long long local_hist[2 * 256];
    __shared__ unsigned long long hist[256];
    __shared__ uint64_t bcast[3];
    __shared__ float red[33];
    __shared__ Share share;
    __shared__ int counts[S_THREADS];
    __shared__ int found[2];
    __shared__ unsigned long long list[SHORT_LIST];      // (key << 32) | ~id, then cumulative weights
    __shared__ int list_id[SHORT_LIST];
    __shared__ int n_list;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x / n_blocks, tid = threadIdx.x;
    const uint32_t rank = blockIdx.x % n_blocks;
    const float* x = logits + (int64_t)row * stride;
    const int per = (valid + n_blocks - 1) / n_blocks;
    const int lo = min(valid, (int)rank * per), hi = min(valid, lo + per);
    int pass = 0;                                                        // radix passes so far (their parity picks a buffer)

    // the maximum, and a refusal of rows with NaN or Inf (the reference throws there)
    float mx = -INFINITY;
    int bad = 0;
    for (int i = lo + tid; i < hi; i += S_THREADS) {
        const float v = x[i];
        if (!isfinite(v)) bad = 1;
        mx = fmaxf(mx, v);
    }
    bad = __syncthreads_or(bad);
    const float thread_max = mx;
    mx = block_max(mx, red);
    if (tid == 0) {
        share.max_logit = mx;
        share.bad = bad;
    }
    cluster_sync();
    for (uint32_t r = 0; r < (uint32_t)n_blocks; ++r) {
        mx = fmaxf(mx, __uint_as_float(remote_u32(&share.max_logit, r)));
        bad |= (int)remote_u32(&share.bad, r);
    }
    if (bad) {                                                           // the same in every block of the cluster
        if (tid == 0 && rank == 0) out[row] = -1;
        cluster_sync();                                                  // nobody leaves while its numbers may be read
        return;
    }
    const double temperature = (double)temperature_f;
    const double max_score = (double)mx / temperature;
    const double u = uniform_of(seed, seq_ids[row], steps != nullptr ? steps[row] : step_all);

    // bitonic sort of the 1024 words of `list`, descending: one element a thread
    auto sort_list = [&]() {
        for (int size = 2; size <= SHORT_LIST; size <<= 1) {
            for (int gap = size >> 1; gap > 0; gap >>= 1) {
                const int other = tid ^ gap;
                if (other > tid) {
                    const unsigned long long a = list[tid], b = list[other];
                    const bool descending = (tid & size) == 0;
                    if ((a < b) == descending) { list[tid] = b; list[other] = a; }
                }
                __syncthreads();
            }
        }
    };
    // Every logit of the row whose key reaches `floor` goes to the list of rank 0 as (key << 32) | ~id: each
    // block lists its own, rank 0 fetches the lists.  Returns how many there are in the row (more than
    // SHORT_LIST: the list of rank 0 is not complete).  Two cluster barriers.
    auto gather = [&](uint32_t floor) {
        if (tid == 0) n_list = 0;
        list[tid] = 0ull;                                                // padding sorts to the end
        __syncthreads();
        for (int i = lo + tid; i < hi; i += S_THREADS) {
            const uint32_t key = float_key(x[i]);
            if (key >= floor) {
                const int at = atomicAdd(&n_list, 1);
                if (at < SHORT_LIST) list[at] = ((unsigned long long)key << 32) | (uint32_t)(~(uint32_t)i);
            }
        }
        __syncthreads();
        if (tid == 0) share.listed = min(n_list, SHORT_LIST + 1);
        cluster_sync();
        int total = 0, mine_at = 0;
        for (uint32_t r = 0; r < (uint32_t)n_blocks; ++r) {
            const int n = (int)remote_u32(&share.listed, r);
            if (r < rank) mine_at += n;
            total += n;
        }
        if (rank == 0 && total <= SHORT_LIST) {
            int at = (int)remote_u32(&share.listed, 0);
            for (uint32_t r = 1; r < (uint32_t)n_blocks; ++r) {
                const int n = (int)remote_u32(&share.listed, r);
                for (int j = tid; j < n; j += S_THREADS) list[at + j] = remote_u64(&list[j], r);
                at += n;
            }
        }
        cluster_sync();                                                  // the other blocks' lists are free again
        return total;
    };

    // top-k: the k-th best key; every key that reaches it stays
    uint32_t floor_key = 0;
    uint64_t n_candidates = (uint64_t)valid;
    bool listed = false;                                                 // the candidates stand sorted in the list of rank 0
    if (top_k > 0 && top_k < valid && top_k <= S_THREADS) {
        // The k-th best of the threads' own maxima is a lower bound of the k-th best logit (k logits reach
        // it), so what reaches that bound holds every candidate, ties included, and is usually a short list.
        list[tid] = thread_max == -INFINITY ? 0ull : (unsigned long long)float_key(thread_max);
        __syncthreads();
        sort_list();
        if (tid == 0) share.bound = (uint32_t)list[top_k - 1];
        cluster_sync();
        uint32_t bound = 0u;
        for (uint32_t r = 0; r < (uint32_t)n_blocks; ++r) bound = max(bound, remote_u32(&share.bound, r));
        if (bound != 0u && gather(bound) <= SHORT_LIST) {
            listed = true;
            if (rank == 0) {
                sort_list();
                floor_key = (uint32_t)(list[top_k - 1] >> 32);
                if ((uint32_t)(list[tid] >> 32) >= floor_key &&
                    (tid + 1 == SHORT_LIST || (uint32_t)(list[tid + 1] >> 32) < floor_key))
                    found[1] = tid + 1;                                  // keys fall along the list: one thread sees the edge
                __syncthreads();
                n_candidates = (uint64_t)found[1];
            }
        }
    }
    if (!listed && top_k > 0 && top_k < valid) {
        const Selected kth = radix_select<false>(x, lo, hi, (uint64_t)top_k, 0u, temperature, max_score, local_hist, hist,
                                                 bcast, private_histograms, pass, n_blocks);
        floor_key = kth.key;
        n_candidates = kth.before + kth.inside;
    }
    if (!listed && n_candidates <= (uint64_t)SHORT_LIST) {
        gather(floor_key);
        listed = true;
        if (rank == 0) sort_list();
    }

    if (listed) {
        // ---- few candidates, sorted as the reference orders them (score down, then id up) in the list of
        // rank 0: walk the running sums there
        if (rank == 0) {
            const int n = (int)n_candidates;
            unsigned long long w = 0ull;
            if (tid < n) {
                const unsigned long long e = list[tid];
                list_id[tid] = (int)(~(uint32_t)e);
                w = fixed_weight(key_float((uint32_t)(e >> 32)), temperature, max_score);
            }
            __syncthreads();
            list[tid] = w;
            __syncthreads();
            for (int off = 1; off < SHORT_LIST; off <<= 1) {             // Hillis-Steele over 1024 words
                const unsigned long long add = tid >= off ? list[tid - off] : 0ull;
                __syncthreads();
                list[tid] += add;
                __syncthreads();
            }
            const uint64_t total = list[n - 1];                          // >= 2^40: the maximum itself has weight one
            uint64_t cut = (uint64_t)ceil((double)top_p * (double)total);
            cut = cut < 1 ? 1 : (cut > total ? total : cut);
            // top-p: the shortest prefix whose weight reaches the cut
            if (tid < n && list[tid] >= cut && (tid == 0 || list[tid - 1] < cut)) found[0] = tid;
            __syncthreads();
            const uint64_t kept = list[found[0]];
            uint64_t r = (uint64_t)(u * (double)kept);
            if (r >= kept) r = kept - 1;
            // the draw: the first candidate whose cumulative weight exceeds r (it lies inside the kept prefix)
            if (tid < n && list[tid] > r && (tid == 0 || list[tid - 1] <= r)) out[row] = list_id[tid];
        }
        return;                                                          // nothing of another block is read after `gather`
    }

    // ---- many candidates (no top-k, or a long run of equal logits at its edge): selection by radix
    // total weight of the candidates
    unsigned long long part = 0ull;
    for (int i = lo + tid; i < hi; i += S_THREADS) {
        const float v = x[i];
        if (float_key(v) >= floor_key) part += fixed_weight(v, temperature, max_score);
    }
    if (tid == 0) share.weight = 0ull;
    __syncthreads();
    if (part) atomicAdd(&share.weight, part);
    cluster_sync();
    uint64_t total = 0;
    for (uint32_t r = 0; r < (uint32_t)n_blocks; ++r) total += remote_u64(&share.weight, r);   // >= 2^40

    // top-p: shortest prefix whose weight reaches top_p * total
    uint64_t cut = (uint64_t)ceil((double)top_p * (double)total);
    cut = cut < 1 ? 1 : (cut > total ? total : cut);
    const Selected edge = radix_select<true>(x, lo, hi, cut, floor_key, temperature, max_score, local_hist, hist, bcast,
                                             private_histograms, pass, n_blocks);
    const uint64_t edge_w = fixed_weight(key_float(edge.key), temperature, max_score);
    uint64_t edge_n = edge_w ? (cut - edge.before + edge_w - 1) / edge_w : 1;
    const uint64_t edge_count = edge_w ? edge.inside / edge_w : 1;
    edge_n = edge_n < 1 ? 1 : (edge_n > edge_count ? edge_count : edge_n);
    const uint64_t kept = edge.before + edge_n * edge_w;

    // the draw: first candidate whose cumulative weight exceeds r = u * kept
    uint64_t r = (uint64_t)(u * (double)kept);
    if (r >= kept) r = kept - 1;
    const Selected hit = radix_select<true>(x, lo, hi, r + 1, floor_key, temperature, max_score, local_hist, hist, bcast,
                                            private_histograms, pass, n_blocks);
    const uint64_t hit_w = fixed_weight(key_float(hit.key), temperature, max_score);
    const uint64_t hit_count = hit_w ? hit.inside / hit_w : 1;
    uint64_t nth = hit_w ? (r - hit.before) / hit_w : 0;  // 0-based place inside the run of equals
    if (nth >= hit_count) nth = hit_count - 1;

    // the nth lowest id among the logits equal to hit.key: the blocks hold ascending id ranges, and so do
    // the threads of a block
    const int chunk = (hi - lo + S_THREADS - 1) / S_THREADS;
    const int t_lo = lo + tid * chunk, t_hi = min(hi, t_lo + chunk);
    int mine = 0;
    for (int i = t_lo; i < t_hi; ++i) mine += float_key(x[i]) == hit.key;
    counts[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        int sum = 0;
        for (int t = 0; t < S_THREADS; ++t) sum += counts[t];
        share.equals = sum;
    }
    cluster_sync();
    int64_t left = (int64_t)nth;
    int owner_rank = -1, last_rank = -1, last_count = 0;
    for (uint32_t q = 0; q < (uint32_t)n_blocks; ++q) {
        const int c = (int)remote_u32(&share.equals, q);
        if (c == 0) continue;
        last_rank = (int)q;
        last_count = c;
        if (left < c) { owner_rank = (int)q; break; }
        left -= c;
    }
    if (owner_rank < 0) { owner_rank = last_rank; left = last_count - 1; }
    cluster_sync();                                                      // the numbers of the other blocks are read
    if (owner_rank < 0) {
        if (tid == 0 && rank == 0) out[row] = -1;
        return;
    }
    if ((int)rank != owner_rank) return;
    if (tid == 0) {
        int owner = -1, last_owner = -1;
        for (int t = 0; t < S_THREADS; ++t) {
            if (counts[t] == 0) continue;
            last_owner = t;
            if (left < counts[t]) { owner = t; break; }
            left -= counts[t];
        }
        if (owner < 0) { owner = last_owner; left = counts[last_owner] - 1; }
        found[0] = owner;
        found[1] = (int)left;
    }
    __syncthreads();
    if (tid == found[0]) {
        int skip = found[1], id = -1;
        for (int i = t_lo; i < t_hi; ++i) {
            if (float_key(x[i]) == hit.key) {
                if (skip == 0) { id = i; break; }
                --skip;
            }
        }
        out[row] = id;
    }
}

}  // namespace

Q3_EXPORT int q3_argmax_f32(const float* logits, int64_t stride, int rows, int valid, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (valid <= 0 || valid > stride) return Q3_ERR_BAD_SIZE;
    if ((int64_t)rows * ARGMAX_BLOCKS > 2147483647LL) return Q3_ERR_TOO_LARGE;
    return (int)q3_launch_cluster(argmax_kernel, dim3(rows * ARGMAX_BLOCKS), dim3(THREADS), 0, (cudaStream_t)stream,
                                  dim3(ARGMAX_BLOCKS, 1, 1), logits, stride, valid, out);
}

// out[row] = -1 marks a row with a non-finite logit.  `steps` may be null: every row is then at step `step_all`.
Q3_EXPORT int q3_sample_f32(const float* logits, int64_t stride, int rows, int valid, float temperature, int top_k,
                            float top_p, uint64_t seed, const int64_t* seq_ids, const int* steps, int step_all, int* out,
                            void* stream) {
    if (rows <= 0) return 0;
    if (valid <= 0 || valid > stride || !(temperature > 0.0f) || top_k < 0 || !(top_p > 0.0f && top_p <= 1.0f))
        return Q3_ERR_BAD_SIZE;
    static Q3PerDevice configured;              // static and dynamic shared memory together pass the default limit of 48 KB
    {
        cudaError_t e = q3_allow_shared_memory(sample_kernel, PRIVATE_BYTES, configured);
        if (e != cudaSuccess) return (int)e;
    }
    // blocks per row: as many as keep the clusters of all rows resident at once (one block of 1,024 threads an SM)
    const int sms = q3_device_sm_count();
    int n_blocks = S_BLOCKS_MAX;
    while (n_blocks > 1 && (int64_t)rows * n_blocks > sms) n_blocks >>= 1;
    return (int)q3_launch_cluster(sample_kernel, dim3(rows * n_blocks), dim3(S_THREADS), PRIVATE_BYTES, (cudaStream_t)stream,
                                  dim3(n_blocks, 1, 1), logits, stride, valid, temperature, top_k, top_p, seed, seq_ids,
                                  steps, step_all, out, n_blocks);
}
