// Attention over the paged cache, in its general form: any head size in steps of 16 up
// to 256, any number of heads and groups, any mix of prompt and decode tokens in one
// launch, float or bf16 elements with 32-bit scores, softmax and sums.  It is the
// 32-bit path's attention and the fallback of the bf16 path for head sizes that the
// tensor-core kernels do not take.
//
//   qkv_prepare : per-head RMSNorm of q and k, rotation, and the write of k and v
//                 into their cache pages - one pass over the projection output where
//                 the reference runs rms_norm x2 (src/model/self_attention.cpp:147-149),
//                 apply_rope x2 (:152, src/ops/rope.cu:60-84) and two strided copies
//                 (src/model/kv_cache.cpp:165-188).
//   attention   : causal grouped-query attention by loop bound, scale after the dot,
//                 online softmax (src/ops/gqa_attention.cu:42-44,84-86,117,119-144,152).
//
// Cache layout: pages [page, kv head, PAGE tokens, head_dim]; `page_table[seq]` lists
// the pages of a sequence in order.  Keys are visited page by page in ascending
// position, so the result for one (position, head) does not depend on how the tokens
// were cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int PAGE = Q3_PAGE_TOKENS;
constexpr int MAX_HEAD_DIM = 256;

template <typename T> __device__ __forceinline__ void load_pack_f32(const T* p, float (&v)[Pack<T>::N]) {
    const Pack<T> k = load_pack<T>(p);
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) v[i] = k.get(i);
}
template <typename T> __device__ __forceinline__ void store_pack_f32(T* p, const float (&v)[Pack<T>::N]) {
    Pack<T> k;
#pragma unroll
    for (int i = 0; i < Pack<T>::N; ++i) k.set(i, v[i]);
    store_pack<T>(p, k);
}

template <typename T>
__global__ void qkv_prepare_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                   T* __restrict__ v_pages, const float* __restrict__ q_norm_w,
                                   const float* __restrict__ k_norm_w, const float* __restrict__ cos_tab,
                                   const float* __restrict__ sin_tab, const int* __restrict__ token_seq,
                                   const int* __restrict__ token_pos, const int* __restrict__ page_table,
                                   int pages_per_seq, int nq, int nkv, int d, float eps, int write_kv, int rot) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x * warps + warp;
    if (head >= nq + 2 * nkv || (head >= nq && !write_kv)) return;   // a layer that reads another layer's cache writes none
    const int64_t t = blockIdx.y;
    const int pos = token_pos[t];
    const T* src = qkv + t * (int64_t)(nq + 2 * nkv) * d + (int64_t)head * d;

    T* dst;
    const float* norm_w = nullptr;
    bool rotate = cos_tab != nullptr;
    if (head < nq) {
        dst = q_out + t * (int64_t)nq * d + (int64_t)head * d;
        norm_w = q_norm_w;
    } else {
        const int kvh = (head - nq) % nkv;
        const bool is_v = head >= nq + nkv;
        const int page = page_table[(int64_t)token_seq[t] * pages_per_seq + pos / PAGE];
        dst = (is_v ? v_pages : k_pages) + (((int64_t)page * nkv + kvh) * PAGE + pos % PAGE) * d;
        norm_w = is_v ? nullptr : k_norm_w;
        rotate = rotate && !is_v;
    }

    // The first `rot` values of the head are rotated in pairs (i, i + rot/2), i = lane + 32 n; the values from
    // `rot` on (none when the whole head is rotated, as in Qwen3) are normalised and pass through.
    const int rhalf = rot >> 1;
    float a[MAX_HEAD_DIM / 64], b[MAX_HEAD_DIM / 64], c[MAX_HEAD_DIM / 32];
    float sq = 0.0f;
#pragma unroll
    for (int n = 0; n < MAX_HEAD_DIM / 64; ++n) {
        const int i = lane + 32 * n;
        a[n] = b[n] = 0.0f;
        if (i < rhalf) {
            a[n] = to_f32<T>(src[i]);
            b[n] = to_f32<T>(src[i + rhalf]);
            sq += a[n] * a[n] + b[n] * b[n];
        }
    }
    if (rot < d) {
#pragma unroll
        for (int n = 0; n < MAX_HEAD_DIM / 32; ++n) {
            const int i = rot + lane + 32 * n;
            c[n] = 0.0f;
            if (i < d) {
                c[n] = to_f32<T>(src[i]);
                sq += c[n] * c[n];
            }
        }
    }
    if (norm_w != nullptr) {
        const float inv = rsqrtf(warp_sum(sq) / (float)d + eps);
#pragma unroll
        for (int n = 0; n < MAX_HEAD_DIM / 64; ++n) {
            const int i = lane + 32 * n;
            if (i < rhalf) {
                a[n] = round_to<T>(round_to<T>(a[n] * inv) * norm_w[i]);
                b[n] = round_to<T>(round_to<T>(b[n] * inv) * norm_w[i + rhalf]);
            }
        }
        if (rot < d) {
#pragma unroll
            for (int n = 0; n < MAX_HEAD_DIM / 32; ++n) {
                const int i = rot + lane + 32 * n;
                if (i < d) c[n] = round_to<T>(round_to<T>(c[n] * inv) * norm_w[i]);
            }
        }
    }
#pragma unroll
    for (int n = 0; n < MAX_HEAD_DIM / 64; ++n) {
        const int i = lane + 32 * n;
        if (i < rhalf) {
            float x = a[n], y = b[n];
            if (rotate) {
                const float cs = cos_tab[(int64_t)pos * rhalf + i], sn = sin_tab[(int64_t)pos * rhalf + i];
                x = a[n] * cs - b[n] * sn;
                y = b[n] * cs + a[n] * sn;
            }
            dst[i] = from_f32<T>(x);
            dst[i + rhalf] = from_f32<T>(y);
        }
    }
    if (rot < d) {
#pragma unroll
        for (int n = 0; n < MAX_HEAD_DIM / 32; ++n) {
            const int i = rot + lane + 32 * n;
            if (i < d) dst[i] = from_f32<T>(c[n]);
        }
    }
}

// The same with 16-byte accesses: a head is shared by half/VEC lanes, each of which owns VEC
// consecutive elements of the first half and the matching VEC of the second half (the two members
// of every rotation pair), so a warp works on several heads at once.  One warp per group of
// consecutive (token, head) pairs.
template <typename T>
__global__ void qkv_prepare_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pages,
                                       T* __restrict__ v_pages, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, const float* __restrict__ cos_tab,
                                       const float* __restrict__ sin_tab, const int* __restrict__ token_seq,
                                       const int* __restrict__ token_pos, const int* __restrict__ page_table,
                                       int pages_per_seq, int nq, int nkv, int d, float eps, int write_kv,
                                       int64_t n_tokens) {
    constexpr int VEC = Pack<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int half = d >> 1, lph = half / VEC, hpw = 32 / lph;       // lanes per head, heads per warp
    const int lane = threadIdx.x & 31, sub = lane % lph, grp = lane / lph;
    const int heads = nq + 2 * nkv;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t pair = warp * hpw + grp;                             // flat (token, head) index
    const bool active = grp < hpw && pair < n_tokens * heads;
    const int64_t t = active ? pair / heads : 0;
    const int head = active ? (int)(pair % heads) : 0;
    const bool is_q = head < nq, is_v = head >= nq + nkv;
    const bool live = active && (is_q || write_kv);
    const int pos = token_pos[t];
    const T* src = qkv + (t * heads + head) * (int64_t)d + sub * VEC;
    float a[VEC], b[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) a[i] = b[i] = 0.0f;
    if (live) {
        load_pack_f32<T>(src, a);
        load_pack_f32<T>(src + half, b);
    }
    const float* norm_w = is_q ? q_norm_w : (is_v ? nullptr : k_norm_w);
    // the sum over the lanes of a head: every lane of the warp takes part in every shuffle
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) sq += a[i] * a[i] + b[i] * b[i];
    float total = 0.0f;
    const int first = grp * lph;
    for (int j = 0; j < lph; ++j) total += __shfl_sync(0xffffffffu, sq, (first + j) & 31);
    if (norm_w != nullptr) {
        const float inv = rsqrtf(total / (float)d + eps);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            a[i] = round_to<T>(round_to<T>(a[i] * inv) * norm_w[sub * VEC + i]);
            b[i] = round_to<T>(round_to<T>(b[i] * inv) * norm_w[half + sub * VEC + i]);
        }
    }
    if (!live) return;
    if (cos_tab != nullptr && !is_v) {
        const float* c = cos_tab + (int64_t)pos * half + sub * VEC;
        const float* sn = sin_tab + (int64_t)pos * half + sub * VEC;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float x = a[i] * c[i] - b[i] * sn[i], y = b[i] * c[i] + a[i] * sn[i];
            a[i] = x;
            b[i] = y;
        }
    }
    T* dst;
    if (is_q) {
        dst = q_out + (t * nq + head) * (int64_t)d;
    } else {
        const int kvh = (head - nq) % nkv;
        const int page = page_table[(int64_t)token_seq[t] * pages_per_seq + pos / PAGE];
        dst = (is_v ? v_pages : k_pages) + (((int64_t)page * nkv + kvh) * PAGE + pos % PAGE) * d;
    }
    store_pack_f32<T>(dst + sub * VEC, a);
    store_pack_f32<T>(dst + half + sub * VEC, b);
}

// One block per (query head, token).  128 threads: the four warps share the keys of a
// page for the scores; thread t owns output dims t and t + 128.
template <typename T>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                         T* __restrict__ out, const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                         const int* __restrict__ page_table, int pages_per_seq, int nq, int nkv, int d, float scale,
                         int window) {
    __shared__ float q_s[MAX_HEAD_DIM];
    __shared__ float score[PAGE];
    __shared__ float prob[PAGE];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, kvh = head / (nq / nkv);
    const int64_t t = blockIdx.y;
    const int pos = token_pos[t];
    const int* pages = page_table + (int64_t)token_seq[t] * pages_per_seq;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int i = tid; i < d; i += 128) q_s[i] = to_f32<T>(q[(t * nq + head) * (int64_t)d + i]);
    __syncthreads();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m_run = -INFINITY, l_run = 0.0f, acc0 = 0.0f, acc1 = 0.0f;
    for (int pg = lo / PAGE; pg <= pos / PAGE; ++pg) {
        const int64_t base = ((int64_t)pages[pg] * nkv + kvh) * PAGE * d;
        const T* kp = k_pages + base;
        const T* vp = v_pages + base;
        const int j_lo = max(lo - pg * PAGE, 0), j_hi = min(pos - pg * PAGE, PAGE - 1);  // inclusive, in-page
        for (int j = warp; j < PAGE; j += 4) {
            float dot = 0.0f;
            if (j >= j_lo && j <= j_hi) {
                for (int i = lane; i < d; i += 32) dot = fmaf(q_s[i], to_f32<T>(kp[(int64_t)j * d + i]), dot);
            }
            dot = warp_sum(dot);
            if (lane == 0) score[j] = (j >= j_lo && j <= j_hi) ? dot * scale : -INFINITY;
        }
        __syncthreads();
        float m_new = m_run;
        for (int j = 0; j < PAGE; ++j) m_new = fmaxf(m_new, score[j]);
        if (tid < PAGE) prob[tid] = (tid >= j_lo && tid <= j_hi) ? expf(score[tid] - m_new) : 0.0f;
        __syncthreads();
        const float alpha = expf(m_run - m_new);  // 0 on the first page (m_run = -inf, m_new finite)
        float l_add = 0.0f, v0 = 0.0f, v1 = 0.0f;
        for (int j = j_lo; j <= j_hi; ++j) {
            const float p = prob[j];
            l_add += p;
            if (tid < d) v0 = fmaf(p, to_f32<T>(vp[(int64_t)j * d + tid]), v0);
            if (tid + 128 < d) v1 = fmaf(p, to_f32<T>(vp[(int64_t)j * d + tid + 128]), v1);
        }
        l_run = l_run * alpha + l_add;
        acc0 = acc0 * alpha + v0;
        acc1 = acc1 * alpha + v1;
        m_run = m_new;
        __syncthreads();  // score/prob are rewritten by the next page
    }
    T* o = out + (t * nq + head) * (int64_t)d;
    if (tid < d) o[tid] = from_f32<T>(acc0 / l_run);
    if (tid + 128 < d) o[tid + 128] = from_f32<T>(acc1 / l_run);
}

template <typename T>
int qkv_prepare_launch(const T* qkv, T* q_out, T* k_pages, T* v_pages, const float* q_norm_w, const float* k_norm_w,
                       const float* cos_tab, const float* sin_tab, const int* token_seq, const int* token_pos,
                       const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d, float eps,
                       int write_kv, int rot, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || d % 2 != 0 || d > MAX_HEAD_DIM || nq <= 0 || nkv <= 0) return Q3_ERR_BAD_SIZE;
    if (rot <= 0) rot = d;                       // the whole head is rotated
    if (rot % 2 != 0 || rot > d) return Q3_ERR_BAD_SIZE;
    constexpr int VEC = Pack<T>::N;
    if (rot == d && n_tokens >= 64 && (d / 2) % VEC == 0 && (d / 2) / VEC <= 32 && aligned16(qkv) && aligned16(q_out) &&
        aligned16(k_pages) && aligned16(v_pages)) {
        const int hpw = 32 / ((d / 2) / VEC);
        const int64_t n_warps = (n_tokens * (nq + 2 * nkv) + hpw - 1) / hpw;
        const int64_t blocks = (n_warps + 7) / 8;
        if (blocks > 0x7fffffffLL) return Q3_ERR_TOO_LARGE;
        return (int)q3_launch(qkv_prepare_vec_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, qkv, q_out, k_pages,
                              v_pages, q_norm_w, k_norm_w, cos_tab, sin_tab, token_seq, token_pos, page_table, pages_per_seq,
                              nq, nkv, d, eps, write_kv, n_tokens);
    }
    if (n_tokens > 65535) return Q3_ERR_TOO_LARGE;
    const int warps = 4;
    const dim3 grid((nq + 2 * nkv + warps - 1) / warps, (unsigned)n_tokens);
    return (int)q3_launch(qkv_prepare_kernel<T>, grid, dim3(warps * 32), 0, stream, qkv, q_out, k_pages, v_pages, q_norm_w,
                          k_norm_w, cos_tab, sin_tab, token_seq, token_pos, page_table, pages_per_seq, nq, nkv, d, eps, write_kv, rot);
}

template <typename T>
int attention_generic_launch(const T* q, const T* k_pages, const T* v_pages, T* out, const int* token_seq,
                             const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq,
                             int nkv, int d, float scale, int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d <= 0 || d > MAX_HEAD_DIM || nq <= 0 || nkv <= 0 || nq % nkv != 0) return Q3_ERR_BAD_SIZE;
    if (n_tokens > 65535) return Q3_ERR_TOO_LARGE;
    const dim3 grid(nq, (unsigned)n_tokens);
    return (int)q3_launch(attention_generic_kernel<T>, grid, dim3(128), 0, stream, q, k_pages, v_pages, out, token_seq,
                          token_pos, page_table, pages_per_seq, nq, nkv, d, scale, window);
}

}  // namespace

#define Q3_ATTENTION_EXPORTS(SUFFIX, T)                                                                               \
    Q3_EXPORT int q3_qkv_prepare_##SUFFIX(const void* qkv, void* q_out, void* k_pages, void* v_pages,                  \
                                          const float* q_norm_w, const float* k_norm_w, const float* cos_tab,         \
                                          const float* sin_tab, const int* token_seq, const int* token_pos,           \
                                          const int* page_table, int pages_per_seq, int64_t n_tokens, int nq,         \
                                          int nkv, int d, float eps, int write_kv, int rotary_dim, void* stream) {   \
        return qkv_prepare_launch<T>((const T*)qkv, (T*)q_out, (T*)k_pages, (T*)v_pages, q_norm_w, k_norm_w, cos_tab, \
                                     sin_tab, token_seq, token_pos, page_table, pages_per_seq, n_tokens, nq, nkv, d,  \
                                     eps, write_kv, rotary_dim, (cudaStream_t)stream);                                \
    }                                                                                                                 \
    Q3_EXPORT int q3_attention_generic_##SUFFIX(const void* q, const void* k_pages, const void* v_pages, void* out,   \
                                                const int* token_seq, const int* token_pos, const int* page_table,    \
                                                int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d,          \
                                                float scale, int window, void* stream) {                              \
        return attention_generic_launch<T>((const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, token_seq,     \
                                           token_pos, page_table, pages_per_seq, n_tokens, nq, nkv, d, scale, window, \
                                           (cudaStream_t)stream);                                                     \
    }

Q3_ATTENTION_EXPORTS(f32, float)
Q3_ATTENTION_EXPORTS(bf16, bf16)
