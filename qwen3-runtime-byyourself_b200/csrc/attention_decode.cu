// Decode attention over the paged cache for bfloat16: one new token per sequence, its
// query heads of one kv group against every cached key, split over the keys.
//
// Replaces the reference's one-block-per-(token, head) kernel with its serial loop over
// keys and a block-wide reduction per key (src/ops/gqa_attention.cu:84-148).  The math is
// the same: score = q.k * d^-0.5, online softmax and weighted sum in 32-bit
// (src/ops/gqa_attention.cu:117-144), here with the dots on the tensor cores.
//
// Work split: grid (split, kv head, sequence).  A block takes a contiguous range of the
// sequence's pages; each of its four warps owns 16 of the 64 keys of every page and runs
// its own online softmax over them, fed by its own cp.async pipeline (the K and V panels
// of 16 keys are contiguous in a page).  All query heads of the group (up to 16) ride as
// the rows of one m16n8k16 tile, so the group's K and V are read once.  The warps' partial
// results are merged in shared memory, the splits' in a second small kernel through a
// float32 scratch buffer.  Compiled for one head size: -DQ3_HEAD_DIM=<multiple of 16>.
#include "common.cuh"

#ifndef Q3_HEAD_DIM
#error "compile with -DQ3_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = Q3_HEAD_DIM;
constexpr int PAGE = 64;
constexpr int WARPS = 4;
constexpr int KEYS_PER_WARP = PAGE / WARPS;        // 16
constexpr int ROW_BYTES = D * 2 + 16;              // padded row: ldmatrix reads without bank conflicts
constexpr int PANEL_BYTES = KEYS_PER_WARP * ROW_BYTES;
constexpr int STAGES = 3;
constexpr int CHUNKS_PER_ROW = D / 8;              // 16-byte chunks
constexpr int NT = D / 8;                          // n-tiles of the output
constexpr int KT = D / 16;                         // k-tiles of the scores
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size: multiples of 16 up to 256");

constexpr int SMEM_PIPE = WARPS * STAGES * 2 * PANEL_BYTES;
constexpr int SMEM_MERGE = WARPS * 16 * (D + 2) * 4;
constexpr int SMEM_BYTES = SMEM_PIPE > SMEM_MERGE ? SMEM_PIPE : SMEM_MERGE;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies one warp's panel (16 keys x D) of a page into padded shared rows.
__device__ __forceinline__ void load_panel(uint32_t dst, const bf16* src, int lane) {
#pragma unroll
    for (int i = lane; i < KEYS_PER_WARP * CHUNKS_PER_ROW; i += 32) {
        const int row = i / CHUNKS_PER_ROW, c = i % CHUNKS_PER_ROW;
        cp_async16(dst + row * ROW_BYTES + c * 16, src + row * D + c * 8);
    }
}

// part_o: [tokens, nq, splits, D] float32 (unnormalised sums); part_ml: [tokens, nq, splits, 2] (max, sum).
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                    float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ token_seq,
                    const int* __restrict__ token_pos, const int* __restrict__ page_table, int pages_per_seq, int nq,
                    int nkv, float scale_log2, int window) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_wait();
    const int split = blockIdx.x, n_splits = gridDim.x, kvh = blockIdx.y, t = blockIdx.z;
    const int G = nq / nkv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int quad = lane >> 2, tq = lane & 3;
    const int pos = token_pos[t];
    const int* pages = page_table + (int64_t)token_seq[t] * pages_per_seq;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_page = lo / PAGE, n_pages = pos / PAGE + 1 - first_page;
    const int per_split = (n_pages + n_splits - 1) / n_splits;
    const int pg_begin = first_page + split * per_split;
    const int pg_end = min(first_page + n_pages, pg_begin + per_split);
    const int count = max(pg_end - pg_begin, 0);

    // query rows of the group as A fragments: row r = head kvh*G + r (rows >= G are zero)
    uint32_t qa[KT][4];
    {
        const bf16* q0 = q + ((int64_t)t * nq + (int64_t)kvh * G) * D;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            const int c = kt * 16 + tq * 2;
            qa[kt][0] = quad < G ? *reinterpret_cast<const uint32_t*>(q0 + quad * D + c) : 0u;
            qa[kt][1] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (quad + 8) * D + c) : 0u;
            qa[kt][2] = quad < G ? *reinterpret_cast<const uint32_t*>(q0 + quad * D + c + 8) : 0u;
            qa[kt][3] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (quad + 8) * D + c + 8) : 0u;
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};   // rows quad and quad + 8

    const uint32_t pipe = smem_u32(smem) + warp * (STAGES * 2 * PANEL_BYTES);
    auto issue = [&](int i) {
        if (i < count) {
            const int64_t base = (((int64_t)pages[pg_begin + i] * nkv + kvh) * PAGE + warp * KEYS_PER_WARP) * D;
            const uint32_t dst = pipe + (i % STAGES) * (2 * PANEL_BYTES);
            load_panel(dst, k_pages + base, lane);
            load_panel(dst + PANEL_BYTES, v_pages + base, lane);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);

    for (int i = 0; i < count; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        issue(i + STAGES - 1);      // its stage was consumed in iteration i - 1
        const uint32_t kbuf = pipe + (i % STAGES) * (2 * PANEL_BYTES), vbuf = kbuf + PANEL_BYTES;

        // scores of the group's rows against this warp's 16 keys
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int krow = (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            uint32_t b[4];
            ldmatrix_x4(b, kbuf + krow * ROW_BYTES + (2 * kt + ((lane >> 3) & 1)) * 16);
            mma_bf16(s[0], qa[kt], b[0], b[1]);
            mma_bf16(s[1], qa[kt], b[2], b[3]);
        }
        // mask keys outside [lo, pos]; key index of s[j][e]: page*64 + warp*16 + j*8 + tq*2 + (e & 1)
        const int key0 = (pg_begin + i) * PAGE + warp * KEYS_PER_WARP + tq * 2;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + j * 8 + (e & 1);
                const float v = (key >= lo && key <= pos) ? s[j][e] * scale_log2 : -INFINITY;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            m_use[r] = m_new == -INFINITY ? 0.0f : m_new;      // a row that has seen no key yet
            alpha[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
        }
        float sum[2] = {0.0f, 0.0f};
        uint32_t pa[4];
        {
            float p[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[j][e] = exp2f(s[j][e] - m_use[e >> 1]);
                    sum[e >> 1] += p[j][e];
                }
            pa[0] = pack_bf16(p[0][0], p[0][1]);
            pa[1] = pack_bf16(p[0][2], p[0][3]);
            pa[2] = pack_bf16(p[1][0], p[1][1]);
            pa[3] = pack_bf16(p[1][2], p[1][3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
            sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
            l_run[r] = l_run[r] * alpha[r] + sum[r];
        }
        // o = o * alpha + P . V over this warp's 16 keys
        const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vbuf + vrow * ROW_BYTES + (n + (lane >> 4)) * 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                o[n + h][0] *= alpha[0]; o[n + h][1] *= alpha[0];
                o[n + h][2] *= alpha[1]; o[n + h][3] *= alpha[1];
            }
            mma_bf16(o[n], pa, b[0], b[1]);
            mma_bf16(o[n + 1], pa, b[2], b[3]);
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();   // the cache has been read: the next kernel may start and fetch its weights
    __syncthreads();     // every warp is done with the pipeline buffers: reuse them for the merge

    // merge the four warps: sm_o[warp][row][D], sm_ml[warp][row][2]
    float* sm_o = reinterpret_cast<float*>(smem);
    float* sm_ml = sm_o + WARPS * 16 * D;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = quad + 8 * r;
        if (tq == 0) {
            sm_ml[(warp * 16 + row) * 2 + 0] = m_run[r];
            sm_ml[(warp * 16 + row) * 2 + 1] = l_run[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float2 v = make_float2(o[n][2 * r], o[n][2 * r + 1]);
            *reinterpret_cast<float2*>(sm_o + (warp * 16 + row) * D + n * 8 + tq * 2) = v;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
        const int row = idx / D, c = idx % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, sm_ml[(w * 16 + row) * 2]);
        float acc = 0.0f, l = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = sm_ml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            acc += f * sm_o[(w * 16 + row) * D + c];
            l += f * sm_ml[(w * 16 + row) * 2 + 1];
        }
        const int64_t slot = ((int64_t)t * nq + kvh * G + row) * n_splits + split;
        part_o[slot * D + c] = acc;
        if (c == 0) {
            part_ml[slot * 2 + 0] = m;
            part_ml[slot * 2 + 1] = l;
        }
    }
}

// One block per (head, token): out = sum_s w_s o_s / sum_s w_s l_s with w_s = 2^(m_s - max m).
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int nq, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = (int64_t)blockIdx.y * nq + blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.0f;
    for (int s = 0; s < n_splits; ++s) l += ml[2 * s] == -INFINITY ? 0.0f : exp2f(ml[2 * s] - m) * ml[2 * s + 1];
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float f = ml[2 * s] == -INFINITY ? 0.0f : exp2f(ml[2 * s] - m);
            acc += f * part_o[(row * n_splits + s) * D + c];
        }
        out[row * D + c] = __float2bfloat16_rn(acc / l);
    }
}

}  // namespace

// Scratch needed for `n_tokens` tokens, in float32 elements: sums then (max, sum) pairs.
Q3_EXPORT int64_t q3_attention_decode_scratch_floats(int64_t n_tokens, int nq, int n_splits) {
    return n_tokens * nq * n_splits * (D + 2);
}

Q3_EXPORT int q3_attention_decode_head_dim() { return D; }

Q3_EXPORT int q3_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                       float* scratch, const int* token_seq, const int* token_pos,
                                       const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv,
                                       float scale, int window, int n_splits, void* stream_) {
    if (n_tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || n_splits <= 0) return Q3_ERR_BAD_SIZE;
    if (n_tokens > 65535 || nkv > 65535) return Q3_ERR_TOO_LARGE;
    cudaStream_t stream = (cudaStream_t)stream_;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    float* part_o = scratch;
    float* part_ml = scratch + n_tokens * nq * n_splits * D;
    const dim3 grid(n_splits, nkv, (unsigned)n_tokens);
    cudaError_t e = q3_launch(decode_split_kernel, grid, dim3(WARPS * 32), SMEM_BYTES, stream, (const bf16*)q,
                              (const bf16*)k_pages, (const bf16*)v_pages, part_o, part_ml, token_seq, token_pos, page_table,
                              pages_per_seq, nq, nkv, scale * 1.4426950408889634f, window);
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(decode_merge_kernel, dim3(nq, (unsigned)n_tokens), dim3(D < 128 ? 32 : 128), 0, stream,
                          (const float*)part_o, (const float*)part_ml, (bf16*)out, nq, n_splits);
}
