// Causal grouped-query attention for prompts (bfloat16) over the paged cache: a tiled
// flash-attention kernel with the dots on the tensor cores.
//
// Replaces the reference's per-(token, head) block with a serial loop over all visible keys
// (src/ops/gqa_attention.cu:84-148), the dominant cost of its prefill.  Same math: causal
// by bound (key <= query position), score = q.k * d^-0.5, online softmax and weighted sum
// in 32-bit, probabilities never leave registers except rounded to bfloat16 as the
// operand of the P.V product.
//
// Grid (query tile, query head, sequence).  A block of four warps takes 64 consecutive new
// tokens of one sequence (16 rows a warp) and walks the sequence's pages from the first to
// the one that holds its last row; a page is the key tile (64 keys): its K and V panels
// of this head's kv group are contiguous and are double-buffered through cp.async.  The
// keys come from the cache, which already holds this step's own tokens, so a prompt that
// continues an earlier step (positions > 0) needs nothing special.  Sequences of unequal
// length share the grid: tiles beyond a sequence's new tokens exit at once.
// Compiled for one head size: -DQ3_HEAD_DIM=<multiple of 16>.
#include "common.cuh"

#ifndef Q3_HEAD_DIM
#error "compile with -DQ3_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = Q3_HEAD_DIM;
constexpr int PAGE = Q3_PAGE_TOKENS;
static_assert(PAGE == 64, "the tiled prompt attention takes one page of 64 keys per step");
constexpr int BM = 64;                              // query rows per block
constexpr int WARPS = 4;
constexpr int ROW_BYTES = D * 2 + 16;               // padded rows: conflict-free ldmatrix
constexpr int TILE_BYTES = PAGE * ROW_BYTES;
constexpr int CHUNKS_PER_ROW = D / 8;
constexpr int KT = D / 16, NT = D / 8;
constexpr int SMEM_BYTES = 2 * 2 * TILE_BYTES;      // two stages of (K, V)
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size: multiples of 16 up to 256");

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

__device__ __forceinline__ void load_tile(uint32_t dst, const bf16* src, int tid) {
#pragma unroll
    for (int i = tid; i < PAGE * CHUNKS_PER_ROW; i += WARPS * 32) {
        const int row = i / CHUNKS_PER_ROW, c = i % CHUNKS_PER_ROW;
        cp_async16(dst + row * ROW_BYTES + c * 16, src + row * D + c * 8);
    }
}

__global__ void __launch_bounds__(WARPS * 32)
prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
               bf16* __restrict__ out, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
               const int* __restrict__ page_table, int pages_per_seq, int nq, int nkv, float scale_log2, int window) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int t0 = seq_start[seq], n_new = seq_start[seq + 1] - t0;
    if (tile * BM >= n_new) return;
    const int kvh = head / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
    const int pos0 = seq_pos0[seq];
    const int* pages = page_table + (int64_t)seq * pages_per_seq;

    // this warp's 16 rows; rows beyond the sequence's new tokens are computed on row 0's data and dropped
    const int r_lo = tile * BM + warp * 16 + quad, r_hi = r_lo + 8;           // rows within the step
    const bool ok_lo = r_lo < n_new, ok_hi = r_hi < n_new;
    const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;                          // absolute positions
    uint32_t qa[KT][4];
    {
        const bf16* q_lo = q + ((int64_t)(t0 + (ok_lo ? r_lo : 0)) * nq + head) * D;
        const bf16* q_hi = q + ((int64_t)(t0 + (ok_hi ? r_hi : 0)) * nq + head) * D;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            const int c = kt * 16 + tq * 2;
            qa[kt][0] = *reinterpret_cast<const uint32_t*>(q_lo + c);
            qa[kt][1] = *reinterpret_cast<const uint32_t*>(q_hi + c);
            qa[kt][2] = *reinterpret_cast<const uint32_t*>(q_lo + c + 8);
            qa[kt][3] = *reinterpret_cast<const uint32_t*>(q_hi + c + 8);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    const int last_row = min(tile * BM + BM, n_new) - 1;
    const int first_key = window > 0 ? max(0, pos0 + tile * BM - window + 1) : 0;
    const int pg_begin = first_key / PAGE, pg_end = (pos0 + last_row) / PAGE + 1;
    const int warp_first_pos = pos0 + tile * BM + warp * 16;                   // lowest position of the warp's rows
    const uint32_t base = smem_u32(smem);

    auto issue = [&](int pg) {
        if (pg < pg_end) {
            const int64_t off = ((int64_t)pages[pg] * nkv + kvh) * PAGE * D;
            const uint32_t dst = base + ((pg - pg_begin) & 1) * (2 * TILE_BYTES);
            load_tile(dst, k_pages + off, threadIdx.x);
            load_tile(dst + TILE_BYTES, v_pages + off, threadIdx.x);
        }
        cp_async_commit();
    };
    issue(pg_begin);
    for (int pg = pg_begin; pg < pg_end; ++pg) {
        issue(pg + 1);              // into the other stage, which every warp left before the last barrier
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kbuf = base + ((pg - pg_begin) & 1) * (2 * TILE_BYTES), vbuf = kbuf + TILE_BYTES;
        const int key_base = pg * PAGE;
        // a warp whose rows all lie before this page has nothing to see in it
        if (key_base <= warp_first_pos + 15) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
            const int krow = (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
            for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {       // pairs of 8-key tiles
                    uint32_t b[4];
                    ldmatrix_x4(b, kbuf + (jp * 16 + krow) * ROW_BYTES + (2 * kt + ((lane >> 3) & 1)) * 16);
                    mma_bf16(s[2 * jp], qa[kt], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], qa[kt], b[2], b[3]);
                }
            }
            const bool edge = key_base + PAGE - 1 > warp_first_pos || window > 0;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[j][e] * scale_log2;
                    if (edge) {
                        const int key = key_base + j * 8 + tq * 2 + (e & 1);
                        const int p = (e >> 1) ? p_hi : p_lo;
                        const bool seen = key <= p && (window <= 0 || key > p - window);
                        v = seen ? v : -INFINITY;
                    }
                    s[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], m_use[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                m_use[r] = m_new == -INFINITY ? 0.0f : m_new;
                alpha[r] = exp2f(m_run[r] - m_use[r]);
                m_run[r] = m_new;
            }
            float sum[2] = {0.0f, 0.0f};
            uint32_t pa[4][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
                const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
                sum[0] += p0 + p1;
                sum[1] += p2 + p3;
                pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                l_run[r] = l_run[r] * alpha[r] + sum[r];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {            // 16 keys at a time
#pragma unroll
                for (int n = 0; n < NT; n += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vbuf + (kk * 16 + vrow) * ROW_BYTES + (n + (lane >> 4)) * 16);
                    mma_bf16(o[n], pa[kk], b[0], b[1]);
                    mma_bf16(o[n + 1], pa[kk], b[2], b[3]);
                }
            }
        }
        __syncthreads();            // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();

    const float inv_lo = 1.0f / l_run[0], inv_hi = 1.0f / l_run[1];
    bf16* o_lo = out + ((int64_t)(t0 + r_lo) * nq + head) * D;
    bf16* o_hi = out + ((int64_t)(t0 + r_hi) * nq + head) * D;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int c = n * 8 + tq * 2;
        if (ok_lo) *reinterpret_cast<uint32_t*>(o_lo + c) = pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
        if (ok_hi) *reinterpret_cast<uint32_t*>(o_hi + c) = pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
}

}  // namespace

Q3_EXPORT int q3_attention_prefill_head_dim() { return D; }

Q3_EXPORT int q3_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                        const int* seq_start, const int* seq_pos0, const int* page_table,
                                        int pages_per_seq, int n_seqs, int max_new, int nq, int nkv, float scale,
                                        int window, void* stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) return Q3_ERR_BAD_SIZE;
    if (n_seqs > 65535 || nq > 65535) return Q3_ERR_TOO_LARGE;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(prefill_kernel, SMEM_BYTES, configured);
        if (e != cudaSuccess) return (int)e;
    }
    const dim3 grid((max_new + BM - 1) / BM, nq, n_seqs);
    return (int)q3_launch(prefill_kernel, grid, dim3(WARPS * 32), SMEM_BYTES, (cudaStream_t)stream, (const bf16*)q,
                          (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, seq_start, seq_pos0, page_table,
                          pages_per_seq, nq, nkv, scale * 1.4426950408889634f, window);
}
