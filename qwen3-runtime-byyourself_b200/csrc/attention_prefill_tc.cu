// Causal grouped-query attention for prompts on the 5th-generation tensor cores (bfloat16):
// S = Q.K^T and O += P.V are tcgen05.mma with the accumulators in tensor memory; Q, K and V
// tiles arrive by TMA straight from the packed query buffer and from the cache pages.
//
// Same math as the reference's kernel (src/ops/gqa_attention.cu:84-153: causal by bound, scale
// after the dot, online softmax and weighted sum in 32-bit), arranged for Blackwell:
//   grid (tile of 128 new tokens, query head, sequence); three roles per block
//   warp 0     TMA: the Q tile once, then the K panels of the cache pages (64 keys of the head's kv
//              group, two 64-column halves at head size 128) into a ring of three
//   warp 6     TMA: the V panels into a ring of two.  K(j) is free again as soon as S(j) is done and
//              V(j) only after O += P(j).V(j), so with rings of their own the K loads run two pages
//              ahead of the products, which covers their latency at two blocks per SM
//   warp 1     one thread issues the products: S(j) = Q.K_j^T into TMEM columns [0,64), then
//              O += P_j.V_j with P read from TMEM and V as an MN-major shared-memory operand;
//              S(j+1) is issued as soon as the softmax warps have read S(j)
//   warps 2-5  softmax: thread r owns query row r (TMEM lane r): loads its 64 scores, masks the
//              diagonal page, keeps a running maximum that is only raised when the new maximum
//              exceeds it by more than 2^8 (the accumulator is then rescaled in TMEM), writes
//              P as packed bfloat16 into TMEM columns [64,96), and at the end normalises O
// Every mbarrier wait is bounded and reports into `status`.  Head sizes 64 and 128, no window;
// other shapes use the mma.sync kernel of attention_prefill.cu.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

#ifndef Q3_HEAD_DIM
#error "compile with -DQ3_HEAD_DIM=<64 or 128>"
#endif

namespace {

constexpr int D = Q3_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention takes head sizes 64 and 128");
constexpr int PAGE = Q3_PAGE_TOKENS, BM = 128, HALVES = D / 64;
static_assert(PAGE == 64, "the tcgen05 prompt attention takes one page of 64 keys per product");
constexpr int THREADS = 224;
constexpr int K_STAGES = 3, V_STAGES = 2;                // pages of K and of V in flight or in use
constexpr int Q_BYTES = HALVES * BM * 128;               // 128 rows x 128 bytes per half
constexpr int PANEL_BYTES = HALVES * PAGE * 128;         // one page of K (or V): 64 keys x 128 bytes per half
// no slack for alignment: two blocks of head size 128 have to fit one SM, and the dynamic shared memory of
// a kernel without static shared memory starts at a 1024-byte boundary (checked when the kernel starts)
constexpr int SMEM_BYTES = Q_BYTES + (K_STAGES + V_STAGES) * PANEL_BYTES + 256;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_S = 0, COL_P = 64, COL_O = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;                // in log2 units: probabilities stay below 2^8

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 operands; bit 16 = B is MN-major.
constexpr uint32_t idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// 2^x by the special-function unit alone (-inf gives 0).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two floats in one 64-bit register, and the arithmetic of this architecture that takes both at once.
__device__ __forceinline__ uint64_t pack_f32x2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, const int* __restrict__ seq_start,
                  const int* __restrict__ seq_pos0, const int* __restrict__ page_table, int pages_per_seq, int n_seqs,
                  int n_tiles, int nq, int nkv, float scale_log2, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    // Blocks start in the order of their index, so the index runs over the tiles from last to first, and for
    // each tile over every sequence and head: the tiles that see the most keys start first on all SMs, and
    // the short ones fill the gaps at the end (with the heads of one sequence side by side, the last heads'
    // long tiles would start when the GPU is nearly done).
    const int tile = n_tiles - 1 - (int)(blockIdx.x / (unsigned)(n_seqs * nq));
    const int seq = (int)(blockIdx.x / (unsigned)nq) % n_seqs, head = (int)(blockIdx.x % (unsigned)nq);
    const int t0 = seq_start[seq], n_new = seq_start[seq + 1] - t0;
    if (tile * BM >= n_new) return;
    const int kvh = head / (nq / nkv);
    const int pos0 = seq_pos0[seq];
    const int* pages = page_table + (int64_t)seq * pages_per_seq;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = min(BM, n_new - tile * BM);
    const int n_pages = (pos0 + tile * BM + rows - 1) / PAGE + 1;        // pages 0 .. the one of the last row

    const uint32_t base = smem_u32(smem_raw);
    if (base & 1023u) {                                  // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicExch(status, 18);
        return;
    }
    const uint32_t q_smem = base, k_smem = base + Q_BYTES, v_smem = k_smem + K_STAGES * PANEL_BYTES;
    const uint32_t bars = v_smem + V_STAGES * PANEL_BYTES;
    const uint32_t bar_q = bars, bar_k_full = bars + 8, bar_k_empty = bar_k_full + 8 * K_STAGES;
    const uint32_t bar_v_full = bar_k_empty + 8 * K_STAGES, bar_v_empty = bar_v_full + 8 * V_STAGES;
    const uint32_t bar_s_full = bar_v_empty + 8 * V_STAGES, bar_s_read = bar_s_full + 8, bar_p_full = bar_s_read + 8;
    const uint32_t bar_pv_done = bar_p_full + 8, tmem_slot = bar_pv_done + 8;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int s = 0; s < K_STAGES; ++s) {
            mbar_init(bar_k_full + 8 * s, 1);
            mbar_init(bar_k_empty + 8 * s, 1);
        }
        for (int s = 0; s < V_STAGES; ++s) {
            mbar_init(bar_v_full + 8 * s, 1);
            mbar_init(bar_v_empty + 8 * s, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_read, 4);
        mbar_init(bar_p_full, 4);
        mbar_init(bar_pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot) : "memory");

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: Q, then the K panels
        if (lane == 0) {
            mbar_expect_tx(bar_q, Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma_load_2d(q_smem + h * BM * 128, &map_q, bar_q, head * D + h * 64, t0 + tile * BM);
            for (int j = 0; j < n_pages; ++j) {
                const int s = j % K_STAGES;
                if (!mbar_wait(bar_k_empty + 8 * s, ((uint32_t)(j / K_STAGES) & 1u) ^ 1u)) { atomicExch(status, 11); break; }
                const uint32_t dst = k_smem + s * PANEL_BYTES;
                const int row = (pages[j] * nkv + kvh) * PAGE;
                mbar_expect_tx(bar_k_full + 8 * s, PANEL_BYTES);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * PAGE * 128, &map_k, bar_k_full + 8 * s, h * 64, row);
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------ TMA producer: the V panels
        if (lane == 0) {
            for (int j = 0; j < n_pages; ++j) {
                const int s = j % V_STAGES;
                if (!mbar_wait(bar_v_empty + 8 * s, ((uint32_t)(j / V_STAGES) & 1u) ^ 1u)) { atomicExch(status, 19); break; }
                const uint32_t dst = v_smem + s * PANEL_BYTES;
                const int row = (pages[j] * nkv + kvh) * PAGE;
                mbar_expect_tx(bar_v_full + 8 * s, PANEL_BYTES);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_2d(dst + h * PAGE * 128, &map_v, bar_v_full + 8 * s, h * 64, row);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc(BM, PAGE, false), idesc_pv = idesc(BM, D, true);
            auto issue_s = [&](int j) {
                const uint32_t k_src = k_smem + (j % K_STAGES) * PANEL_BYTES;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * (BM * 128) + (kk & 3) * 32, koff = (kk >> 2) * (PAGE * 128) + (kk & 3) * 32;
                    tc_mma_ss(tmem + COL_S, desc_k_major(q_smem + off), desc_k_major(k_src + koff), idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full);
                tc_commit(bar_k_empty + 8 * (j % K_STAGES));                 // the page's K is consumed
            };
            bool ok = mbar_wait(bar_q, 0) && mbar_wait(bar_k_full, 0);
            if (!ok) atomicExch(status, 12);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < n_pages && ok; ++j) {
                // S(j+1) may overwrite the score columns once the softmax warps hold S(j) in registers
                if (j + 1 < n_pages) {
                    ok = mbar_wait(bar_s_read, (uint32_t)j & 1u) &&
                         mbar_wait(bar_k_full + 8 * ((j + 1) % K_STAGES), (uint32_t)((j + 1) / K_STAGES) & 1u);
                    if (!ok) { atomicExch(status, 13); break; }
                    tc_fence_after();
                    issue_s(j + 1);
                }
                ok = mbar_wait(bar_p_full, (uint32_t)j & 1u) &&              // P(j) is in TMEM, O is rescaled
                     mbar_wait(bar_v_full + 8 * (j % V_STAGES), (uint32_t)(j / V_STAGES) & 1u);
                if (!ok) { atomicExch(status, 14); break; }
                tc_fence_after();
                const uint32_t v_src = v_smem + (j % V_STAGES) * PANEL_BYTES;
#pragma unroll
                for (int kk = 0; kk < PAGE / 16; ++kk)
                    tc_mma_ts(tmem + COL_O, tmem + COL_P + kk * 8, desc_mn_major(v_src + kk * 16 * 128, PAGE * 128), idesc_pv,
                              (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(bar_v_empty + 8 * (j % V_STAGES));                 // the page's V is consumed
                tc_commit(bar_pv_done);
            }
        }
    } else {
        // ------------------------------------------------ softmax and epilogue: thread = query row
        const int lane_base = (warp & 3) * 32;
        const int r = lane_base + lane;                                     // row of the tile
        const int p_row = pos0 + tile * BM + r;                             // its absolute position
        const uint32_t t_row = tmem + ((uint32_t)lane_base << 16);
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_pages && ok; ++j) {
            ok = mbar_wait(bar_s_full, (uint32_t)j & 1u);
            if (!ok) { if (lane == 0) atomicExch(status, 15); break; }
            tc_fence_after();
            uint32_t s[64];
            tc_ld32(t_row + COL_S, s);
            tc_ld32(t_row + COL_S + 32, s + 32);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_read);
            const int key0 = j * PAGE;
            const bool edge = key0 + PAGE - 1 > pos0 + tile * BM;           // some key of the page lies after some row
            if (edge) {
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (key0 + c > p_row) s[c] = 0xff800000u;                // -inf
            }
            // the page's maximum on the raw dots (the scale is positive), four chains side by side
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; c += 8) {                               // two scores per instruction and chain
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e] = max3(mx[e], __uint_as_float(s[c + e]), __uint_as_float(s[c + 4 + e]));
            }
            const float m_page = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
            float alpha = 1.0f;
            bool raise = false;
            if (j == 0) {
                m_run = m_page == -INFINITY ? 0.0f : m_page;                 // the first page overwrites O: nothing to rescale
            } else if (m_page > m_run + RESCALE_THRESHOLD) {
                alpha = ex2_approx(m_run - m_page);
                m_run = m_page;
                raise = true;
            }
            // p = 2^(dot * scale - m): one multiply-add and one ex2 per score, four sums side by side
            const float neg_m = -m_run;
            // (the multiply-adds and the sums take two scores an instruction: fma.rn.f32x2, add.f32x2)
            const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(neg_m, neg_m);
            uint64_t part2[2] = {pack_f32x2(0.0f, 0.0f), pack_f32x2(0.0f, 0.0f)};
            uint32_t p[32];
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                float x0, x1, x2, x3;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), scale2, neg_m2), x0, x1);
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])), scale2, neg_m2), x2, x3);
                const float a = ex2_approx(x0), b = ex2_approx(x1), e = ex2_approx(x2), f = ex2_approx(x3);
                part2[0] = add_f32x2(part2[0], pack_f32x2(a, b));
                part2[1] = add_f32x2(part2[1], pack_f32x2(e, f));
                p[c >> 1] = pack_bf16(a, b);
                p[(c >> 1) + 1] = pack_bf16(e, f);
            }
            float part[4];
            unpack_f32x2(part2[0], part[0], part[1]);
            unpack_f32x2(part2[1], part[2], part[3]);
            const float sum = (part[0] + part[1]) + (part[2] + part[3]);
            l_run = l_run * alpha + sum;
            if (j > 0) {
                ok = mbar_wait(bar_pv_done, (uint32_t)(j - 1) & 1u);         // O and the P columns are free again
                if (!ok) { if (lane == 0) atomicExch(status, 16); break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, raise)) {                        // the loads and stores are warp-wide
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tc_ld32(t_row + COL_O + c, o);
                        tc_wait_ld();
                        const uint64_t alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll
                        for (int e = 0; e < 32; e += 2) {
                            float x, y;
                            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(o[e]), __uint_as_float(o[e + 1])), alpha2), x, y);
                            o[e] = __float_as_uint(x);
                            o[e + 1] = __float_as_uint(y);
                        }
                        tc_st32(t_row + COL_O + c, o);
                    }
                }
            }
            tc_st32(t_row + COL_P, p);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full);
        }
        if (ok) {
            ok = mbar_wait(bar_pv_done, (uint32_t)(n_pages - 1) & 1u);
            if (!ok && lane == 0) atomicExch(status, 17);
        }
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            bf16* dst = out + ((int64_t)(t0 + tile * BM + r) * nq + head) * D;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t o[32];
                tc_ld32(t_row + COL_O + c, o);
                tc_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + e) = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

Q3_EXPORT int q3_attention_prefill_tc_head_dim() { return D; }

// q: [n_tokens, nq * D]; k_pages, v_pages: [n_cache_pages, nkv, 64, D]; out: [n_tokens, nq * D].
Q3_EXPORT int q3_attention_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                           const int* seq_start, const int* seq_pos0, const int* page_table,
                                           int pages_per_seq, int n_seqs, int max_new, int64_t n_tokens,
                                           int64_t n_cache_pages, int nq, int nkv, float scale, int* status, void* stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || !(scale > 0.0f)) return Q3_ERR_BAD_SIZE;   // the row maximum is taken before scaling
    if (n_seqs > 65535 || nq > 65535) return Q3_ERR_TOO_LARGE;
    if (!aligned16(q) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(out)) return Q3_ERR_MISALIGNED;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(prefill_tc_kernel, SMEM_BYTES, configured);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap map_q, map_k, map_v;
    if (!q3_make_map_bf16(&map_q, q, n_tokens, (int64_t)nq * D, BM, 64, true) || !q3_make_map_bf16(&map_k, k_pages, n_cache_pages * nkv * PAGE, D, PAGE, 64, true) ||
        !q3_make_map_bf16(&map_v, v_pages, n_cache_pages * nkv * PAGE, D, PAGE, 64, true))
        return Q3_ERR_BAD_SIZE;
    const int n_tiles = (max_new + BM - 1) / BM;
    const int64_t blocks = (int64_t)n_tiles * n_seqs * nq;
    if (blocks > 0x7fffffff) return Q3_ERR_TOO_LARGE;
    return (int)q3_launch(prefill_tc_kernel, dim3((unsigned)blocks), dim3(THREADS), (size_t)SMEM_BYTES, (cudaStream_t)stream, map_q,
                          map_k, map_v, (bf16*)out, seq_start, seq_pos0, page_table, pages_per_seq, n_seqs, n_tiles, nq, nkv,
                          scale * 1.4426950408889634f, status);
}
