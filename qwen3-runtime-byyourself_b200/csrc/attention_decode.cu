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
//
// The fused form does the whole attention of a decode step in one launch: it takes the output of
// the q/k/v projection as it is, normalises and rotates the group's query heads itself (what
// qkv_prepare does, src/model/self_attention.cpp:147-152), the block that owns the sequence's last
// page does the same for the new key, writes key and value into the cache and puts them into its own
// copy of the page, and the splits of a (sequence, kv head) form a thread-block cluster that merges
// its partial results through distributed shared memory: no scratch buffer, no second and third kernel.
#include "common.cuh"

#ifndef Q3_HEAD_DIM
#error "compile with -DQ3_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = Q3_HEAD_DIM;
constexpr int PAGE = Q3_PAGE_TOKENS;
static_assert(PAGE == 64, "the decode attention gives each of its four warps 16 keys of a page");
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
// the fused form keeps, behind the pipeline: first the prepared queries [16][D] and the new key and value
// (bf16), later - in the same place - the block's merged result [16][D] float32 and its (max, sum) pairs
constexpr int SMEM_PREP = (16 + 2) * D * 2;
constexpr int SMEM_RESULT = 16 * (D + 2) * 4;
constexpr int SMEM_FUSED = SMEM_BYTES + (SMEM_PREP > SMEM_RESULT ? SMEM_PREP : SMEM_RESULT);
constexpr int MAX_CLUSTER = 16;                    // the fused form takes up to 16 splits (above 8 the cluster size is the
                                                   // device's non-portable one, asked for at the launch)

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

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
    uint32_t addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// One head vector of the projection output, normalised (if `norm_w`) and rotated (if `cos_tab`), by one warp:
// the first `rot` values are rotated in pairs (i, i + rot/2), i = lane + 32 n, the values from `rot` on (none when
// the whole head is rotated) pass through - exactly as qkv_prepare does (attention.cu), so the values are the same
// to the bit.  dst: D bf16.
__device__ __forceinline__ void prepare_head(const bf16* __restrict__ src, bf16* dst, const float* __restrict__ norm_w,
                                             const float* __restrict__ cos_tab, const float* __restrict__ sin_tab, int pos,
                                             float eps, int rot, int lane) {
    constexpr int ITER = (D / 2 + 31) / 32, REST = (D + 31) / 32;
    const int rhalf = rot >> 1;
    float a[ITER], b[ITER], wa[ITER], wb[ITER], cs[ITER], sn[ITER], c[REST], wc[REST];
    // every load first (they do not depend on one another), then the arithmetic
#pragma unroll
    for (int n = 0; n < ITER; ++n) {
        const int i = lane + 32 * n;
        a[n] = b[n] = 0.0f;
        wa[n] = wb[n] = cs[n] = 1.0f;
        sn[n] = 0.0f;
        if (i < rhalf) {
            a[n] = __bfloat162float(src[i]);
            b[n] = __bfloat162float(src[i + rhalf]);
            if (norm_w != nullptr) {
                wa[n] = norm_w[i];
                wb[n] = norm_w[i + rhalf];
            }
            if (cos_tab != nullptr) {
                cs[n] = cos_tab[(int64_t)pos * rhalf + i];
                sn[n] = sin_tab[(int64_t)pos * rhalf + i];
            }
        }
    }
    if (rot < D) {
#pragma unroll
        for (int n = 0; n < REST; ++n) {
            const int i = rot + lane + 32 * n;
            c[n] = 0.0f;
            wc[n] = 1.0f;
            if (i < D) {
                c[n] = __bfloat162float(src[i]);
                if (norm_w != nullptr) wc[n] = norm_w[i];
            }
        }
    }
    float sq = 0.0f;
#pragma unroll
    for (int n = 0; n < ITER; ++n) sq += a[n] * a[n] + b[n] * b[n];      // lanes beyond the head add zeros
    if (rot < D) {
#pragma unroll
        for (int n = 0; n < REST; ++n) sq += c[n] * c[n];
    }
    if (norm_w != nullptr) {
        const float inv = rsqrtf(warp_sum(sq) / (float)D + eps);
#pragma unroll
        for (int n = 0; n < ITER; ++n) {
            a[n] = round_to<bf16>(round_to<bf16>(a[n] * inv) * wa[n]);
            b[n] = round_to<bf16>(round_to<bf16>(b[n] * inv) * wb[n]);
        }
        if (rot < D) {
#pragma unroll
            for (int n = 0; n < REST; ++n) c[n] = round_to<bf16>(round_to<bf16>(c[n] * inv) * wc[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < ITER; ++n) {
        const int i = lane + 32 * n;
        if (i < rhalf) {
            float x = a[n], y = b[n];
            if (cos_tab != nullptr) {
                x = a[n] * cs[n] - b[n] * sn[n];
                y = b[n] * cs[n] + a[n] * sn[n];
            }
            dst[i] = __float2bfloat16_rn(x);
            dst[i + rhalf] = __float2bfloat16_rn(y);
        }
    }
    if (rot < D) {
#pragma unroll
        for (int n = 0; n < REST; ++n) {
            const int i = rot + lane + 32 * n;
            if (i < D) dst[i] = __float2bfloat16_rn(c[n]);
        }
    }
}

// What the fused form needs beyond the split form's arguments.
struct FusedArgs {
    const bf16* qkv;               // [tokens, (nq + 2 nkv) * D]: the projection output as it is
    bf16* out;                     // [tokens, nq * D]
    const float* q_norm_w;         // [D] or null
    const float* k_norm_w;
    const float* cos_tab;          // [positions, D/2] or null
    const float* sin_tab;
    float eps;
    int rot;                       // the first `rot` values of a head are rotated (the head size: all of them)
    int write_kv;                  // 0: the layer reads another layer's cache, which holds the new key and value already
};

// Copies one warp's panel (16 keys x D) of a page into padded shared rows.
__device__ __forceinline__ void load_panel(uint32_t dst, const bf16* src, int lane) {
#pragma unroll
    for (int i = lane; i < KEYS_PER_WARP * CHUNKS_PER_ROW; i += 32) {
        const int row = i / CHUNKS_PER_ROW, c = i % CHUNKS_PER_ROW;
        cp_async16(dst + row * ROW_BYTES + c * 16, src + row * D + c * 8);
    }
}

// part_o: [tokens, nq, splits, D] float32 (unnormalised sums); part_ml: [tokens, nq, splits, 2] (max, sum).
// FUSED: `q`, `part_o` and `part_ml` are unused; the grid's x dimension is a cluster.
template <bool FUSED>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(const bf16* __restrict__ q, const bf16* k_pages, const bf16* v_pages,
                    float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ token_seq,
                    const int* __restrict__ token_pos, const int* __restrict__ page_table, int pages_per_seq, int nq,
                    int nkv, float scale_log2, int window, const FusedArgs fused) {
    extern __shared__ __align__(16) unsigned char smem[];
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

    // the first pages are asked for before anything else: what follows runs under their flight
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
    // the pages and the step's positions do not depend on the kernel before this one (the new token's key and
    // value are this kernel's own to write); its output - the projections - is read from here on
    pdl_wait();

    // the block that holds the sequence's last page owns the new token's key and value
    const bool owner = FUSED && fused.write_kv && count > 0 && pg_end == first_page + n_pages;
    bf16* prep = reinterpret_cast<bf16*>(smem + SMEM_BYTES);            // [16][D] queries, then the new key, then the new value
    if constexpr (FUSED) {
        const bf16* row = fused.qkv + (int64_t)t * (nq + 2 * nkv) * D;
        for (int r = warp; r < G; r += WARPS)
            prepare_head(row + (int64_t)(kvh * G + r) * D, prep + r * D, fused.q_norm_w, fused.cos_tab, fused.sin_tab, pos,
                         fused.eps, fused.rot, lane);
        if (owner) {
            if (warp == (G % WARPS))
                prepare_head(row + (int64_t)(nq + kvh) * D, prep + 16 * D, fused.k_norm_w, fused.cos_tab, fused.sin_tab, pos,
                             fused.eps, fused.rot, lane);
            if (warp == ((G + 1) % WARPS))
                for (int i = lane; i < D; i += 32) prep[17 * D + i] = row[(int64_t)(nq + nkv + kvh) * D + i];
        }
        __syncthreads();
        if (owner) {       // into the cache for the steps to come; this step reads them from `prep`
            const int64_t at = (((int64_t)pages[pos / PAGE] * nkv + kvh) * PAGE + pos % PAGE) * D;
            for (int i = threadIdx.x; i < D; i += WARPS * 32) {
                const_cast<bf16*>(k_pages)[at + i] = prep[16 * D + i];
                const_cast<bf16*>(v_pages)[at + i] = prep[17 * D + i];
            }
        }
    }
    // query rows of the group as A fragments: row r = head kvh*G + r (rows >= G are zero)
    uint32_t qa[KT][4];
    {
        const bf16* q0 = FUSED ? prep : q + ((int64_t)t * nq + (int64_t)kvh * G) * D;
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

    for (int i = 0; i < count; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        issue(i + STAGES - 1);      // its stage was consumed in iteration i - 1
        const uint32_t kbuf = pipe + (i % STAGES) * (2 * PANEL_BYTES), vbuf = kbuf + PANEL_BYTES;
        if constexpr (FUSED) {
            // the new token's own key and value: not in the cache when this page was asked for
            if (owner && i == count - 1 && (pos % PAGE) / KEYS_PER_WARP == warp) {
                unsigned char* stage = smem + warp * (STAGES * 2 * PANEL_BYTES) + (i % STAGES) * (2 * PANEL_BYTES);
                const int key_row = (pos % PAGE) % KEYS_PER_WARP;
                for (int c = lane; c < D / 8; c += 32) {
                    *reinterpret_cast<uint4*>(stage + key_row * ROW_BYTES + c * 16) = *reinterpret_cast<const uint4*>(prep + 16 * D + c * 8);
                    *reinterpret_cast<uint4*>(stage + PANEL_BYTES + key_row * ROW_BYTES + c * 16) =
                        *reinterpret_cast<const uint4*>(prep + 17 * D + c * 8);
                }
                __syncwarp();
            }
        }

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
    float* res_o = reinterpret_cast<float*>(smem + SMEM_BYTES);         // FUSED: [16][D], then (max, sum) [16][2]
    float* res_ml = res_o + 16 * D;
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
        if constexpr (FUSED) {
            res_o[row * D + c] = acc;
            if (c == 0) {
                res_ml[row * 2 + 0] = m;
                res_ml[row * 2 + 1] = l;
            }
        } else {
            const int64_t slot = ((int64_t)t * nq + kvh * G + row) * n_splits + split;
            part_o[slot * D + c] = acc;
            if (c == 0) {
                part_ml[slot * 2 + 0] = m;
                part_ml[slot * 2 + 1] = l;
            }
        }
    }
    if constexpr (FUSED) {
        // the splits of this (sequence, kv head) are the blocks of one cluster: each finishes a share of the
        // group's values from everybody's partial results, in split order (the order of the merge kernel)
        cluster_sync_all();
        for (int idx = threadIdx.x * n_splits + split; idx < G * D; idx += WARPS * 32 * n_splits) {
            const int row = idx / D, c = idx % D;
            float ms[MAX_CLUSTER], ls[MAX_CLUSTER], os[MAX_CLUSTER];
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; ++s2) {               // every peer's values first, then the arithmetic
                ms[s2] = -INFINITY;
                ls[s2] = os[s2] = 0.0f;
                if (s2 < n_splits) {
                    ms[s2] = ld_peer_f32(res_ml + row * 2, s2);
                    ls[s2] = ld_peer_f32(res_ml + row * 2 + 1, s2);
                    os[s2] = ld_peer_f32(res_o + row * D + c, s2);
                }
            }
            float m = -INFINITY;
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; ++s2) m = fmaxf(m, ms[s2]);
            float l = 0.0f, acc = 0.0f;
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; ++s2)
                if (s2 < n_splits) l += ms[s2] == -INFINITY ? 0.0f : exp2f(ms[s2] - m) * ls[s2];
#pragma unroll
            for (int s2 = 0; s2 < MAX_CLUSTER; ++s2)
                if (s2 < n_splits) acc += (ms[s2] == -INFINITY ? 0.0f : exp2f(ms[s2] - m)) * os[s2];
            fused.out[((int64_t)t * nq + kvh * G + row) * D + c] = __float2bfloat16_rn(acc / l);
        }
        cluster_sync_all();      // nobody leaves while its results are still being read
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
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(decode_split_kernel<false>, SMEM_BYTES, configured);
        if (e != cudaSuccess) return (int)e;
    }
    float* part_o = scratch;
    float* part_ml = scratch + n_tokens * nq * n_splits * D;
    const dim3 grid(n_splits, nkv, (unsigned)n_tokens);
    cudaError_t e = q3_launch(decode_split_kernel<false>, grid, dim3(WARPS * 32), SMEM_BYTES, stream, (const bf16*)q,
                              (const bf16*)k_pages, (const bf16*)v_pages, part_o, part_ml, token_seq, token_pos, page_table,
                              pages_per_seq, nq, nkv, scale * 1.4426950408889634f, window, FusedArgs{});
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(decode_merge_kernel, dim3(nq, (unsigned)n_tokens), dim3(D < 128 ? 32 : 128), 0, stream,
                          (const float*)part_o, (const float*)part_ml, (bf16*)out, nq, n_splits);
}

// The most key splits (blocks of a cluster) the one-launch form can take on the current device: 16 where a cluster of
// that size can be placed (it is beyond the portable size), else 8.
Q3_EXPORT int q3_attention_decode_fused_max_splits() {
    static int cached[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 8;
    if (cached[device] == 0) {
        cached[device] = 8;
        static Q3PerDevice configured;
        if (q3_allow_shared_memory(decode_split_kernel<true>, SMEM_FUSED, configured) == cudaSuccess &&
            cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(MAX_CLUSTER, 8, 1);
            cfg.blockDim = dim3(WARPS * 32);
            cfg.dynamicSmemBytes = SMEM_FUSED;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = MAX_CLUSTER;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, decode_split_kernel<true>, &cfg) == cudaSuccess && clusters > 0)
                cached[device] = MAX_CLUSTER;
        }
        cudaGetLastError();        // a refusal above is an answer, not an error to keep
    }
    return cached[device];
}

// The whole attention of a decode step in one launch (see the top of the file): `qkv` is the projection output
// [tokens, (nq + 2 nkv) * head size]; norm weights and rotation tables ([positions, rotary_dim / 2]) may be null;
// `rotary_dim` 0 = the head size; `n_splits` <= 16.
Q3_EXPORT int q3_attention_decode_fused_bf16(const void* qkv, void* k_pages, void* v_pages, void* out, const float* q_norm_w,
                                             const float* k_norm_w, const float* cos_tab, const float* sin_tab, float eps,
                                             const int* token_seq, const int* token_pos, const int* page_table,
                                             int pages_per_seq, int64_t n_tokens, int nq, int nkv, float scale, int window,
                                             int n_splits, int write_kv, int rotary_dim, void* stream_) {
    if (n_tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || n_splits <= 0 || n_splits > MAX_CLUSTER) return Q3_ERR_BAD_SIZE;
    if ((cos_tab == nullptr) != (sin_tab == nullptr)) return Q3_ERR_BAD_SIZE;
    if (rotary_dim <= 0) rotary_dim = D;
    if (rotary_dim % 2 != 0 || rotary_dim > D) return Q3_ERR_BAD_SIZE;
    if (n_tokens > 65535 || nkv > 65535) return Q3_ERR_TOO_LARGE;
    if (!aligned16(qkv) || !aligned16(k_pages) || !aligned16(v_pages)) return Q3_ERR_MISALIGNED;
    cudaStream_t stream = (cudaStream_t)stream_;
    static Q3PerDevice configured, configured_large;
    cudaError_t e = q3_allow_shared_memory(decode_split_kernel<true>, SMEM_FUSED, configured);
    if (e != cudaSuccess) return (int)e;
    if (n_splits > 8) {                                     // one sequence, or two, with a long context: clusters of up to 16
        int device = 0;
        if ((e = cudaGetDevice(&device)) != cudaSuccess) return (int)e;
        if (device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
        if (!configured_large.done[device]) {
            e = cudaFuncSetAttribute(decode_split_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return (int)e;
            configured_large.done[device] = true;
        }
    }
    FusedArgs fused;
    fused.qkv = (const bf16*)qkv;
    fused.out = (bf16*)out;
    fused.q_norm_w = q_norm_w;
    fused.k_norm_w = k_norm_w;
    fused.cos_tab = cos_tab;
    fused.sin_tab = sin_tab;
    fused.eps = eps;
    fused.rot = rotary_dim;
    fused.write_kv = write_kv;
    const dim3 grid(n_splits, nkv, (unsigned)n_tokens);
    return (int)q3_launch_cluster(decode_split_kernel<true>, grid, dim3(WARPS * 32), (size_t)SMEM_FUSED, stream, dim3(n_splits, 1, 1),
                                  (const bf16*)nullptr, (const bf16*)k_pages, (const bf16*)v_pages, (float*)nullptr, (float*)nullptr,
                                  token_seq, token_pos, page_table, pages_per_seq, nq, nkv, scale * 1.4426950408889634f, window,
                                  fused);
}
