// Blackwell matrix products for the projections: Y[M,N] = X[M,K] . W[N,K]^T, bfloat16
// operands, 32-bit accumulation in tensor memory, bfloat16 or float32 output.  They replace
// the reference's cublasGemmEx call per projection (src/ops/linear.cpp:165-193).
//
// Two forms share the building blocks (TMA loads of 128-byte-swizzled K-major tiles into a
// ring of shared-memory stages, tcgen05.mma issued by one thread, accumulator in tensor
// memory, tcgen05.ld epilogue):
//
//   * the "weights first" form for 17..128 rows (large decode batches, short prompts), where
//     the product is bound by reading W once: D[128 rows of W, MT tokens] = W_tile . X_tile^T,
//     so the 128-row operand of the instruction is full whatever the number of tokens.  When W
//     has few rows, K is split over the blocks of a thread-block cluster; their partial tiles
//     meet in shared memory (each block reduces a share of the tokens over distributed shared
//     memory, in block order) and one kernel writes the finished output.
//   * the "tokens first" persistent form for prompts, further down.
//
// Roles in a block of the first form:
//   warp 0     TMA producer
//   warp 1     allocates tensor memory; one thread issues tcgen05.mma (M=128, N=MT, K=16,
//              four per stage) and commits each stage back to the producer
//   warps 2-5  drain the accumulator (one TMEM lane = one row of W per thread) into shared memory
//   all        after the cluster barrier: reduce over the cluster, convert, store (optionally
//              SiLU(gate) * up of interleaved rows)
// Every wait on an mbarrier is bounded: after Q3_WAIT_LIMIT polls the thread records where it
// gave up in `status` and the block winds down (tensor memory is freed on every path, and the
// cluster barriers are reached by every thread on every path).
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace {

constexpr int BM = 128;                 // rows of W per tile (the UMMA M)
constexpr int BK = 64;                  // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    tc_mma_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) { return desc_k_major(smem_addr); }

// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 to_out<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- thread-block cluster helpers
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `addr` (a shared-memory address of this block) in the block of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

constexpr int PART_LD = BM + 4;         // floats per token in the partial tile (rows stay 16-byte aligned)

template <typename OutT> __device__ __forceinline__ void store4(OutT* p, float4 v, bool vec, int valid);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v, bool vec, int valid) {
    if (vec && valid >= 4) { *reinterpret_cast<float4*>(p) = v; return; }
    const float e[4] = {v.x, v.y, v.z, v.w};
    for (int i = 0; i < 4 && i < valid; ++i) p[i] = e[i];
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v, bool vec, int valid) {
    if (vec && valid >= 4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        return;
    }
    const float e[4] = {v.x, v.y, v.z, v.w};
    for (int i = 0; i < 4 && i < valid; ++i) p[i] = __float2bfloat16_rn(e[i]);
}

// Grid (tiles of 128 rows of W, K ranges, tiles of MT tokens); the blocks of one tile form a cluster
// (1, gridDim.y, 1).
// GATED: W holds gate and up rows interleaved in blocks of eight and Y is [M, N/2] = round(silu(g)) * u.
template <int MT, int STAGES, int MINB, bool GATED, typename OutT>
__global__ void __launch_bounds__(THREADS, MINB)
gemm_tcgen05_mid_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        OutT* __restrict__ Y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = MT * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // multiples of 1024
    constexpr uint32_t TMEM_COLS = MT < 32 ? 32 : MT;
    static_assert(MT % 16 == 0 && MT >= 16 && MT <= 256, "token tile: the N of an M=128 tcgen05.mma");
    // the partial tile reuses the stages (and what lies behind them, if it is the larger of the two)
    constexpr int RING_BYTES = STAGES * STAGE_BYTES > MT * PART_LD * 4 ? STAGES * STAGE_BYTES : (MT * PART_LD * 4 + 1023) / 1024 * 1024;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;         // 128-byte swizzle wants 1024-byte tiles
    const uint32_t bars = base + RING_BYTES;                              // full[STAGES], empty[STAGES], done, tmem slot
    const uint32_t bar_done = bars + 2 * STAGES * 8, tmem_slot = bar_done + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.z * MT;
    const uint32_t rank = cluster_rank(), ranks = gridDim.y;
    const int nkb_all = (K + BK - 1) / BK;
    const int kb_begin = (int)(((int64_t)rank * nkb_all) / ranks);
    const int kb_end = (int)(((int64_t)(rank + 1) * nkb_all) / ranks);
    const int nkb = kb_end - kb_begin;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bars + s * 8, 1);
            mbar_init(bars + (STAGES + s) * 8, 1);
        }
        mbar_init(bar_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // the producer starts its stream now; tensor memory is handed out meanwhile and its address goes to
    // the warps that use it over a barrier of their own (warps 1..5)
    uint32_t tmem_base = 0;
    if (warp >= 1) {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(THREADS - 32) : "memory");
        tc_fence_after();
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
    }

    if (warp == 0) {
        // ---------------- producer
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(bars + (STAGES + s) * 8, phase ^ 1u)) {      // the stage is free
                    atomicExch(status, 1);
                    break;
                }
                const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                mbar_expect_tx(bars + s * 8, STAGE_BYTES);
                tma_load_2d(a, &map_w, bars + s * 8, (kb_begin + i) * BK, n0);      // weights: independent of the
                if (i == 0) pdl_wait();                                              // kernel before; X is not
                tma_load_2d(b, &map_x, bars + s * 8, (kb_begin + i) * BK, m0);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(MT);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
                if (!mbar_wait(bars + s * 8, phase)) {                       // the tiles have landed
                    atomicExch(status, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                const uint64_t da = make_desc(a), db = make_desc(b);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)                        // 32 bytes further along K per step
                    tc_mma(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(bars + (STAGES + s) * 8);                          // frees the stage when the MMAs are done
            }
            tc_commit(bar_done);                                             // accumulator complete (or abandoned)
        }
    } else {
        // ---------------- warps 2..5 own TMEM lanes 32*(warp % 4) ..: accumulator -> part[token][row of W]
        const bool ok = mbar_wait(bar_done, 0);                              // every load has landed and been consumed,
        if (!ok && lane == 0) atomicExch(status, 3);                         // so the stages may be overwritten
        tc_fence_after();
        float* part = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
        const int lane_base = (warp & 3) * 32;
#pragma unroll 1
        for (int c = 0; c < MT; c += 16) {
            uint32_t r[16];
            if (ok && nkb > 0) {
                tc_ld16(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)c, r);
                tc_wait_ld();
            } else {                                                          // an empty K range adds nothing
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) part[(c + j) * PART_LD + lane_base + lane] = __uint_as_float(r[j]);
        }
    }
    tc_fence_before();
    __syncwarp();
    if (ranks > 1) cluster_sync();                                            // every block's partial tile is in place
    else __syncthreads();                                                     // (a block on its own: its own tile)

    // ---------------- reduce over the cluster: this block finishes the tokens m with m % ranks == rank
    pdl_wait();                                                               // no global write before this
    {
        const int out_n = GATED ? (N >> 1) : N;
        const bool vec = (out_n % 4 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
        constexpr int GROUPS = GATED ? 16 : 32;                               // groups of four outputs per token and tile
        const int my_tokens = (MT - (int)rank + (int)ranks - 1) / (int)ranks;
        for (int idx = threadIdx.x; idx < my_tokens * GROUPS; idx += THREADS) {
            const int local = (idx / GROUPS) * (int)ranks + (int)rank, g = idx % GROUPS;
            const int m = m0 + local;
            if (m >= M) continue;
            if constexpr (!GATED) {
                const uint32_t addr = base + (uint32_t)(local * PART_LD + 4 * g) * 4u;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t s = 0; s < ranks; ++s) {
                    const float4 v = ld_cluster_f4(map_to_rank(addr, s));
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const int n = n0 + 4 * g;
                if (n < N) store4<OutT>(Y + (int64_t)m * N + n, sum, vec, N - n);
            } else {
                // rows 16t + 4h .. +3 are gates, rows 16t + 8 + 4h .. +3 the ups of features 8t + 4h .. +3
                const int t = g >> 1, h = g & 1;
                const uint32_t addr_g = base + (uint32_t)(local * PART_LD + 16 * t + 4 * h) * 4u, addr_u = addr_g + 32u;
                float4 gs = make_float4(0.f, 0.f, 0.f, 0.f), us = gs;
                for (uint32_t s = 0; s < ranks; ++s) {
                    const float4 a = ld_cluster_f4(map_to_rank(addr_g, s)), b = ld_cluster_f4(map_to_rank(addr_u, s));
                    gs.x += a.x; gs.y += a.y; gs.z += a.z; gs.w += a.w;
                    us.x += b.x; us.y += b.y; us.z += b.z; us.w += b.w;
                }
                // both sums are rounded to bfloat16 as the two separate products of the reference would be,
                // then round(silu(g)) * u (src/ops/elementwise.cu:47-65)
                auto gate = [](float gv, float uv) {
                    gv = round_to<bf16>(gv);
                    uv = round_to<bf16>(uv);
                    return round_to<bf16>(gv / (1.0f + expf(-gv))) * uv;
                };
                const float4 o = make_float4(gate(gs.x, us.x), gate(gs.y, us.y), gate(gs.z, us.z), gate(gs.w, us.w));
                const int f = (n0 >> 1) + 8 * t + 4 * h;
                if (f < out_n) store4<OutT>(Y + (int64_t)m * out_n + f, o, vec, out_n - f);
            }
        }
    }
    __syncwarp();
    if (ranks > 1) cluster_sync();                                            // nobody leaves while its tile is being read
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The prompt form: persistent, tokens first.  D[128 tokens, BN rows of W] per tile, so a thread of
// the epilogue owns one token and writes a contiguous run of outputs.  Each block walks tiles
// (tile = blockIdx.x, += gridDim.x; the token tile varies fastest so that blocks running at the
// same time share W tiles in the L2); the accumulator is double-buffered in tensor memory
// (2 x BN columns), so the epilogue of one tile runs under the products of the next.
constexpr uint32_t make_idesc_mn(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

template <typename OutT> __device__ __forceinline__ void store_run8(OutT* p, const uint32_t* r);
template <> __device__ __forceinline__ void store_run8<float>(float* p, const uint32_t* r) {
    reinterpret_cast<uint4*>(p)[0] = make_uint4(r[0], r[1], r[2], r[3]);
    reinterpret_cast<uint4*>(p)[1] = make_uint4(r[4], r[5], r[6], r[7]);
}
template <> __device__ __forceinline__ void store_run8<bf16>(bf16* p, const uint32_t* r) {
    uint4 v;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(__uint_as_float(r[0]), __uint_as_float(r[1])); v.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(__uint_as_float(r[2]), __uint_as_float(r[3])); v.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(__uint_as_float(r[4]), __uint_as_float(r[5])); v.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(__uint_as_float(r[6]), __uint_as_float(r[7])); v.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(p) = v;
}

// GATED: W holds gate and up rows interleaved in blocks of eight (as the decode kernel's gated form);
// the epilogue then writes round(silu(g)) * u, [M, N/2], instead of the raw product.
// 32 consecutive columns (rows of W n0 + c ..) of one token's accumulator row, converted and stored; `row` points at
// the token's first output of this tile.  GATED: the columns are gate[8] up[8] gate[8] up[8] of 16 features and
// the output is round(silu(g)) * u with both rounded to bfloat16 first (src/ops/elementwise.cu:47-65).
template <bool GATED, typename OutT>
__device__ __forceinline__ void store_chunk32(const uint32_t (&r)[32], OutT* row, int c, int n0, bool token_valid, int N,
                                              bool vec_ok) {
    if (!token_valid) return;
    if constexpr (GATED) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + c + h * 16;           // first gate column of this block
            uint32_t packed[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float g = round_to<bf16>(__uint_as_float(r[h * 16 + e]));
                const float u = round_to<bf16>(__uint_as_float(r[h * 16 + 8 + e]));
                packed[e] = __float_as_uint(round_to<bf16>(g / (1.0f + expf(-g))) * u);
            }
            OutT* dst = row + ((c + h * 16) >> 1);
            if (n + 16 <= N && vec_ok) {
                store_run8<OutT>(dst, packed);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (n + 8 + e < N) dst[e] = to_out<OutT>(__uint_as_float(packed[e]));
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int n = n0 + c + j;
            if (vec_ok && n + 8 <= N) {
                store_run8<OutT>(row + c + j, r + j);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (n + e < N) row[c + j + e] = to_out<OutT>(__uint_as_float(r[j + e]));
            }
        }
    }
}

template <int BN, int STAGES, bool GATED, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_prompt_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                           OutT* __restrict__ Y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN;      // two accumulators
    static_assert(2 * BN <= 512, "two accumulators have to fit the 512 columns of tensor memory");
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;       // full[S], empty[S], acc_full[2], acc_empty[2], slot
    const uint32_t bar_acc_full = bars + 2 * STAGES * 8, bar_acc_empty = bar_acc_full + 16, tmem_slot = bar_acc_empty + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN, tiles = m_tiles * n_tiles;
    const int nkb = (K + BK - 1) / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bars + s * 8, 1);
            mbar_init(bars + (STAGES + s) * 8, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + b * 8, 1);
            mbar_init(bar_acc_empty + b * 8, 4);             // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();                                       // X is the output of the kernel before
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(bars + (STAGES + s) * 8, ((it / STAGES) & 1u) ^ 1u);
                    if (!ok) { atomicExch(status, 1); break; }
                    const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                    mbar_expect_tx(bars + s * 8, STAGE_BYTES);
                    tma_load_2d(a, &map_x, bars + s * 8, kb * BK, m0);
                    tma_load_2d(b, &map_w, bars + s * 8, kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_mn(BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1u;
                ok = mbar_wait(bar_acc_empty + buf * 8, ((local >> 1) & 1u) ^ 1u);      // the epilogue has drained it
                if (!ok) { atomicExch(status, 4); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(bars + s * 8, (it / STAGES) & 1u);
                    if (!ok) { atomicExch(status, 2); break; }
                    tc_fence_after();
                    const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                    const uint64_t da = make_desc(a), db = make_desc(b);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit(bars + (STAGES + s) * 8);
                }
                tc_commit(bar_acc_full + buf * 8);
            }
        }
    } else {
        pdl_wait();
        const int lane_base = (warp & 3) * 32;
        const bool vec_ok = ((GATED ? (N >> 1) : N) % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
        uint32_t local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const uint32_t buf = local & 1u;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            if (!mbar_wait(bar_acc_full + buf * 8, (local >> 1) & 1u)) {
                if (lane == 0) atomicExch(status, 3);
                break;
            }
            tc_fence_after();
            const int m = m0 + lane_base + lane;
            OutT* row = Y + (int64_t)m * (GATED ? (N >> 1) : N) + (GATED ? (n0 >> 1) : n0);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)lane_base << 16) + buf * BN + (uint32_t)c, r);
                tc_wait_ld();
                store_chunk32<GATED, OutT>(r, row, c, n0, m < M, N, vec_ok);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + buf * 8);          // this warp's quarter is drained
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The prompt form on pairs of SMs (tcgen05 cta_group::2).  A tile of 128 tokens by 256 rows of W
// costs an SM 48 KB of shared-memory fill per K step of 64, and what an SM can pull from the L2 then
// bounds the product below what its tensor cores could do.  Here two blocks on neighbouring SMs (a
// cluster of two) share one tile of 256 tokens by 256 rows of W: each loads its own 128 tokens and
// only HALF of the W tile (its 128 rows), the instruction reads both halves from both blocks'
// shared memory, and each block's tensor memory receives the accumulator of its own 128 tokens.
// Per K step a block now fills 32 KB for the same arithmetic.
//
// Protocol (rank 0 of the pair leads):
//   full[s]       in the leader: both blocks' TMA loads report their bytes there
//   empty[s]      in each block: the leader's tcgen05.commit arrives at both (multicast)
//   acc_full[b]   in each block: likewise, when a tile's accumulator is complete
//   acc_empty[b]  in the leader: the eight drain warps of both blocks arrive there
// Only the leader issues tcgen05.mma.  Every wait is bounded as above, and both blocks meet at a
// cluster barrier before either leaves (the peer's shared memory and barriers are in use until then).
// The epilogue of the q/k/v product for prompts: what qkv_prepare (attention.cu) does to the product's output, done
// on the accumulator instead, so that the [tokens, (nq + 2 nkv) d] matrix is never written and read back.  A thread
// of the epilogue owns one token and, in a tile of 256 columns, 256 / d whole heads of it: the sum of squares of
// a head, its normalisation (round(round(x * inv) * w), as the reference's per-head RMSNorm), the rotation of
// the pairs (i, i + d/2) by the token's position and the write - q to its matrix, k and v to the token's place
// in the pages - are all the thread's own.  The accumulator is rounded to bfloat16 first, as the product's
// output would have been.  Head sizes 64, 128 and 256 (whole heads in a tile, halves of whole 32-column chunks).
// What it costs: a thread's token has its own row of the rotation tables and its own rows of q and of the pages, so
// every load and store of a warp touches 32 lines, and the four warps of a block share one path to memory: a tile's
// epilogue takes about 12 us where the plain one takes 3.  Under the next tile's K steps (21 us at K = 4,096) that is
// hidden, for a pair's last tile it is not: at 8,192 tokens the fused product takes 321-338 us against 381-412 for
// product + qkv_prepare, at 2,048 tokens 83.5 against 86, at 512 tokens (one tile a pair) 41 against 34 - so it
// is used from 2,048 tokens on (parts/attention.py).

struct QkvEpilogue {
    bf16* q_out;                   // [tokens, nq * d]
    bf16* k_pages;                 // [pages, nkv, Q3_PAGE_TOKENS, d]
    bf16* v_pages;
    const float* q_norm_w;         // [d] or null
    const float* k_norm_w;
    const float* cos_tab;          // [positions, d / 2] or null
    const float* sin_tab;
    const int* token_seq;          // [tokens]: row of the page table
    const int* token_pos;          // [tokens]: position in the sequence
    const int* page_table;         // [sequences, pages_per_seq]
    int pages_per_seq, nq, nkv, d, write_kv;
    float eps;
};

__device__ __forceinline__ void store_bf16x8(bf16* p, const float (&v)[8]) {
    uint4 o;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(p) = o;
}
__device__ __forceinline__ void load_f32x8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// One head of one token: D accumulator columns from `acc` on.  D = 64 or 128: the whole head is taken into
// registers with one wait, so the sum of squares, the normalisation and the rotation need no second pass over
// tensor memory.
template <int D>
__device__ __forceinline__ void qkv_head_in_registers(uint32_t acc, bool live, bf16* dst, const float* nw, float eps,
                                                      const float* cs_row, const float* sn_row) {
    constexpr int HALF = D / 2, CHUNKS = D / 32;
    uint32_t r[CHUNKS][32];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) tc_ld32(acc + (uint32_t)(c * 32), r[c]);
    tc_wait_ld();
    if (!live) return;
    float inv = 1.0f;
    if (nw != nullptr) {
        float sq = 0.0f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float v = round_to<bf16>(__uint_as_float(r[c][j]));
                sq += v * v;
            }
        inv = rsqrtf(sq / (float)D + eps);
    }
#pragma unroll
    for (int i0 = 0; i0 < HALF; i0 += 8) {
        float x[8], y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            x[i] = round_to<bf16>(__uint_as_float(r[(i0 + i) / 32][(i0 + i) % 32]));
            y[i] = round_to<bf16>(__uint_as_float(r[(HALF + i0 + i) / 32][(HALF + i0 + i) % 32]));
        }
        if (nw != nullptr) {
            float wx[8], wy[8];
            load_f32x8(nw + i0, wx);
            load_f32x8(nw + HALF + i0, wy);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[i] = round_to<bf16>(round_to<bf16>(x[i] * inv) * wx[i]);
                y[i] = round_to<bf16>(round_to<bf16>(y[i] * inv) * wy[i]);
            }
        }
        if (cs_row != nullptr) {
            float cs[8], sn[8];
            load_f32x8(cs_row + i0, cs);
            load_f32x8(sn_row + i0, sn);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float xr = x[i] * cs[i] - y[i] * sn[i], yr = y[i] * cs[i] + x[i] * sn[i];
                x[i] = xr;
                y[i] = yr;
            }
        }
        store_bf16x8(dst + i0, x);
        store_bf16x8(dst + HALF + i0, y);
    }
}

// The same for any head size that is a multiple of 64 (here: 256), in two passes over tensor memory.
__device__ __forceinline__ void qkv_head_two_passes(uint32_t acc, int d, bool live, bf16* dst, const float* nw, float eps,
                                                    const float* cs_row, const float* sn_row) {
    const int half = d >> 1;
    float inv = 1.0f;
    if (nw != nullptr) {
        float sq = 0.0f;
#pragma unroll 1
        for (int c = 0; c < d; c += 32) {
            uint32_t r[32];
            tc_ld32(acc + (uint32_t)c, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float v = round_to<bf16>(__uint_as_float(r[j]));
                sq += v * v;
            }
        }
        inv = rsqrtf(sq / (float)d + eps);
    }
#pragma unroll 1
    for (int c = 0; c < half; c += 32) {
        uint32_t a[32], b[32];                             // columns c .. c + 31 of both halves of the head
        tc_ld32(acc + (uint32_t)c, a);
        tc_ld32(acc + (uint32_t)(half + c), b);
        tc_wait_ld();
        if (!live) continue;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            float x[8], y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[i] = round_to<bf16>(__uint_as_float(a[j + i]));
                y[i] = round_to<bf16>(__uint_as_float(b[j + i]));
            }
            if (nw != nullptr) {
                float wx[8], wy[8];
                load_f32x8(nw + c + j, wx);
                load_f32x8(nw + half + c + j, wy);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    x[i] = round_to<bf16>(round_to<bf16>(x[i] * inv) * wx[i]);
                    y[i] = round_to<bf16>(round_to<bf16>(y[i] * inv) * wy[i]);
                }
            }
            if (cs_row != nullptr) {
                float cs[8], sn[8];
                load_f32x8(cs_row + c + j, cs);
                load_f32x8(sn_row + c + j, sn);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xr = x[i] * cs[i] - y[i] * sn[i], yr = y[i] * cs[i] + x[i] * sn[i];
                    x[i] = xr;
                    y[i] = yr;
                }
            }
            store_bf16x8(dst + c + j, x);
            store_bf16x8(dst + half + c + j, y);
        }
    }
}

// `acc`: the thread's row of the tile's accumulator in tensor memory; token `m`, tile columns n0 .. n0 + 255.
__device__ __forceinline__ void qkv_tile_epilogue(uint32_t acc, int m, bool token_valid, int n0, int N, const QkvEpilogue& e) {
    const int d = e.d, half = d >> 1;
    int pos = 0;
    int64_t page = 0;
    if (token_valid) {
        pos = e.token_pos[m];
        if (e.write_kv) page = e.page_table[(int64_t)e.token_seq[m] * e.pages_per_seq + pos / Q3_PAGE_TOKENS];
    }
    for (int h0 = 0; h0 < 256 && n0 + h0 < N; h0 += d) {       // the same heads for every thread of the warp
        const int head = (n0 + h0) / d;
        const bool is_q = head < e.nq, is_v = head >= e.nq + e.nkv;
        const float* nw = is_q ? e.q_norm_w : (is_v ? nullptr : e.k_norm_w);
        const bool live = token_valid && (is_q || e.write_kv);
        const bool rotate = e.cos_tab != nullptr && !is_v;
        bf16* dst = nullptr;
        if (live)
            dst = is_q ? e.q_out + ((int64_t)m * e.nq + head) * d
                       : (is_v ? e.v_pages : e.k_pages) +
                             ((page * e.nkv + (head - e.nq) % e.nkv) * Q3_PAGE_TOKENS + pos % Q3_PAGE_TOKENS) * d;
        const float* cs_row = rotate ? e.cos_tab + (int64_t)pos * half : nullptr;
        const float* sn_row = rotate ? e.sin_tab + (int64_t)pos * half : nullptr;
        if (d == 128) qkv_head_in_registers<128>(acc + (uint32_t)h0, live, dst, nw, e.eps, cs_row, sn_row);
        else if (d == 64) qkv_head_in_registers<64>(acc + (uint32_t)h0, live, dst, nw, e.eps, cs_row, sn_row);
        else qkv_head_two_passes(acc + (uint32_t)h0, d, live, dst, nw, e.eps, cs_row, sn_row);
    }
}

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_in_leader, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_in_leader), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far are done, at the barrier at this offset in both blocks of the pair.
// `mask`: the two blocks of the pair by their ranks in the cluster (3 for a cluster that is one pair).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask = 3) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int STAGES, bool GATED, typename OutT, bool QKV = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         OutT* __restrict__ Y, int M, int N, int K, int* __restrict__ status, const QkvEpilogue qkv) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int BN = 256, PAIR_M = 2 * BM;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;                    // two accumulators of 128 tokens x 256 rows of W
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;       // full[S], empty[S], acc_full[2], acc_empty[2], slot
    const uint32_t bar_acc_full = bars + 2 * STAGES * 8, bar_acc_empty = bar_acc_full + 16, tmem_slot = bar_acc_empty + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pairs_m = (M + PAIR_M - 1) / PAIR_M, n_tiles = (N + BN - 1) / BN, tiles = pairs_m * n_tiles;
    const int first = blockIdx.x >> 1, stride = gridDim.x >> 1;
    const int nkb = (K + BK - 1) / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bars + s * 8, 1);
            mbar_init(bars + (STAGES + s) * 8, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + b * 8, 1);
            mbar_init(bar_acc_empty + b * 8, 8);             // one arrival per drain warp of the pair
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                           // the peer's barriers exist before anything signals them
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();                                       // X is the output of the kernel before
            uint32_t it = 0;
            bool ok = true;
            for (int tile = first; tile < tiles && ok; tile += stride) {
                const int m0 = (tile % pairs_m) * PAIR_M + (int)rank * BM;
                const int n0 = (tile / pairs_m) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(bars + (STAGES + s) * 8, ((it / STAGES) & 1u) ^ 1u);
                    if (!ok) { atomicExch(status, 1); break; }
                    const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                    const uint32_t full_in_leader = map_to_rank(bars + s * 8, 0);
                    if (rank == 0) mbar_expect_tx(bars + s * 8, 2 * STAGE_BYTES);       // both blocks' bytes
                    tma_load_2d_pair(a, &map_x, full_in_leader, kb * BK, m0);
                    tma_load_2d_pair(b, &map_w, full_in_leader, kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_mn(PAIR_M, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = first; tile < tiles && ok; tile += stride, ++local) {
                const uint32_t buf = local & 1u;
                ok = mbar_wait(bar_acc_empty + buf * 8, ((local >> 1) & 1u) ^ 1u);      // both blocks have drained it
                if (!ok) { atomicExch(status, 4); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(bars + s * 8, (it / STAGES) & 1u);
                    if (!ok) { atomicExch(status, 2); break; }
                    tc_fence_after();
                    const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                    const uint64_t da = make_desc(a), db = make_desc(b);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(bars + (STAGES + s) * 8);
                }
                tc_commit_pair(bar_acc_full + buf * 8);
            }
        }
    } else {
        pdl_wait();
        const int lane_base = (warp & 3) * 32;
        const bool vec_ok = ((GATED ? (N >> 1) : N) % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
        uint32_t local = 0;
        for (int tile = first; tile < tiles; tile += stride, ++local) {
            const uint32_t buf = local & 1u;
            const int m0 = (tile % pairs_m) * PAIR_M + (int)rank * BM, n0 = (tile / pairs_m) * BN;
            if (!mbar_wait(bar_acc_full + buf * 8, (local >> 1) & 1u)) {
                if (lane == 0) atomicExch(status, 3);
                break;
            }
            tc_fence_after();
            const int m = m0 + lane_base + lane;
            if constexpr (QKV) {
                qkv_tile_epilogue(tmem_base + ((uint32_t)lane_base << 16) + buf * BN, m, m < M, n0, N, qkv);
            } else {
                OutT* row = Y + (int64_t)m * (GATED ? (N >> 1) : N) + (GATED ? (n0 >> 1) : n0);
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)lane_base << 16) + buf * BN + (uint32_t)c, r);
                    tc_wait_ld();
                    store_chunk32<GATED, OutT>(r, row, c, n0, m < M, N, vec_ok);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(bar_acc_empty + buf * 8, 0));   // this warp's share is drained
        }
    }
    tc_fence_before();
    __syncwarp();
    cluster_sync();                                           // the peer reads this block's memory and barriers until here
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The same tile on pairs of SMs with K split over the pairs of one cluster, for the shapes whose 256 x 256
// tiles are too few (or just too many) for the 74 pairs of the GPU: a few hundred tokens, or a tile count
// slightly above a whole number of waves.  A cluster of 2 S blocks is S pairs; pair s multiplies the K
// range s of one tile, and the S partial accumulators meet over distributed shared memory: every block
// finishes every S-th chunk of 32 columns; it sends the other chunks of its accumulator into the (by then
// idle) stages of the blocks of its own parity that finish them - remote stores, which do not wait, where
// remote loads took 1.8 us a round - and adds what it received to its own in pair order 0 .. S-1: a fixed
// order, so the sum does not depend on which block computes it.  One tile per cluster, one accumulator.
// Grid (2 S, tiles): the rank in the cluster is blockIdx.x; the token tile varies fastest in blockIdx.y.
constexpr int SPLITK_CHUNK_BYTES = BM * 32 * 4;       // one parked chunk: 128 tokens x 32 columns of float32

__device__ __forceinline__ uint32_t parked_addr(uint32_t base, int chunk, int row, int quad) {
    // a thread only ever reads back what the thread of the same row wrote, so the layout is free: the 32 lanes of
    // one store (one 16-byte quad each) fill 512 consecutive bytes, which the network between SMs moves whole
    return base + (uint32_t)chunk * SPLITK_CHUNK_BYTES + (uint32_t)(row >> 5) * 4096u + (uint32_t)quad * 512u + (uint32_t)(row & 31) * 16u;
}

template <int STAGES, bool GATED, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_splitk_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                OutT* __restrict__ Y, int M, int N, int K, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int BN = 256, PAIR_M = 2 * BM, CHUNKS = BN / 32;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = BN;
    static_assert(6 * SPLITK_CHUNK_BYTES <= STAGES * STAGE_BYTES, "the received chunks reuse the stages (at most 3 senders x 2 or 2 x 3 or 1 x 4)");
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;       // full[S], empty[S], acc_full, slot
    const uint32_t bar_acc_full = bars + 2 * STAGES * 8, tmem_slot = bar_acc_full + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank(), parity = rank & 1u, leader = rank & ~1u;
    const int split = (int)(rank >> 1), splits = (int)(gridDim.x >> 1);
    const int pairs_m = (M + PAIR_M - 1) / PAIR_M;
    const int tile = blockIdx.y;
    const int m0 = (tile % pairs_m) * PAIR_M + (int)parity * BM, n0 = (tile / pairs_m) * BN;
    const int nkb_all = (K + BK - 1) / BK;
    const int kb_begin = (int)(((int64_t)split * nkb_all) / splits), kb_end = (int)(((int64_t)(split + 1) * nkb_all) / splits);
    const int nkb = kb_end - kb_begin;                       // the host keeps splits <= nkb_all: at least one step

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bars + s * 8, 1);
            mbar_init(bars + (STAGES + s) * 8, 1);
        }
        mbar_init(bar_acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                           // the peers' barriers exist before anything signals them
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

    bool acc_ok = true;
    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(bars + (STAGES + s) * 8, ((uint32_t)(i / STAGES) & 1u) ^ 1u)) { atomicExch(status, 1); break; }
                const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                const uint32_t full_in_leader = map_to_rank(bars + s * 8, leader);
                if (parity == 0) mbar_expect_tx(bars + s * 8, 2 * STAGE_BYTES);         // both blocks' bytes
                tma_load_2d_pair(b, &map_w, full_in_leader, (kb_begin + i) * BK, n0 + (int)parity * (BN / 2));
                if (i == 0) pdl_wait();                       // the weights do not depend on the kernel before; X does
                tma_load_2d_pair(a, &map_x, full_in_leader, (kb_begin + i) * BK, m0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && parity == 0) {
            constexpr uint32_t idesc = make_idesc_mn(PAIR_M, BN);
            const uint16_t mask = (uint16_t)(3u << leader);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(bars + s * 8, (uint32_t)(i / STAGES) & 1u)) { atomicExch(status, 2); break; }
                tc_fence_after();
                const uint32_t a = base + s * STAGE_BYTES, b = a + A_BYTES;
                const uint64_t da = make_desc(a), db = make_desc(b);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tc_mma_pair(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit_pair(bars + (STAGES + s) * 8, mask);
            }
            tc_commit_pair(bar_acc_full, mask);               // accumulator complete (or abandoned)
        }
    } else {
        acc_ok = mbar_wait(bar_acc_full, 0);
        if (!acc_ok && lane == 0) atomicExch(status, 3);
    }
    tc_fence_before();
    __syncwarp();
    cluster_sync();                   // every pair's loads have landed and been consumed: the stages of all blocks are free
    tc_fence_after();
    const int lane_base = (warp & 3) * 32, row = lane_base + lane;
    if (warp >= 2 && acc_ok) {
        // send the chunks that another block finishes into that block's stages (remote stores do not wait)
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c) {
            const int owner = c % splits;
            if (owner == split) continue;
            uint32_t r[32];
            tc_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(c * 32), r);
            tc_wait_ld();
            // slot of (sender, the owner's n-th chunk) in the owner: senders in pair order, the owner itself left out
            const int slot = (split - (split > owner ? 1 : 0)) * ((CHUNKS + splits - 1) / splits) + c / splits;
            const uint32_t dst_rank = (uint32_t)(2 * owner) + parity;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};"
                             ::"r"(map_to_rank(parked_addr(base, slot, row, q), dst_rank)), "r"(r[4 * q]), "r"(r[4 * q + 1]),
                               "r"(r[4 * q + 2]), "r"(r[4 * q + 3]) : "memory");
        }
    }
    __syncwarp();
    cluster_sync();                                           // every block holds the partials of its chunks

    if (warp >= 2 && acc_ok) {
        pdl_wait();                                           // no global write before this
        const bool vec_ok = ((GATED ? (N >> 1) : N) % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
        const int m = m0 + row;
        OutT* out_row = Y + (int64_t)m * (GATED ? (N >> 1) : N) + (GATED ? (n0 >> 1) : n0);
#pragma unroll 1
        for (int c = split; c < CHUNKS; c += splits) {
            uint32_t own[32], r[32];
            tc_ld32(tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(c * 32), own);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;           // 0.0f
            for (int s = 0; s < splits; ++s) {                // pair order, whoever adds
                if (s == split) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(own[j]));
                } else {
                    const int slot = (s - (s > split ? 1 : 0)) * ((CHUNKS + splits - 1) / splits) + c / splits;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 v;
                        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                                     : "r"(parked_addr(base, slot, row, q)) : "memory");
                        r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + v.x);
                        r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + v.y);
                        r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + v.z);
                        r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + v.w);
                    }
                }
            }
            store_chunk32<GATED, OutT>(r, out_row, c * 32, n0, m < M, N, vec_ok);
        }
    }
    tc_fence_before();
    __syncwarp();
    cluster_sync();                                           // the pair gives its tensor memory back together
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// A [rows, K] bfloat16 row-major matrix, fetched in boxes of [box_rows, 64] with 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    return q3_make_map_bf16(map, ptr, rows, K, box_rows, BK, true);
}

int sm_count() { return q3_device_sm_count(); }

// K ranges (blocks per cluster) for a matrix of N rows: the largest power of two up to the portable
// cluster size that keeps the grid within 2.6 blocks per SM (two are resident; more blocks than that keep
// more loads in flight and still measured faster: gate/up of an 8B-sized layer at 64 rows 39.5 us with two
// ranges against 45.0 with one) - within one block per SM for the 256-token tile, of which one fits - and
// leaves every block 16 K steps.  `token_tiles` = 0 stands for at most 128 tokens.
int mid_splits(int N, int K, int token_tiles) {
    const int tiles = ((N + BM - 1) / BM) * (token_tiles > 0 ? token_tiles : 1), nkb = (K + BK - 1) / BK;
    const int limit = token_tiles > 0 ? sm_count() : sm_count() * 13 / 5;
    int s = 1;
    while (s < 8 && tiles * (2 * s) <= limit && nkb / (2 * s) >= 16) s *= 2;
    return s;
}

template <int MT, int STAGES, int MINB, bool GATED, typename OutT>
int launch_mid(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int splits, int* status, cudaStream_t stream) {
    constexpr int RING = STAGES * (BM * BK * 2 + MT * BK * 2), PART = (MT * PART_LD * 4 + 1023) / 1024 * 1024;
    constexpr int SMEM = (RING > PART ? RING : PART) + 1024 + 256;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(gemm_tcgen05_mid_kernel<MT, STAGES, MINB, GATED, OutT>, SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, W, N, K, BM) || !make_map(&map_x, X, M, K, MT)) return Q3_ERR_BAD_SIZE;
    const dim3 grid((N + BM - 1) / BM, splits, (M + MT - 1) / MT);
    return (int)q3_launch_cluster(gemm_tcgen05_mid_kernel<MT, STAGES, MINB, GATED, OutT>, grid, dim3(THREADS), (size_t)SMEM, stream,
                                  dim3(1, splits, 1), map_w, map_x, Y, M, N, K, status);
}

// Stages and blocks per SM come from a sweep on the projections of an 8B-sized layer: a grid that fits
// the GPU at two blocks per SM wants the deeper ring; a grid of many waves (the output projection onto the
// vocabulary) wants three blocks per SM with a shorter ring, so that one block's start and end hide behind
// the others' streams (gate/up of an 8B-sized layer at 128 rows: 41.5 us with three blocks of two stages per SM, all
// 384 blocks resident, against 49.9 with two blocks of three stages).
template <bool GATED, typename OutT>
int dispatch_mid(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int splits, int* status, cudaStream_t stream) {
    const bool waves = (int64_t)((N + BM - 1) / BM) * splits > 2 * sm_count();
#define Q3_MID(MT, ST, MB) return launch_mid<MT, ST, MB, GATED, OutT>(X, W, Y, M, N, K, splits, status, stream)
    if (M <= 16) { if (waves) Q3_MID(16, 4, 3); Q3_MID(16, 5, 2); }
    if (M <= 32) { if (waves) Q3_MID(32, 3, 3); Q3_MID(32, 5, 2); }
    if (M <= 64) { if (waves) Q3_MID(64, 3, 3); Q3_MID(64, 4, 2); }
    if (M <= 128) { if (waves) Q3_MID(128, 2, 3); Q3_MID(128, 3, 2); }
    Q3_MID(256, 4, 1);                  // one or more tiles of 256 tokens (grid.z)
#undef Q3_MID
}

template <int BN, int STAGES, bool GATED, typename OutT>
int launch_prompt(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int* status, cudaStream_t stream) {
    constexpr int SMEM = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 256;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(gemm_tcgen05_prompt_kernel<BN, STAGES, GATED, OutT>, SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, X, M, K, BM) || !make_map(&map_w, W, N, K, BN)) return Q3_ERR_BAD_SIZE;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int blocks = tiles < sm_count() ? tiles : sm_count();
    return (int)q3_launch(gemm_tcgen05_prompt_kernel<BN, STAGES, GATED, OutT>, dim3(blocks), dim3(THREADS), (size_t)SMEM, stream,
                          map_x, map_w, Y, M, N, K, status);
}

template <int STAGES, bool GATED, typename OutT, bool QKV = false>
int launch_pair(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int* status, cudaStream_t stream,
                const QkvEpilogue& qkv = QkvEpilogue{}) {
    constexpr int SMEM = STAGES * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(gemm_tcgen05_pair_kernel<STAGES, GATED, OutT, QKV>, SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, X, M, K, BM) || !make_map(&map_w, W, N, K, 128)) return Q3_ERR_BAD_SIZE;
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    return (int)q3_launch_cluster(gemm_tcgen05_pair_kernel<STAGES, GATED, OutT, QKV>, dim3(2 * pairs), dim3(THREADS), (size_t)SMEM,
                                  stream, dim3(2, 1, 1), map_x, map_w, Y, M, N, K, status, qkv);
}

template <int STAGES, bool GATED, typename OutT>
int launch_pair_splitk(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int splits, int* status, cudaStream_t stream) {
    constexpr int SMEM = STAGES * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256;
    static Q3PerDevice configured;
    {
        cudaError_t e = q3_allow_shared_memory(gemm_tcgen05_pair_splitk_kernel<STAGES, GATED, OutT>, SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, X, M, K, BM) || !make_map(&map_w, W, N, K, 128)) return Q3_ERR_BAD_SIZE;
    const int64_t tiles = (int64_t)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    if (tiles > 65535) return Q3_ERR_TOO_LARGE;
    return (int)q3_launch_cluster(gemm_tcgen05_pair_splitk_kernel<STAGES, GATED, OutT>, dim3(2 * splits, (unsigned)tiles), dim3(THREADS),
                                  (size_t)SMEM, stream, dim3(2 * splits, 1, 1), map_x, map_w, Y, M, N, K, status);
}

// How many pairs of SMs run at the same time when a cluster is `splits` pairs (what the device can place).
int pair_capacity(int splits) {
    static int cached[64][5];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || splits < 1 || splits > 4) return 0;
    if (cached[dev][splits] == 0) {
        constexpr int SMEM = 6 * (BM * BK * 2 + 128 * BK * 2) + 1024 + 256;
        static Q3PerDevice configured;
        auto kernel = gemm_tcgen05_pair_splitk_kernel<6, false, bf16>;
        if (q3_allow_shared_memory(kernel, SMEM, configured) != cudaSuccess) return 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * splits, 1024);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2 * splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
        cached[dev][splits] = clusters * splits;
    }
    return cached[dev][splits];
}

}  // namespace

// The prompt form: persistent blocks, 128 tokens x `tile_n` (128 or 256) rows of W per tile.
Q3_EXPORT int q3_gemm_tcgen05_prompt_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32,
                                          int tile_n, int* status, void* stream_) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (tile_n == 256)
        return out_is_f32 ? launch_prompt<256, 4, false, float>(x, w, (float*)Y, M, N, K, status, stream)
                          : launch_prompt<256, 4, false, bf16>(x, w, (bf16*)Y, M, N, K, status, stream);
    if (tile_n == 128)
        return out_is_f32 ? launch_prompt<128, 6, false, float>(x, w, (float*)Y, M, N, K, status, stream)
                          : launch_prompt<128, 6, false, bf16>(x, w, (bf16*)Y, M, N, K, status, stream);
    return Q3_ERR_BAD_SIZE;
}

// The prompt form on pairs of SMs: tiles of 256 tokens x 256 rows of W, each block of a pair loading half of
// the W tile.  `gated` as below (bfloat16 output only).  `splits` (1..4) > 1: K split over that many pairs of a
// cluster, one tile per cluster.
Q3_EXPORT int q3_gemm_tcgen05_pair_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated,
                                        int splits, int* status, void* stream_) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || (gated && (N % 16 != 0 || out_is_f32)) || splits < 1 || splits > 4) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (splits > (K + BK - 1) / BK) splits = (K + BK - 1) / BK;
    if (splits > 1) {
        if (gated) return launch_pair_splitk<6, true, bf16>(x, w, (bf16*)Y, M, N, K, splits, status, stream);
        return out_is_f32 ? launch_pair_splitk<6, false, float>(x, w, (float*)Y, M, N, K, splits, status, stream)
                          : launch_pair_splitk<6, false, bf16>(x, w, (bf16*)Y, M, N, K, splits, status, stream);
    }
    if (gated) return launch_pair<6, true, bf16>(x, w, (bf16*)Y, M, N, K, status, stream);
    return out_is_f32 ? launch_pair<6, false, float>(x, w, (float*)Y, M, N, K, status, stream)
                      : launch_pair<6, false, bf16>(x, w, (bf16*)Y, M, N, K, status, stream);
}

// Pairs of SMs that run at once when K is split over `splits` pairs of a cluster (0: the device cannot place it).
Q3_EXPORT int q3_gemm_tcgen05_pair_capacity(int splits) { return pair_capacity(splits); }

// The q/k/v product of a prompt step with qkv_prepare's work in its epilogue (see QkvEpilogue): W [(nq + 2 nkv) d, K]
// holds the q, k and v rows one after the other; q goes to q_out [M, nq d], k and v (if write_kv) to the pages.
// Head sizes 64, 128 and 256; the rotation tables cover the whole head ([positions, d / 2]) or are null.
Q3_EXPORT int q3_gemm_tcgen05_pair_qkv_bf16(const void* X, const void* W, int M, int K, void* q_out, void* k_pages, void* v_pages,
                                            const float* q_norm_w, const float* k_norm_w, const float* cos_tab,
                                            const float* sin_tab, float eps, const int* token_seq, const int* token_pos,
                                            const int* page_table, int pages_per_seq, int nq, int nkv, int d, int write_kv,
                                            int* status, void* stream_) {
    if (M <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || nq <= 0 || nkv <= 0 || (d != 64 && d != 128 && d != 256)) return Q3_ERR_BAD_SIZE;
    if ((cos_tab == nullptr) != (sin_tab == nullptr) || (q_norm_w == nullptr) != (k_norm_w == nullptr)) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W) || !aligned16(q_out) || !aligned16(k_pages) || !aligned16(v_pages) || !aligned16(q_norm_w) ||
        !aligned16(k_norm_w) || !aligned16(cos_tab) || !aligned16(sin_tab))
        return Q3_ERR_MISALIGNED;
    const int64_t N = (int64_t)(nq + 2 * nkv) * d;
    if (N > 0x7fffffff) return Q3_ERR_TOO_LARGE;
    QkvEpilogue e;
    e.q_out = (bf16*)q_out; e.k_pages = (bf16*)k_pages; e.v_pages = (bf16*)v_pages;
    e.q_norm_w = q_norm_w; e.k_norm_w = k_norm_w; e.cos_tab = cos_tab; e.sin_tab = sin_tab;
    e.token_seq = token_seq; e.token_pos = token_pos; e.page_table = page_table;
    e.pages_per_seq = pages_per_seq; e.nq = nq; e.nkv = nkv; e.d = d; e.write_kv = write_kv; e.eps = eps;
    return launch_pair<6, false, bf16, true>((const bf16*)X, (const bf16*)W, (bf16*)nullptr, M, (int)N, K, status,
                                             (cudaStream_t)stream_, e);
}

// W [N, K] holds gate and up rows interleaved in blocks of eight; Y [M, N/2] = round(silu(g)) * u, bfloat16.
Q3_EXPORT int q3_gemm_tcgen05_prompt_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int* status,
                                                void* stream_) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || N % 16 != 0) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    return launch_prompt<256, 4, true, bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, status, (cudaStream_t)stream_);
}

// The weights-first form for a few hundred rows of X at most (W is read once per 256 rows).  `splits` K ranges per tile of 128 rows of W (one cluster;
// 0 = chosen from N and K).  `gated`: W [N, K] holds gate and up rows interleaved in blocks of eight and
// Y is [M, N/2] = round(silu(g)) * u.  `status` is a device int that a kernel sets to 1/2/3 if a bounded
// wait ran out (0 otherwise).
Q3_EXPORT int q3_gemm_tcgen05_mid_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated,
                                       int splits, int* status, void* stream_) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || M > 256 * 1024 || splits < 0 || splits > 8 || (gated && N % 16 != 0)) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    cudaStream_t stream = (cudaStream_t)stream_;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (splits == 0) splits = mid_splits(N, K, M <= 128 ? 0 : (M + 255) / 256);
    if (splits > (K + BK - 1) / BK) splits = (K + BK - 1) / BK;
    if (gated)
        return out_is_f32 ? dispatch_mid<true, float>(x, w, (float*)Y, M, N, K, splits, status, stream)
                          : dispatch_mid<true, bf16>(x, w, (bf16*)Y, M, N, K, splits, status, stream);
    return out_is_f32 ? dispatch_mid<false, float>(x, w, (float*)Y, M, N, K, splits, status, stream)
                      : dispatch_mid<false, bf16>(x, w, (bf16*)Y, M, N, K, splits, status, stream);
}

Q3_EXPORT int q3_gemm_tcgen05_mid_splits(int N, int K, int M) { return mid_splits(N, K, M <= 128 ? 0 : (M + 255) / 256); }
