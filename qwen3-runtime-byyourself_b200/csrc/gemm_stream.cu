// Weight-streaming matrix product for decode steps: Y[M,N] = X[M,K] . W[N,K]^T with a handful of
// rows M (one per sequence of the batch), bfloat16 operands, 32-bit accumulation.
//
// In the reference every projection is one cublasGemmEx call whatever M is
// (src/ops/linear.cpp:165-193).  With few rows the product is bound by reading W once, and what
// decides its speed is how many bytes of W each SM keeps in flight, from the first microsecond of
// the kernel to the last.  So the kernel is persistent: one block per SM owns an equal share of the
// rows of W (to the row; to 16 rows when gate and up rows are interleaved), which it walks in pieces
// of 16, 8, 4, 2 or 1 rows, so that all blocks end together whatever N is.  Every warp feeds itself
// through a ring of shared-memory stages filled by bulk tensor copies (TMA): lane 0 asks for a box
// of one piece's rows x 128 k-values (4 KB at most) per stage, several stages ahead, across the
// boundaries of its pieces, and the ring is filled before the kernel waits for its predecessor
// (weights do not depend on it).  K is split over the warps of a block;
// a warp reads its 16-byte operands of mma.m16n8k16 straight out of the stage (W as the 16-row
// operand, the batch rows as the 8-column operand, both with the same permutation of k, which a
// sum over k does not mind) and the warps' partial sums meet in shared memory in warp order, which
// fixes the summation order for every M.
#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int KC = 128;                          // k-values per stage
constexpr int TILE = 16;                         // rows of W per tile
constexpr int STAGE_BYTES = TILE * KC * 2;       // 4 KB
constexpr int KB_PER_STAGE = KC / 32;            // k-blocks of 32: one 16-byte chunk per lane and row

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#ifdef Q3_STREAM_TRACE
__device__ unsigned long long* g_trace = nullptr;
__device__ unsigned int g_trace_launch = 0;
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TRACE(slot) do { if (threadIdx.x == 0 && g_trace) g_trace[((size_t)trace_launch * 160 + blockIdx.x) * 8 + (slot)] = gtime(); } while (0)
#else
#define TRACE(slot) do {} while (0)
#endif

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 to_out<bf16>(float v) { return __float2bfloat16_rn(v); }

// Tensor maps of W with boxes of 16, 8, 4, 2 and 1 rows.
struct StreamMaps {
    CUtensorMap rows[5];
};

// The rows of the piece that starts at `row` in a share that ends at `end`: 16, or the largest power of two that fits.
__device__ __forceinline__ int piece_rows(int row, int end) {
    const int left = end - row;
    return left >= TILE ? TILE : (1 << (31 - __clz(left)));
}

template <int MT, int WARPS, int STAGES> struct StreamSmem {
    static constexpr int LD = TILE + 1;
    static constexpr int RING = WARPS * STAGES * STAGE_BYTES;
    static constexpr int RED = 2 * WARPS * 8 * MT * LD * 4;           // two tiles' partial sums
    static constexpr int BARS = WARPS * STAGES * 8;
    static constexpr int TOTAL = RING + RED + BARS;
};

// MT: tiles of 8 batch rows (M <= 8*MT).  WARPS: K is split over them.  STAGES: 4 KB boxes a warp keeps
// in flight.  GATED: W holds gate and up rows interleaved in blocks of eight (rows 16t..16t+7 gate,
// 16t+8..16t+15 up, both for features 8t..8t+7); the kernel then writes round(silu(g)) * u, [M, N/2].
template <int MT, int WARPS, int STAGES, bool GATED, typename OutT>
__global__ void __launch_bounds__(WARPS * 32, 1)
gemm_stream_kernel(const __grid_constant__ StreamMaps maps, const bf16* __restrict__ X, OutT* __restrict__ Y, int M,
                   int N, int K, int early, int* __restrict__ status) {
    using L = StreamSmem<MT, WARPS, STAGES>;
    extern __shared__ __align__(1024) unsigned char smem[];
    float* red = reinterpret_cast<float*>(smem + L::RING);
    const uint32_t ring = smem_u32(smem), bars = smem_u32(smem + L::RING + L::RED);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
    constexpr int LD = L::LD, COLS = 8 * MT;
#ifdef Q3_STREAM_TRACE
    const unsigned int trace_launch = early >> 8;
    early &= 1;
#endif
    TRACE(0);

    const int n_chunks = (K + KC - 1) / KC;
    const int chunk_begin = (int)(((int64_t)warp * n_chunks) / WARPS), chunk_end = (int)(((int64_t)(warp + 1) * n_chunks) / WARPS);
    const int my_chunks = chunk_end - chunk_begin;
    // this block's share of the rows, in granules of one row (16 when gate and up rows are interleaved)
    constexpr int GRANULE = GATED ? TILE : 1;
    const int64_t granules = (N + GRANULE - 1) / GRANULE;
    const int row_begin = (int)(((int64_t)blockIdx.x * granules) / gridDim.x) * GRANULE;
    const int row_end = min(N, (int)(((int64_t)(blockIdx.x + 1) * granules) / gridDim.x) * GRANULE);
    int n_pieces = 0;
    for (int row = row_begin; row < row_end; row += piece_rows(row, row_end)) ++n_pieces;
    const int total_units = n_pieces * my_chunks;
    const uint32_t my_ring = ring + warp * (STAGES * STAGE_BYTES), my_bars = bars + warp * (STAGES * 8);

    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(my_bars + s * 8, 1);
        mbar_init_fence();
    }
    __syncwarp();
    // lane 0 asks for the warp's next unit (a chunk of k of a piece of rows), in order
    int ask_unit = 0, ask_row = row_begin, ask_chunk = 0;
    auto issue = [&]() {
        if (lane == 0 && ask_unit < total_units) {
            const int rows = piece_rows(ask_row, row_end);
            const uint32_t bar = my_bars + (ask_unit % STAGES) * 8;
            mbar_expect_tx(bar, rows * KC * 2);
            tma_load_2d(my_ring + (ask_unit % STAGES) * STAGE_BYTES, &maps.rows[4 - (31 - __clz(rows))], bar,
                        (chunk_begin + ask_chunk) * KC, ask_row);
            ++ask_unit;
            if (++ask_chunk == my_chunks) {
                ask_chunk = 0;
                ask_row += rows;
            }
        }
    };
    // the weights do not depend on the kernel before this one: fill the ring, then wait for it
    for (int s = 0; s < STAGES; ++s) issue();
    TRACE(1);
    if (early) pdl_launch_dependents();
    pdl_wait();
    TRACE(2);

    const bf16* xrow[MT];
    bool xok[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int row = m * 8 + quad;
        xok[m] = row < M;
        xrow[m] = X + (int64_t)(xok[m] ? row : 0) * K + tq * 8;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // the batch rows' k-values for one unit, in registers one unit ahead of their use
    auto load_x = [&](uint4 (&x)[KB_PER_STAGE][MT], int c) {
        const int k0 = (chunk_begin + c) * KC;
#pragma unroll
        for (int kb = 0; kb < KB_PER_STAGE; ++kb)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int k = k0 + kb * 32 + tq * 8;              // K is a multiple of 8: a chunk is inside or outside
                x[kb][m] = (xok[m] && c < my_chunks && k + 8 <= K) ? *reinterpret_cast<const uint4*>(xrow[m] + k0 + kb * 32) : zero;
            }
    };
    bool failed = false;
    int u = 0;
    uint4 x[KB_PER_STAGE][MT], x_next[KB_PER_STAGE][MT];
    load_x(x, 0);
    int n0 = row_begin;
    for (int ti = 0; ti < n_pieces; ++ti) {
        const int rows = piece_rows(n0, row_end);
        float acc[MT][4];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.0f;
        for (int c = 0; c < my_chunks; ++c, ++u) {
            load_x(x_next, c + 1 < my_chunks ? c + 1 : 0);        // the next unit's: the same k-range again in the next tile
            if (!failed && !mbar_wait(my_bars + (u % STAGES) * 8, (u / STAGES) & 1)) {
                failed = true;                                      // give up waiting: the result is not valid
                if (lane == 0) atomicExch(status, 5);
            }
            if (u == 0) TRACE(3);
            const uint32_t stage = my_ring + (u % STAGES) * STAGE_BYTES + quad * (KC * 2) + tq * 16;
#pragma unroll
            for (int kb = 0; kb < KB_PER_STAGE; ++kb) {
                const uint4 w0 = lds16(stage + kb * 64), w1 = lds16(stage + 8 * (KC * 2) + kb * 64);
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16(acc[m], w0.x, w1.x, w0.y, w1.y, x[kb][m].x, x[kb][m].y);
                    mma_bf16(acc[m], w0.z, w1.z, w0.w, w1.w, x[kb][m].z, x[kb][m].w);
                }
            }
            __syncwarp();                      // every lane has read the stage
            if (lane == 0) fence_proxy_async();
            issue();
#pragma unroll
            for (int kb = 0; kb < KB_PER_STAGE; ++kb)
#pragma unroll
                for (int m = 0; m < MT; ++m) x[kb][m] = x_next[kb][m];
        }
        if (!early && ti == n_pieces - 1) pdl_launch_dependents();   // all of this block's weights are asked for
        if (ti == n_pieces - 1) TRACE(4);

        // accumulator (row n = quad [+8], column m = 2*tq [+1]) -> red[piece parity][warp][m][n]; rows beyond the
        // piece's own hold sums over whatever the stage held there and are dropped
        float* mine = red + ((ti & 1) * WARPS + warp) * COLS * LD;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int cc = m * 8 + tq * 2;
            mine[cc * LD + quad] = acc[m][0];
            mine[(cc + 1) * LD + quad] = acc[m][1];
            mine[cc * LD + quad + 8] = acc[m][2];
            mine[(cc + 1) * LD + quad + 8] = acc[m][3];
        }
        __syncthreads();                       // one barrier per piece: the other parity is written a piece later
        const float* sums = red + (ti & 1) * WARPS * COLS * LD;
        if constexpr (!GATED) {
            for (int idx = threadIdx.x; idx < TILE * COLS; idx += WARPS * 32) {
                const int n = idx % TILE, m = idx / TILE;
                if (m >= M || n >= rows) continue;
                float sum = 0.0f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; ++w2) sum += sums[w2 * COLS * LD + m * LD + n];
                Y[(int64_t)m * N + n0 + n] = to_out<OutT>(sum);
            }
        } else {
            // feature 8t + j has its gate in row 16t + j and its up in row 16t + 8 + j; both sums are rounded to
            // bfloat16 as the two separate products of the reference would be, then round(silu(g)) * u as in
            // src/ops/elementwise.cu:47-65
            const int half_n = N >> 1;
            for (int idx = threadIdx.x; idx < 8 * COLS; idx += WARPS * 32) {
                const int j = idx % 8, m = idx / 8;
                const int feature = (n0 >> 1) + j;
                if (m >= M || feature >= half_n || rows < TILE) continue;
                float g = 0.0f, up = 0.0f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; ++w2) {
                    g += sums[w2 * COLS * LD + m * LD + j];
                    up += sums[w2 * COLS * LD + m * LD + j + 8];
                }
                g = round_to<bf16>(g);
                up = round_to<bf16>(up);
                Y[(int64_t)m * half_n + feature] = to_out<OutT>(round_to<bf16>(g / (1.0f + expf(-g))) * up);
            }
        }
        n0 += rows;
    }
    if (n_pieces == 0) pdl_launch_dependents();
    TRACE(5);
}

#ifdef Q3_STREAM_TRACE
}
Q3_EXPORT int q3_stream_trace_set(void* p) { unsigned long long* v = (unsigned long long*)p; return (int)cudaMemcpyToSymbol(g_trace, &v, sizeof(v)); }
namespace {
#endif

template <int MT, int WARPS, int STAGES, bool GATED, typename OutT>
int launch(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int blocks_cap, int early, int* status, cudaStream_t stream) {
    using L = StreamSmem<MT, WARPS, STAGES>;
    static bool configured[64] = {false};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= 64) return Q3_ERR_BAD_SIZE;
    if (!configured[device]) {
        e = cudaFuncSetAttribute(gemm_stream_kernel<MT, WARPS, STAGES, GATED, OutT>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
        configured[device] = true;
    }
    StreamMaps maps;
    for (int i = 0; i < 5; ++i)
        if (!q3_make_map_bf16(&maps.rows[i], W, N, K, TILE >> i, KC, false)) return Q3_ERR_BAD_SIZE;
    const int granules = GATED ? (N + TILE - 1) / TILE : N;
    int blocks = blocks_cap > 0 ? blocks_cap : q3_sm_count();
    if (blocks > granules) blocks = granules;
    return (int)q3_launch(gemm_stream_kernel<MT, WARPS, STAGES, GATED, OutT>, dim3(blocks), dim3(WARPS * 32), (size_t)L::TOTAL,
                          stream, maps, X, Y, M, N, K, early, status);
}

template <bool GATED, typename OutT>
int dispatch(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, int variant, int blocks_cap, int* status,
             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || M > 16 || (GATED && N % 16 != 0)) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    int early = variant >= 10;
    variant %= 10;
#ifdef Q3_STREAM_TRACE
    early |= (blocks_cap >> 16) << 8;      // the launch's row in the trace
    blocks_cap &= 0xFFFF;
#endif
    if (M <= 8) {
        switch (variant) {
            case 1: return launch<1, 8, 4, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 2: return launch<1, 8, 6, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 3: return launch<1, 16, 3, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 4: return launch<1, 4, 6, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 6: return launch<1, 8, 3, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 7: return launch<1, 8, 2, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            case 5: return launch<1, 4, 12, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
            default: return launch<1, 8, 6, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
        }
    }
    return launch<2, 8, 6, GATED, OutT>(X, W, Y, M, N, K, blocks_cap, early, status, stream);
}

}  // namespace

// `variant` and `blocks` choose the block shape and the grid for measurements; 0 takes the defaults.
Q3_EXPORT int q3_gemm_stream_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated,
                                  int variant, int blocks, int* status, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (gated) {
        if (out_is_f32) return Q3_ERR_BAD_SIZE;
        return dispatch<true, bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, variant, blocks, status, s);
    }
    return out_is_f32 ? dispatch<false, float>((const bf16*)X, (const bf16*)W, (float*)Y, M, N, K, variant, blocks, status, s)
                      : dispatch<false, bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, variant, blocks, status, s);
}
