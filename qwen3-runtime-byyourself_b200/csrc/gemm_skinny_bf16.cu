// Weight-streaming matrix product for decode: Y[M,N] = X[M,K] . W[N,K]^T with a handful of
// rows M (one per sequence of the batch), bfloat16 operands, 32-bit accumulation.
//
// In the reference every projection is one cublasGemmEx call whatever M is
// (src/ops/linear.cpp:165-193).  With M <= 64 the product is bound by reading W once, so
// this kernel is built around that stream: a block owns 16 rows of W and splits K over
// its warps; every lane reads 16 contiguous bytes of a W row per step and feeds them
// straight to the tensor cores as the 16-row operand of mma.m16n8k16, with the batch rows
// as the 8-column operand.  Since a sum over k does not care about the order of k, the
// eight k-values a lane loads are used as they come (both operands permute k the same
// way), so there is no shuffle and no shared-memory staging.  Each warp keeps several
// k-blocks of W in flight in registers, and the first of them are requested before the
// kernel waits for its predecessor (weights do not depend on it), so the stream of W
// starts while the kernel before this one drains.  The warps' partial sums are
// added in shared memory in warp order, which fixes the summation order for every M.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;   // not volatile: the compiler may hoist and batch these loads
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename OutT> __device__ __forceinline__ OutT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 to_out<bf16>(float v) { return __float2bfloat16_rn(v); }

// MT: tiles of 8 batch rows (M <= 8*MT).  R: tiles of 16 rows of W per block.  WARPS: K is split
// over them.  PF: k-blocks (of 32) a warp keeps in flight in registers.  MINB: blocks per SM the
// register budget is held to, so that the whole grid is resident at once for the layer sizes.
// GATED: W holds gate and up rows interleaved in blocks of eight (rows 16t..16t+7 gate, 16t+8..
// 16t+15 up, both for features 8t..8t+7); the kernel then writes round(silu(g)) * u, [M, N/2].
template <int MT, int R, int WARPS, int PF, int MINB, bool GATED, typename OutT>
__global__ void __launch_bounds__(WARPS * 32, MINB)
gemm_skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, OutT* __restrict__ Y, int M, int N, int K) {
    extern __shared__ __align__(16) float red[];   // [WARPS][8*MT][16*R + 1]
    constexpr int ROWS = 16 * R, COLS = 8 * MT, LD = ROWS + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, tq = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int nkb = (K + 31) >> 5;
    const int kb_begin = (int)(((int64_t)warp * nkb) / WARPS), kb_end = (int)(((int64_t)(warp + 1) * nkb) / WARPS);

    float acc[R][MT][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m][0] = acc[r][m][1] = acc[r][m][2] = acc[r][m][3] = 0.0f;

    const bf16* wrow[R][2];
    bool wok[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + r * 16 + h * 8 + quad;
            wok[r][h] = n < N;
            wrow[r][h] = W + (int64_t)(wok[r][h] ? n : 0) * K + tq * 8;
        }
    const bf16* xrow[MT];
    bool xok[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int row = m * 8 + quad;
        xok[m] = row < M;
        xrow[m] = X + (int64_t)(xok[m] ? row : 0) * K + tq * 8;
    }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 w[PF][R][2], x[PF][MT];

    auto load_w = [&](int s, int kb) {
        const int k = kb * 32;
        const bool in = kb < kb_end && k + tq * 8 + 8 <= K;   // K is a multiple of 8: a chunk is inside or outside
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int h = 0; h < 2; ++h) w[s][r][h] = (in && wok[r][h]) ? ld_stream16(wrow[r][h] + k) : zero;
    };
    auto load_x = [&](int s, int kb) {
        const int k = kb * 32;
        const bool in = kb < kb_end && k + tq * 8 + 8 <= K;
#pragma unroll
        for (int m = 0; m < MT; ++m) x[s][m] = (in && xok[m]) ? *reinterpret_cast<const uint4*>(xrow[m] + k) : zero;
    };

    // the weights do not depend on the kernel before this one: fetch the first blocks, then wait for it
#pragma unroll
    for (int s = 0; s < PF; ++s) load_w(s, kb_begin + s);
    pdl_wait();
#pragma unroll
    for (int s = 0; s < PF; ++s) load_x(s, kb_begin + s);

    for (int kb = kb_begin; kb < kb_end; kb += PF) {
#pragma unroll
        for (int s = 0; s < PF; ++s) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16(acc[r][m], w[s][r][0].x, w[s][r][1].x, w[s][r][0].y, w[s][r][1].y, x[s][m].x, x[s][m].y);
                    mma_bf16(acc[r][m], w[s][r][0].z, w[s][r][1].z, w[s][r][0].w, w[s][r][1].w, x[s][m].z, x[s][m].w);
                }
            load_w(s, kb + s + PF);      // blocks past the end load zeros, which add nothing
            load_x(s, kb + s + PF);
        }
    }

    // the stream of W is over: the next kernel may start fetching its own weights while this one adds up
    pdl_launch_dependents();

    // accumulator (row n = quad [+8], column m = 2*tq [+1]) -> red[warp][m][n]
    float* mine = red + warp * COLS * LD;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int n = r * 16 + quad, c = m * 8 + tq * 2;
            mine[c * LD + n] = acc[r][m][0];
            mine[(c + 1) * LD + n] = acc[r][m][1];
            mine[c * LD + n + 8] = acc[r][m][2];
            mine[(c + 1) * LD + n + 8] = acc[r][m][3];
        }
    __syncthreads();
    if constexpr (!GATED) {
        for (int idx = threadIdx.x; idx < ROWS * COLS; idx += WARPS * 32) {
            const int n = idx % ROWS, m = idx / ROWS;
            if (m >= M || n0 + n >= N) continue;
            float sum = 0.0f;
#pragma unroll
            for (int w2 = 0; w2 < WARPS; ++w2) sum += red[w2 * COLS * LD + m * LD + n];
            Y[(int64_t)m * N + n0 + n] = to_out<OutT>(sum);
        }
    } else {
        // feature f = (row tile) * 8 + j has its gate in row 16t + j and its up in row 16t + 8 + j; both
        // sums are rounded to bfloat16 as the two separate products of the reference would be, then
        // round(silu(g)) * u as in src/ops/elementwise.cu:47-65
        constexpr int FEATS = ROWS / 2;
        const int half_n = N >> 1;
        for (int idx = threadIdx.x; idx < FEATS * COLS; idx += WARPS * 32) {
            const int f = idx % FEATS, m = idx / FEATS;
            const int n = (f >> 3) * 16 + (f & 7);
            const int feature = (n0 >> 1) + f;
            if (m >= M || feature >= half_n) continue;
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int w2 = 0; w2 < WARPS; ++w2) {
                g += red[w2 * COLS * LD + m * LD + n];
                u += red[w2 * COLS * LD + m * LD + n + 8];
            }
            g = round_to<bf16>(g);
            u = round_to<bf16>(u);
            Y[(int64_t)m * half_n + feature] = to_out<OutT>(round_to<bf16>(g / (1.0f + expf(-g))) * u);
        }
    }
}

template <int MT, int R, int WARPS, int PF, int MINB, bool GATED, typename OutT>
int launch(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, cudaStream_t stream) {
    constexpr int SMEM = WARPS * 8 * MT * (16 * R + 1) * 4;
    static Q3PerDevice configured;
    if (SMEM > 48 * 1024) {
        cudaError_t e = q3_allow_shared_memory(gemm_skinny_kernel<MT, R, WARPS, PF, MINB, GATED, OutT>, SMEM, configured);
        if (e != cudaSuccess) return (int)e;
    }
    const int blocks = (N + 16 * R - 1) / (16 * R);
    return (int)q3_launch(gemm_skinny_kernel<MT, R, WARPS, PF, MINB, GATED, OutT>, dim3(blocks), dim3(WARPS * 32), SMEM,
                          stream, X, W, Y, M, N, K);
}

// The shapes below come from a sweep over (rows per block, k-blocks in flight, blocks per SM, warps)
// on the projections of an 8B-sized layer at batch 8: 16 rows of W per block always won; matrices of
// few rows (one block per SM or less) want 16 warps sharing K, the others 8 warps and three blocks per SM.
template <bool GATED, typename OutT>
int dispatch(const bf16* X, const bf16* W, OutT* Y, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || M > 64 || (GATED && N % 16 != 0)) return Q3_ERR_BAD_SIZE;
    if (!aligned16(X) || !aligned16(W)) return Q3_ERR_MISALIGNED;
    const bool few_rows = (N + 15) / 16 <= 296;
    if (M <= 8) {
        if (few_rows) return launch<1, 1, 16, 2, 2, GATED, OutT>(X, W, Y, M, N, K, stream);
        // one wave of three blocks per SM: two k-blocks in flight per warp measured a little faster than four
        if ((N + 15) / 16 <= 444) return launch<1, 1, 8, 2, 3, GATED, OutT>(X, W, Y, M, N, K, stream);
        return launch<1, 1, 8, 4, 3, GATED, OutT>(X, W, Y, M, N, K, stream);
    }
    if (M <= 16)
        return few_rows ? launch<2, 1, 16, 2, 1, GATED, OutT>(X, W, Y, M, N, K, stream)
                        : launch<2, 1, 8, 2, 3, GATED, OutT>(X, W, Y, M, N, K, stream);
    // the split of K over warps depends on N alone, so a row's sum has the same order for every M
    if (M <= 32)
        return few_rows ? launch<4, 1, 16, 1, 1, GATED, OutT>(X, W, Y, M, N, K, stream)
                        : launch<4, 1, 8, 2, 2, GATED, OutT>(X, W, Y, M, N, K, stream);
    return few_rows ? launch<8, 1, 16, 1, 1, GATED, OutT>(X, W, Y, M, N, K, stream)
                    : launch<8, 1, 8, 1, 2, GATED, OutT>(X, W, Y, M, N, K, stream);
}

}  // namespace

Q3_EXPORT int q3_gemm_skinny_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream) {
    return dispatch<false, bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, (cudaStream_t)stream);
}

Q3_EXPORT int q3_gemm_skinny_bf16_f32out(const void* X, const void* W, void* Y, int M, int N, int K, void* stream) {
    return dispatch<false, float>((const bf16*)X, (const bf16*)W, (float*)Y, M, N, K, (cudaStream_t)stream);
}

// W [N, K] holds gate and up rows interleaved in blocks of eight; Y [M, N/2] = round(silu(g)) * u.
Q3_EXPORT int q3_gemm_skinny_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream) {
    return dispatch<true, bf16>((const bf16*)X, (const bf16*)W, (bf16*)Y, M, N, K, (cudaStream_t)stream);
}
