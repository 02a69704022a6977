// True 32-bit matrix product of the check path: Y[M,N] = X[M,K] . W[N,K]^T with float
// operands, fmaf accumulation and no tensor-core mode of reduced precision.
//
// It replaces the reference's single cublasGemmEx call per projection
// (src/ops/linear.cpp:165-193) on the 32-bit path only.  Every output element is the
// sum over k = 0..K-1 in ascending tiles of 16 and ascending order inside a tile,
// whatever M, N or the tile an element falls in, so a row's result does not depend on
// which other rows are in the batch.
//
// The same kernel with bfloat16 operands (32-bit accumulation, bfloat16 or float output)
// takes the bfloat16 products whose width is no multiple of 8, which the tensor-core
// kernels refuse (their 16-byte loads and TMA strides need one).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool VEC4, typename InT, typename OutT>
__global__ void __launch_bounds__(256)
gemm_tn_kernel(const InT* __restrict__ X, const InT* __restrict__ W, OutT* __restrict__ Y, int M, int N, int K,
               int64_t ldx, int64_t ldw, int64_t ldy) {
    __shared__ float Xs[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;  // thread tile: rows ty*4.., cols tx*4..
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    // each thread stages 4 consecutive k of one row of X and one row of W
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
        float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int gm = m0 + lr, gn = n0 + lr, gk = k0 + lk;
        if (gm < M) {
            const InT* p = X + (int64_t)gm * ldx + gk;
            if (VEC4 && gk + 3 < K) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                xv[0] = t.x; xv[1] = t.y; xv[2] = t.z; xv[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (gk + i < K) xv[i] = to_f32<InT>(p[i]);
            }
        }
        if (gn < N) {
            const InT* p = W + (int64_t)gn * ldw + gk;
            if (VEC4 && gk + 3 < K) {
                const float4 t = *reinterpret_cast<const float4*>(p);
                wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (gk + i < K) wv[i] = to_f32<InT>(p[i]);
            }
        }
        __syncthreads();  // the previous tile has been consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            Xs[lk + i][lr] = xv[i];
            Ws[lk + i][lr] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = Xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) Y[(int64_t)gm * ldy + gn] = from_f32<OutT>(acc[i][j]);
        }
    }
}

}  // namespace

Q3_EXPORT int q3_gemm_tn_f32(const float* X, const float* W, float* Y, int M, int N, int K, int64_t ldx, int64_t ldw,
                             int64_t ldy, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return Q3_ERR_BAD_SIZE;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return Q3_ERR_TOO_LARGE;
    const bool vec = aligned16(X) && aligned16(W) && ldx % 4 == 0 && ldw % 4 == 0;
    if (vec)
        return (int)q3_launch(gemm_tn_kernel<true, float, float>, grid, dim3(256), 0, (cudaStream_t)stream, X, W, Y, M, N, K,
                              ldx, ldw, ldy);
    return (int)q3_launch(gemm_tn_kernel<false, float, float>, grid, dim3(256), 0, (cudaStream_t)stream, X, W, Y, M, N, K,
                          ldx, ldw, ldy);
}

// bfloat16 operands of any width, 32-bit accumulation in the same fixed order; Y bfloat16 or float.
Q3_EXPORT int q3_gemm_tn_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldw,
                              int64_t ldy, int out_is_f32, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return Q3_ERR_BAD_SIZE;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return Q3_ERR_TOO_LARGE;
    if (out_is_f32)
        return (int)q3_launch(gemm_tn_kernel<false, bf16, float>, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)X,
                              (const bf16*)W, (float*)Y, M, N, K, ldx, ldw, ldy);
    return (int)q3_launch(gemm_tn_kernel<false, bf16, bf16>, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)X,
                          (const bf16*)W, (bf16*)Y, M, N, K, ldx, ldw, ldy);
}
