// Memory-bound kernels around the matrix products: embedding gather, RMSNorm with
// the residual sum fused in, SiLU(gate)*up, and the row gather before the final norm.
// Each is templated on the element type (float for the 32-bit path, bf16 for the
// serving path); sums, means, roots and products are 32-bit in both.
//
// Formulas follow the reference (RicardoMin/Qwen3-Runtime-ByYourself):
//   embedding   src/ops/embedding.cu:38-52    (an id outside the table gives a zero row)
//   RMSNorm     src/ops/rms_norm.cu:87-120    (eps inside the root; round(x*inv) then * w)
//   residual    src/ops/elementwise.cu:30-34  (32-bit sum, stored in the element type)
//   SiLU*up     src/ops/elementwise.cu:47-65  (round(silu(g)) * u)
// The reference runs the sum and the norm as two kernels; here one kernel writes the
// new residual and its normalised copy, so the row is read once.
#include "common.cuh"

template <typename T, int VEC> __device__ __forceinline__ void load_vec(const T* p, float (&v)[VEC]) {
    if constexpr (VEC == 1) {
        v[0] = to_f32<T>(p[0]);
    } else {
        Pack<T> k = load_pack<T>(p);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = k.get(i);
    }
}

template <typename T, int VEC> __device__ __forceinline__ void store_vec(T* p, const float (&v)[VEC]) {
    if constexpr (VEC == 1) {
        p[0] = from_f32<T>(v[0]);
    } else {
        Pack<T> k;
#pragma unroll
        for (int i = 0; i < VEC; ++i) k.set(i, v[i]);
        store_pack<T>(p, k);
    }
}

// ---------------------------------------------------------------- embedding
template <typename T, int VEC>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int hidden, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* src = table + (int64_t)(ok ? id : 0) * hidden;
    T* dst = out + t * hidden;
    for (int c = threadIdx.x * VEC; c < hidden; c += blockDim.x * VEC) {
        float v[VEC];
        if (ok) {
            load_vec<T, VEC>(src + c, v);
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = 0.0f;
        }
        store_vec<T, VEC>(dst + c, v);
    }
}

template <typename T>
static int embedding_launch(const int* ids, const T* table, T* out, int64_t n_tokens, int hidden, int vocab,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    constexpr int V = Pack<T>::N;
    const bool vec = hidden % V == 0 && aligned16(table) && aligned16(out);
    const int threads = 128;
    if (vec)
        return (int)q3_launch(embedding_kernel<T, V>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, ids, table, out,
                              hidden, vocab);
    return (int)q3_launch(embedding_kernel<T, 1>, dim3((unsigned)n_tokens), dim3(threads), 0, stream, ids, table, out,
                          hidden, vocab);
}

// ---------------------------------------------------------------- RMSNorm (+ residual sum)
// One block per row.  If `delta` is given: residual[row] = residual[row] + delta[row]
// (stored in T), and the norm reads the stored sum.  y may alias nothing else.
template <typename T, int VEC>
__global__ void rms_norm_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ w,
                                T* __restrict__ y, int size, float eps, int64_t x_stride, int64_t y_stride) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = blockIdx.x;
    T* xr = x + row * x_stride;
    const T* dr = delta ? delta + row * x_stride : nullptr;
    T* yr = y + row * y_stride;
    float sq = 0.0f;
    for (int c = threadIdx.x * VEC; c < size; c += blockDim.x * VEC) {
        float v[VEC];
        load_vec<T, VEC>(xr + c, v);
        if (dr) {
            float d[VEC];
            load_vec<T, VEC>(dr + c, d);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = round_to<T>(v[i] + d[i]);
            store_vec<T, VEC>(xr + c, v);
        }
#pragma unroll
        for (int i = 0; i < VEC; ++i) sq += v[i] * v[i];
    }
    const float total = block_sum(sq, scratch);
    const float inv = rsqrtf(total / (float)size + eps);
    for (int c = threadIdx.x * VEC; c < size; c += blockDim.x * VEC) {
        float v[VEC];
        load_vec<T, VEC>(xr + c, v);  // own writes of the first pass: same thread, same addresses
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = round_to<T>(v[i] * inv) * w[c + i];
        store_vec<T, VEC>(yr + c, v);
    }
}

// The same for rows that fit the registers of a block: every thread keeps PER packets of its row, so
// the row is read once (twice with `delta`) and written once (twice); used for prompts, where the norms
// are bound by memory traffic.  A block walks rows (blockIdx.x, += gridDim.x) and asks for the packets
// of its next row before it reduces the current one, so that loads are in flight across the barriers.
template <typename T, int PER>
__global__ void rms_norm_reg_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ w,
                                    T* __restrict__ y, int64_t rows, int size, float eps, int64_t x_stride,
                                    int64_t y_stride) {
    constexpr int VEC = Pack<T>::N;
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    Pack<T> xin[PER], din[PER];
    auto fetch = [&](int64_t row) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * VEC;
            if (c < size) {
                xin[p] = load_pack<T>(x + row * x_stride + c);
                if (delta) din[p] = load_pack<T>(delta + row * x_stride + c);
            }
        }
    };
    int64_t row = blockIdx.x;
    if (row < rows) fetch(row);
    for (; row < rows; row += gridDim.x) {
        T* xr = x + row * x_stride;
        T* yr = y + row * y_stride;
        float v[PER][VEC];
        float sq = 0.0f;
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * VEC;
            if (c < size) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[p][i] = delta ? round_to<T>(xin[p].get(i) + din[p].get(i)) : xin[p].get(i);
                if (delta) store_vec<T, VEC>(xr + c, v[p]);
#pragma unroll
                for (int i = 0; i < VEC; ++i) sq += v[p][i] * v[p][i];
            }
        }
        if (row + gridDim.x < rows) fetch(row + gridDim.x);          // under the reduction and the stores below
        const float inv = rsqrtf(block_sum(sq, scratch) / (float)size + eps);
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int c = (p * blockDim.x + threadIdx.x) * VEC;
            if (c < size) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[p][i] = round_to<T>(v[p][i] * inv) * w[c + i];
                store_vec<T, VEC>(yr + c, v[p]);
            }
        }
    }
}

template <typename T>
static int rms_norm_launch(T* x, const T* delta, const float* w, T* y, int64_t rows, int size, float eps,
                           int64_t x_stride, int64_t y_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (size <= 0) return Q3_ERR_BAD_SIZE;
    constexpr int V = Pack<T>::N;
    const bool vec = size % V == 0 && x_stride % V == 0 && y_stride % V == 0 && aligned16(x) && aligned16(y) &&
                     (delta == nullptr || aligned16(delta));
    if (vec && rows >= 64) {
        const int packs = size / V;
        const int per = (packs + 255) / 256;                       // packets a thread keeps
        const int threads = ((packs + per - 1) / per + 31) / 32 * 32;
        auto launch = [&](auto kernel) {
            int sms = 0, device = 0, per_sm = 0;                      // blocks the GPU holds at once
            cudaGetDevice(&device);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0);
            const int64_t resident = (int64_t)(sms > 0 ? sms : 1) * (per_sm > 0 ? per_sm : 1);
            const unsigned blocks = (unsigned)(rows < resident ? rows : resident);
            return (int)q3_launch(kernel, dim3(blocks), dim3(threads), 0, stream, x, delta, w, y, rows, size, eps, x_stride,
                                  y_stride);
        };
        if (per == 1) return launch(rms_norm_reg_kernel<T, 1>);
        if (per == 2) return launch(rms_norm_reg_kernel<T, 2>);
        if (per <= 4) return launch(rms_norm_reg_kernel<T, 4>);
    }
    const int per = vec ? V : 1;
    int threads = (size / per + 31) / 32 * 32;
    threads = threads < 32 ? 32 : (threads > 512 ? 512 : threads);
    if (vec)
        return (int)q3_launch(rms_norm_kernel<T, V>, dim3((unsigned)rows), dim3(threads), 0, stream, x, delta, w, y, size,
                              eps, x_stride, y_stride);
    return (int)q3_launch(rms_norm_kernel<T, 1>, dim3((unsigned)rows), dim3(threads), 0, stream, x, delta, w, y, size, eps,
                          x_stride, y_stride);
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gate_up: [rows, 2*inter]; out: [rows, inter].  Two layouts of a row: the gate in the first
// `inter` columns and the up values in the rest, or (interleaved) blocks of eight gate
// columns followed by the eight up columns of the same features.
template <typename T, int VEC>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t rows, int inter,
                                int interleaved) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t per_row = inter / VEC;
    const int64_t total = rows * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row;
        const int c = (int)(i % per_row) * VEC;
        float g[VEC], u[VEC];
        const int64_t gate_at = interleaved ? (int64_t)(c >> 3) * 16 + (c & 7) : c;
        const int64_t up_at = interleaved ? gate_at + 8 : (int64_t)inter + c;
        load_vec<T, VEC>(gate_up + r * 2 * inter + gate_at, g);
        load_vec<T, VEC>(gate_up + r * 2 * inter + up_at, u);
#pragma unroll
        for (int k = 0; k < VEC; ++k) g[k] = round_to<T>(g[k] / (1.0f + expf(-g[k]))) * u[k];
        store_vec<T, VEC>(out + r * inter + c, g);
    }
}

template <typename T>
static int silu_mul_launch(const T* gate_up, T* out, int64_t rows, int inter, int interleaved, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || (interleaved && inter % 8 != 0)) return Q3_ERR_BAD_SIZE;
    constexpr int V = Pack<T>::N;
    const bool vec = inter % V == 0 && aligned16(gate_up) && aligned16(out);
    const int threads = 256;
    const int64_t work = rows * (inter / (vec ? V : 1));
    int64_t blocks = (work + threads - 1) / threads;
    const int64_t resident = (int64_t)q3_device_sm_count() * 16;       // blocks of 128 threads an SM holds
    if (blocks > resident) blocks = resident;
    if (vec)
        return (int)q3_launch(silu_mul_kernel<T, V>, dim3((unsigned)blocks), dim3(threads), 0, stream, gate_up, out, rows,
                              inter, interleaved);
    return (int)q3_launch(silu_mul_kernel<T, 1>, dim3((unsigned)blocks), dim3(threads), 0, stream, gate_up, out, rows, inter,
                          interleaved);
}

// ---------------------------------------------------------------- gather rows (+ pending branch)
// out[r] = x[idx[r]] (+ delta[idx[r]]): the rows whose logits are wanted, with the
// last branch output added in 32-bit.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, const T* __restrict__ delta, const int* __restrict__ idx,
                                   T* __restrict__ out, int size) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t r = blockIdx.x;
    const int64_t src = idx[r];
    for (int c = threadIdx.x; c < size; c += blockDim.x) {
        float v = to_f32<T>(x[src * size + c]);
        if (delta) v += to_f32<T>(delta[src * size + c]);
        out[r * size + c] = from_f32<T>(v);
    }
}

template <typename T>
static int gather_rows_launch(const T* x, const T* delta, const int* idx, T* out, int64_t rows, int size,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    return (int)q3_launch(gather_rows_kernel<T>, dim3((unsigned)rows), dim3(256), 0, stream, x, delta, idx, out, size);
}

// ---------------------------------------------------------------- rows of a checkpoint tensor into their place (load time)
// dst row = dst_row0 + (r / block_rows) * dst_block_stride + r % block_rows for source row r, converted from S to
// D on the way (bfloat16 -> float32 exactly, float32 -> bfloat16 by rounding).  With block_rows = the row count it
// is a copy of consecutive rows (the q, k and v matrices into one); with block_rows 8 and a stride of 16 it
// interleaves the gate rows (dst_row0 0) and the up rows (dst_row0 8) of a feed-forward in blocks of eight.
template <typename S, typename D>
__global__ void place_rows_kernel(const S* __restrict__ src, D* __restrict__ dst, int64_t rows, int64_t cols,
                                  int64_t block_rows, int64_t dst_block_stride, int64_t dst_row0) {
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i % cols;
        const int64_t to = dst_row0 + (r / block_rows) * dst_block_stride + r % block_rows;
        dst[to * cols + c] = from_f32<D>(to_f32<S>(src[i]));
    }
}

template <typename S, typename D>
static int place_rows_launch(const void* src, void* dst, int64_t rows, int64_t cols, int64_t block_rows,
                             int64_t dst_block_stride, int64_t dst_row0, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (block_rows <= 0 || dst_block_stride < block_rows || dst_row0 < 0) return Q3_ERR_BAD_SIZE;
    const int threads = 256;
    int64_t blocks = (rows * cols + threads - 1) / threads;
    const int64_t resident = (int64_t)q3_device_sm_count() * 8;
    if (blocks > resident) blocks = resident;
    return (int)q3_launch(place_rows_kernel<S, D>, dim3((unsigned)blocks), dim3(threads), 0, stream, (const S*)src, (D*)dst, rows,
                          cols, block_rows, dst_block_stride, dst_row0);
}

// src_kind / dst_kind: 0 = float32, 1 = bfloat16.
Q3_EXPORT int q3_place_rows(const void* src, int src_kind, void* dst, int dst_kind, int64_t rows, int64_t cols,
                            int64_t block_rows, int64_t dst_block_stride, int64_t dst_row0, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (src_kind == 0 && dst_kind == 0) return place_rows_launch<float, float>(src, dst, rows, cols, block_rows, dst_block_stride, dst_row0, s);
    if (src_kind == 0 && dst_kind == 1) return place_rows_launch<float, bf16>(src, dst, rows, cols, block_rows, dst_block_stride, dst_row0, s);
    if (src_kind == 1 && dst_kind == 0) return place_rows_launch<bf16, float>(src, dst, rows, cols, block_rows, dst_block_stride, dst_row0, s);
    if (src_kind == 1 && dst_kind == 1) return place_rows_launch<bf16, bf16>(src, dst, rows, cols, block_rows, dst_block_stride, dst_row0, s);
    return Q3_ERR_BAD_SIZE;
}

// ---------------------------------------------------------------- exported entry points
#define Q3_ELEMENTWISE_EXPORTS(SUFFIX, T)                                                                          \
    Q3_EXPORT int q3_embedding_##SUFFIX(const int* ids, const void* table, void* out, int64_t n_tokens, int hidden, \
                                        int vocab, void* stream) {                                                  \
        return embedding_launch<T>(ids, (const T*)table, (T*)out, n_tokens, hidden, vocab, (cudaStream_t)stream);   \
    }                                                                                                               \
    Q3_EXPORT int q3_rms_norm_##SUFFIX(void* x, const void* delta, const float* w, void* y, int64_t rows, int size, \
                                       float eps, int64_t x_stride, int64_t y_stride, void* stream) {               \
        return rms_norm_launch<T>((T*)x, (const T*)delta, w, (T*)y, rows, size, eps, x_stride, y_stride,            \
                                  (cudaStream_t)stream);                                                            \
    }                                                                                                               \
    Q3_EXPORT int q3_silu_mul_##SUFFIX(const void* gate_up, void* out, int64_t rows, int inter, int interleaved,    \
                                       void* stream) {                                                              \
        return silu_mul_launch<T>((const T*)gate_up, (T*)out, rows, inter, interleaved, (cudaStream_t)stream);      \
    }                                                                                                               \
    Q3_EXPORT int q3_gather_rows_##SUFFIX(const void* x, const void* delta, const int* idx, void* out, int64_t rows, \
                                          int size, void* stream) {                                                 \
        return gather_rows_launch<T>((const T*)x, (const T*)delta, idx, (T*)out, rows, size, (cudaStream_t)stream); \
    }

Q3_ELEMENTWISE_EXPORTS(f32, float)
Q3_ELEMENTWISE_EXPORTS(bf16, bf16)
