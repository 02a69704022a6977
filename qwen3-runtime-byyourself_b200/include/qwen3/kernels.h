// qwen3/kernels.h - the C interface of the library's sm_100a kernels, for host programs that drive them
// without Python.  Each group of entry points lives in a shared library of its own, built from the source
// named beside it (csrc/, nvcc -gencode arch=compute_100a,code=sm_100a); the attention libraries are
// compiled for one head size (-DQ3_HEAD_DIM=<multiple of 16>).
//
// Conventions, the same everywhere:
//   * pointers are device pointers unless a comment says otherwise; `stream` is a cudaStream_t;
//   * nothing allocates: scratch is passed in (q3_attention_decode_bf16_static keeps its own, see
//     csrc/attention_decode_static.h);
//   * the result is 0, a cudaError_t of the launch, or one of the argument errors below - a size the kernel
//     does not take is refused, never computed wrongly;
//   * matrices are row-major; weights are [out, in] and used as x . W^T; bfloat16 values are passed as
//     `void*`; rows of activations are contiguous;
//   * the cache is paged: k_pages / v_pages [pages, kv heads, 64 tokens, head size]; page_table [sequences,
//     pages_per_seq] lists a sequence's pages in order; token_seq / token_pos give every token's sequence and
//     position; seq_start [sequences + 1] and seq_pos0 [sequences] describe packed prompts;
//   * `status` is one int32 word on the device into which a kernel whose bounded wait ran out writes where it
//     gave up (0 = none); read it where the host waits for the device anyway.
//
// The reference's counterparts: src/ops/{embedding,rms_norm,rope,elementwise,gqa_attention,argmax}.cu, the
// cublasGemmEx call of src/ops/linear.cpp:165-193, the CPU sampler of src/generation/sampler.cpp:137-247.
#pragma once

#include <stdint.h>

#define Q3_ERR_BAD_SIZE 10001        /* a size the kernel does not take */
#define Q3_ERR_TOO_LARGE 10002       /* more rows, heads or blocks than one launch takes */
#define Q3_ERR_MISALIGNED 10003      /* a pointer or stride that is not 16-byte aligned */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- elementwise.cu: float32 (`f32`) and bfloat16 (`bf16`) forms ---------------------------------------- */
/* out[t] = table[ids[t]] (a zero row for an id outside [0, vocab)) */
int q3_embedding_f32(const int* ids, const void* table, void* out, int64_t n_tokens, int hidden, int vocab, void* stream);
int q3_embedding_bf16(const int* ids, const void* table, void* out, int64_t n_tokens, int hidden, int vocab, void* stream);
/* if delta: x += delta (32-bit sum, stored in x's type); y = round(x * rsqrt(mean(x^2) + eps)) * w */
int q3_rms_norm_f32(void* x, const void* delta, const float* w, void* y, int64_t rows, int size, float eps, int64_t x_stride,
                    int64_t y_stride, void* stream);
int q3_rms_norm_bf16(void* x, const void* delta, const float* w, void* y, int64_t rows, int size, float eps, int64_t x_stride,
                     int64_t y_stride, void* stream);
/* out = round(silu(gate)) * up; a row of gate_up holds the gate then the up values, or (interleaved) blocks of 8 + 8 */
int q3_silu_mul_f32(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, void* stream);
int q3_silu_mul_bf16(const void* gate_up, void* out, int64_t rows, int inter, int interleaved, void* stream);
/* out[r] = x[idx[r]] (+ delta[idx[r]]) */
int q3_gather_rows_f32(const void* x, const void* delta, const int* idx, void* out, int64_t rows, int size, void* stream);
int q3_gather_rows_bf16(const void* x, const void* delta, const int* idx, void* out, int64_t rows, int size, void* stream);
/* load time: rows of src into dst with conversion (kinds: 0 float32, 1 bfloat16); source row r goes to row
   dst_row0 + (r / block_rows) * dst_block_stride + r % block_rows */
int q3_place_rows(const void* src, int src_kind, void* dst, int dst_kind, int64_t rows, int64_t cols, int64_t block_rows,
                  int64_t dst_block_stride, int64_t dst_row0, void* stream);

/* ---- attention.cu: every head size in steps of 16 up to 256, float32 and bfloat16 ------------------------ */
/* per-head RMSNorm of q and k (weights may be null), rotation of the first rotary_dim values of a head (0: all of
   them; tables [positions, rotary_dim/2], may be null), and the write of k and v into their pages (write_kv = 0: q only) */
int q3_qkv_prepare_f32(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* q_norm_w, const float* k_norm_w,
                       const float* cos_tab, const float* sin_tab, const int* token_seq, const int* token_pos, const int* page_table,
                       int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d, float eps, int write_kv, int rotary_dim, void* stream);
int q3_qkv_prepare_bf16(const void* qkv, void* q_out, void* k_pages, void* v_pages, const float* q_norm_w, const float* k_norm_w,
                        const float* cos_tab, const float* sin_tab, const int* token_seq, const int* token_pos, const int* page_table,
                        int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d, float eps, int write_kv, int rotary_dim, void* stream);
/* causal grouped-query attention of every token over its sequence's pages; window 0 = every key */
int q3_attention_generic_f32(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_seq,
                             const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d,
                             float scale, int window, void* stream);
int q3_attention_generic_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_seq,
                              const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv, int d,
                              float scale, int window, void* stream);

/* ---- attention_decode.cu (-DQ3_HEAD_DIM): one new token per sequence, bfloat16 ---------------------------- */
int q3_attention_decode_head_dim(void);
int64_t q3_attention_decode_scratch_floats(int64_t n_tokens, int nq, int n_splits);
/* split over the keys + merge; scratch: q3_attention_decode_scratch_floats(...) float32 */
int q3_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, float* scratch, const int* token_seq,
                             const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv,
                             float scale, int window, int n_splits, void* stream);
/* the whole attention of a decode step from the q/k/v projection's output: norm, rotation, cache write, attention,
   merge of up to 8 splits inside a thread-block cluster; no scratch */
int q3_attention_decode_fused_max_splits(void);   /* 16 where clusters of 16 blocks can be placed, else 8 */
int q3_attention_decode_fused_bf16(const void* qkv, void* k_pages, void* v_pages, void* out, const float* q_norm_w,
                                   const float* k_norm_w, const float* cos_tab, const float* sin_tab, float eps, const int* token_seq,
                                   const int* token_pos, const int* page_table, int pages_per_seq, int64_t n_tokens, int nq, int nkv,
                                   float scale, int window, int n_splits, int write_kv, int rotary_dim, void* stream);

/* ---- attention_prefill.cu, attention_prefill_tc.cu (-DQ3_HEAD_DIM): prompts, bfloat16 --------------------- */
int q3_attention_prefill_head_dim(void);
int q3_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                              const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new, int nq, int nkv,
                              float scale, int window, void* stream);
int q3_attention_prefill_tc_head_dim(void);
/* both products on tcgen05 (head sizes 64 and 128, no window) */
int q3_attention_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_start,
                                 const int* seq_pos0, const int* page_table, int pages_per_seq, int n_seqs, int max_new,
                                 int64_t n_tokens, int64_t n_cache_pages, int nq, int nkv, float scale, int* status, void* stream);

/* ---- matrix products Y[M, N] = X[M, K] . W[N, K]^T -------------------------------------------------------- */
/* gemm_f32.cu: true 32-bit (fmaf, ascending k); and bfloat16 operands of any width on the CUDA cores */
int q3_gemm_tn_f32(const float* X, const float* W, float* Y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, void* stream);
int q3_gemm_tn_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, int out_is_f32,
                    void* stream);
/* gemm_skinny_bf16.cu: up to 64 rows, W streamed once; `gated`: W holds gate and up rows interleaved in blocks of
   eight and Y is [M, N / 2] = round(silu(g)) * u */
int q3_gemm_skinny_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
int q3_gemm_skinny_bf16_f32out(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
int q3_gemm_skinny_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, void* stream);
/* gemm_tcgen05.cu: TMA + tcgen05; weights first with K split over a cluster (`mid`), tokens first on single SMs
   (`prompt`, tile_n 128 or 256) and on pairs of SMs (`pair`) */
int q3_gemm_tcgen05_mid_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated, int splits,
                             int* status, void* stream);
int q3_gemm_tcgen05_mid_splits(int N, int K, int M);
int q3_gemm_tcgen05_prompt_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int tile_n, int* status,
                                void* stream);
int q3_gemm_tcgen05_prompt_gated_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int* status, void* stream);
/* the q/k/v product of a prompt step with q3_qkv_prepare's work in its epilogue: W [(nq + 2 nkv) d, K]; q to q_out
   [M, nq d], k and v (write_kv) to the pages; d 64, 128 or 256; norm weights and whole-head tables may be null */
int q3_gemm_tcgen05_pair_qkv_bf16(const void* X, const void* W, int M, int K, void* q_out, void* k_pages, void* v_pages,
                                  const float* q_norm_w, const float* k_norm_w, const float* cos_tab, const float* sin_tab, float eps,
                                  const int* token_seq, const int* token_pos, const int* page_table, int pages_per_seq, int nq,
                                  int nkv, int d, int write_kv, int* status, void* stream);
/* splits 1..4: K split over that many pairs of SMs of one cluster (1: persistent pairs, no split) */
int q3_gemm_tcgen05_pair_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int out_is_f32, int gated, int splits,
                              int* status, void* stream);
int q3_gemm_tcgen05_pair_capacity(int splits);

/* ---- sampling.cu ------------------------------------------------------------------------------------------ */
/* out[r] = index of the highest logit among the first `valid` (lowest id among equals, NaN as -inf) */
int q3_argmax_f32(const float* logits, int64_t stride, int rows, int valid, int* out, void* stream);
/* temperature -> top-k (ties stay) -> order by score then id -> softmax -> top-p -> inverse CDF; the uniform number of
   row r is a hash of (seed, seq_ids[r], steps ? steps[r] : step_all); out[r] = -1 for a row with a non-finite logit */
int q3_sample_f32(const float* logits, int64_t stride, int rows, int valid, float temperature, int top_k, float top_p, uint64_t seed,
                  const int64_t* seq_ids, const int* steps, int step_all, int* out, void* stream);

/* every library: programmatic dependent launch for its kernels on (1) or off (0, the default) */
void q3_set_pdl(int on);

#ifdef __cplusplus
}
#endif
