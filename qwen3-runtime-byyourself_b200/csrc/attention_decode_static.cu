// The allocation-free variant of the decode attention (see attention_decode_static.h for
// who needs it and for the rules of use).  The kernels are the ones of attention_decode.cu,
// included below unchanged; only the home of the scratch differs: a fixed device array of
// this file instead of a buffer from the caller.
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "attention_decode.cu"
#include "attention_decode_static.h"

namespace {

// The splits' partial sums and (max, sum) pairs meet here.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a pointer a kernel could use.
static __device__ __align__(256) float g_static_scratch[Q3_DECODE_STATIC_MAX_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_address[MAX_DEVICES];      // device address of the array, per device, once looked up
std::atomic<bool> g_device_ready[MAX_DEVICES];
std::mutex g_prepare_mutex;

// First call on the current device: find the array's device address and raise the kernel's
// shared-memory limit.  Neither allocates.  Not meant to run under stream capture.  Host threads
// that make their first call at the same time take turns here; the flag is published last.
int prepare_device(int device) {
    std::lock_guard<std::mutex> lock(g_prepare_mutex);
    if (g_device_ready[device].load(std::memory_order_acquire)) return 0;
    float* address = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&address, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(decode_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    g_scratch_address[device] = address;
    g_device_ready[device].store(true, std::memory_order_release);
    return 0;
}

// n_tokens * nq * n_splits * (D + 2) <= limit, checked factor by factor so that no product can wrap.
bool fits_static_scratch(int64_t n_tokens, int nq, int n_splits) {
    int64_t room = Q3_DECODE_STATIC_MAX_FLOATS / (D + 2);
    if (n_tokens > room) return false;
    room /= n_tokens;
    if (nq > room) return false;
    room /= nq;
    return n_splits <= room;
}

}  // namespace

Q3_EXPORT int q3_attention_decode_bf16_static(const void* q, const void* k_pages, const void* v_pages, void* out,
                                              const int* token_seq, const int* token_pos, const int* page_table,
                                              int pages_per_seq, int64_t n_tokens, int nq, int nkv, float scale,
                                              int window, int n_splits, void* stream_) {
    if (n_tokens <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || nq / nkv > 16 || n_splits <= 0) return Q3_ERR_BAD_SIZE;
    if (n_tokens > 65535 || nkv > 65535 || n_splits > 65535) return Q3_ERR_TOO_LARGE;
    if (!fits_static_scratch(n_tokens, nq, n_splits)) {
        fprintf(stderr,
                "q3_attention_decode_bf16_static: %lld tokens x %d heads x %d splits x (%d + 2) float32 of "
                "scratch, the built-in array holds %d; use fewer splits or tokens, or q3_attention_decode_bf16 with "
                "a scratch buffer of your own\n",
                (long long)n_tokens, nq, n_splits, D, Q3_DECODE_STATIC_MAX_FLOATS);
        return Q3_ERR_STATIC_SCRATCH;
    }
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) return Q3_ERR_BAD_SIZE;
    if (!g_device_ready[device].load(std::memory_order_acquire)) {
        const int rc = prepare_device(device);
        if (rc != 0) return rc;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    float* part_o = g_scratch_address[device];
    float* part_ml = part_o + n_tokens * nq * n_splits * D;
    const dim3 grid(n_splits, nkv, (unsigned)n_tokens);
    e = q3_launch(decode_split_kernel<false>, grid, dim3(WARPS * 32), SMEM_BYTES, stream, (const bf16*)q, (const bf16*)k_pages,
                  (const bf16*)v_pages, part_o, part_ml, token_seq, token_pos, page_table, pages_per_seq, nq, nkv,
                  scale * 1.4426950408889634f, window, FusedArgs{});
    if (e != cudaSuccess) return (int)e;
    return (int)q3_launch(decode_merge_kernel, dim3(nq, (unsigned)n_tokens), dim3(D < 128 ? 32 : 128), 0, stream,
                          (const float*)part_o, (const float*)part_ml, (bf16*)out, nq, n_splits);
}
