// Shared device helpers of the sm_100a kernels: element conversion, reductions,
// 16-byte vector access.  Every exported entry point is `extern "C"`, takes raw
// device pointers plus the stream to launch on, allocates nothing, and returns
// the cudaError_t of its launch as an int (0 = success).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

#define Q3_EXPORT extern "C" __attribute__((visibility("default")))

// Tokens per page of the key/value cache.  The build passes the cache's own constant
// (-DQ3_PAGE_TOKENS=<cache.book.PAGE_TOKENS>); the attention kernels are tiled for 64.
#ifndef Q3_PAGE_TOKENS
#define Q3_PAGE_TOKENS 64
#endif

// Multiprocessors of the current device (asked once per device).
static inline int q3_device_sm_count() {
    static int counts[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
    if (counts[device] == 0) cudaDeviceGetAttribute(&counts[device], cudaDevAttrMultiProcessorCount, device);
    return counts[device] > 0 ? counts[device] : 1;
}

// Raises a kernel's limit of dynamic shared memory, once per device (the attribute belongs to the device's
// copy of the kernel).  `done` is a static array of the call site.
struct Q3PerDevice {
    bool done[64] = {};
};
template <typename Kernel>
static inline cudaError_t q3_allow_shared_memory(Kernel kernel, int bytes, Q3PerDevice& state) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (state.done[device]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) state.done[device] = true;
    return e;
}

// Error codes of argument checks, above the cudaError_t range.
#define Q3_ERR_BAD_SIZE 10001
#define Q3_ERR_TOO_LARGE 10002
#define Q3_ERR_MISALIGNED 10003

// ---- programmatic dependent launch ------------------------------------------------------
// Kernels of a step run back to back on one stream.  Launched with the programmatic
// attribute, a kernel may start while its predecessor drains: it does what needs no input
// of the predecessor (address arithmetic, fetching weights) and then waits in `pdl_wait()`,
// which returns once the predecessor has completed and its writes are visible.  Rules that
// every kernel here keeps: `pdl_launch_dependents()` first thing, and no read of an
// activation and no write to global memory before `pdl_wait()`.  Without the attribute
// both calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static int g_q3_pdl = 0;
// Switches the programmatic attribute on or off for the launches of this library.
Q3_EXPORT void q3_set_pdl(int on) { g_q3_pdl = on; }

template <typename... KArgs, typename... Args>
static inline cudaError_t q3_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_q3_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a kernel whose blocks form thread-block clusters of `cluster` blocks.
template <typename... KArgs, typename... Args>
static inline cudaError_t q3_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_q3_pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Rounds a 32-bit value to the storage type and back: the identity for float,
// one bfloat16 rounding for bf16.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 33 floats.  Every thread
// gets the result.  The order of the additions is fixed by the thread layout.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// A 16-byte packet of elements of type T.
template <typename T> struct Pack;
template <> struct Pack<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
    __device__ __forceinline__ void set(int i, float v) { (&raw.x)[i] = v; }
};
template <> struct Pack<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ float get(int i) const {
        return __bfloat162float(reinterpret_cast<const bf16*>(&raw)[i]);
    }
    __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<bf16*>(&raw)[i] = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ Pack<T> load_pack(const T* p) {
    Pack<T> r;
    r.raw = *reinterpret_cast<const decltype(r.raw)*>(p);
    return r;
}
template <typename T> __device__ __forceinline__ void store_pack(T* p, const Pack<T>& v) {
    *reinterpret_cast<decltype(v.raw)*>(p) = v.raw;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
