// Shared helpers of the kernel libraries: status codes, the thread-local error text, dtype codes and
// small device functions.  Every exported launcher returns PH_OK or sets the error text and returns a
// non-zero status; nothing here traps or spins without a bound.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

#define PH_OK 0
#define PH_ERR_ARG 1
#define PH_ERR_LAUNCH 2
#define PH_ERR_UNSUPPORTED 3

#define PH_F32 0
#define PH_BF16 1

// A library that compiles another library's source into itself defines PH_EXPORT first (hidden) to keep that
// source's entry points to itself.
#ifndef PH_EXPORT
#define PH_EXPORT extern "C" __attribute__((visibility("default")))
#endif

namespace ph {

inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return PH_OK;
}

inline bool valid_dtype(int d) { return d == PH_F32 || d == PH_BF16; }

// Programmatic dependent launch.  A kernel launched through launch_overlapped may start while the kernel
// before it in the stream is still running: its blocks become resident as soon as every block of that kernel has
// called pdl_launch_dependents() (or exited), run whatever does not depend on that kernel's results (set-up,
// prefetch of weights), and stop at pdl_wait() until that kernel has completed and its writes are visible.  Every
// such kernel calls pdl_wait() before it reads anything a predecessor produced and before it writes global
// memory at all.  PURHIE_PDL=0 in the environment turns the attribute off (the device calls are then no-ops).
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PURHIE_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The first position that the position z sees: z - window + 1 under a window of `window` positions (0: none), and not
// before the start of z's own block under a mask of blocks of `chunk` positions counted from 0 (0: none).
__device__ __forceinline__ int first_seen(int z, int window, int chunk) {
    int lo = (window > 0 && z - window + 1 > 0) ? z - window + 1 : 0;
    if (chunk > 0) {
        const int start = z / chunk * chunk;
        if (start > lo) lo = start;
    }
    return lo;
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every thread gets the result.  The
// order of additions depends on NT only.
template <int NT> __device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < NT / 32) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

// Sum over the block, whatever its size (a multiple of 32, at most 1024): the order of additions depends on the block
// size only.
__device__ __forceinline__ float block_sum_any(float v, float* scratch /* >= 32 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < warps ? scratch[lane] : 0.0f;
    return warp_sum(t);
}

// Four consecutive elements as floats (8 bytes of bfloat16, 16 of float32); the address is aligned to that.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// Eight consecutive elements as floats (16 bytes of bfloat16, 32 of float32), and back; the address is 16-byte aligned.
__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[2 * i] = __low2float(h[i]); v[2 * i + 1] = __high2float(h[i]); }
}
__device__ __forceinline__ void store4(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void store8(float* p, const float* v) { store4(p, v); store4(p + 4, v + 4); }
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
}

}  // namespace ph

// Dispatch on a dtype code: runs BODY with type alias NAME bound to float or __nv_bfloat16.
#define PH_DISPATCH(CODE, NAME, ...)                                  \
    do {                                                              \
        if ((CODE) == PH_F32) { using NAME = float; __VA_ARGS__; }    \
        else { using NAME = __nv_bfloat16; __VA_ARGS__; }             \
    } while (0)

// Every library exports its own copy of this under the library's prefix.
#define PH_DEFINE_LAST_ERROR(PREFIX) \
    PH_EXPORT const char* PREFIX##_last_error() { return ph::error_buffer(); }
