// Shared helpers of the sm_100a kernel library.
//
// Every launcher is an `extern "C"` function that takes raw device pointers,
// sizes and a stream, checks its arguments, launches, and returns 0 or a
// non-zero code after storing a message that pb_last_error() returns.  A
// launcher never allocates and never synchronises.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define PB_API extern "C" __attribute__((visibility("default")))

// element type codes of the C interface
enum PbDtype : int { PB_F32 = 0, PB_BF16 = 1 };

// error plumbing (defined in common.cu)
int pb_fail(const char* fmt, ...);
#define PB_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) return pb_fail(__VA_ARGS__); \
    } while (0)
#define PB_CHECK_LAUNCH(name)                                                   \
    do {                                                                        \
        cudaError_t e_ = cudaGetLastError();                                    \
        if (e_ != cudaSuccess) return pb_fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

static inline bool pb_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------
// device-side element access: everything is computed in float
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float pb_ld(const T* p);
template <> __device__ __forceinline__ float pb_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float pb_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void pb_st(T* p, float v);
template <> __device__ __forceinline__ void pb_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void pb_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float pb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float pb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Dispatch a launcher body on an element type code.
#define PB_DISPATCH_DTYPE(code, T, ...)                              \
    do {                                                             \
        if ((code) == PB_F32) { using T = float; __VA_ARGS__; }      \
        else if ((code) == PB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return pb_fail("unknown element type code %d", (int)(code)); \
    } while (0)
