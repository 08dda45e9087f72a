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

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Kernels of this library are launched with
// the attribute that lets the next kernel on the stream start while this one is
// still running.  Every kernel calls pb_grid_dep_launch() as early as it can
// (its dependents may then be placed on free multiprocessors) and
// pb_grid_dep_wait() before it first touches memory that the kernel before it
// on the stream may write or read; the wait returns when that kernel has
// finished and its writes are visible.  What runs before the wait - index
// arithmetic, barrier set-up, reads of data that older kernels produced -
// overlaps the tail of the previous kernel.  A kernel launched without the
// attribute passes both calls at once.  PRELUDE_NO_PDL=1 turns the attribute off.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pb_grid_dep_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pb_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

bool pb_pdl_enabled();   // common.cu

template <typename... KArgs, typename... Args>
static inline cudaError_t pb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = pb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------
// Layout of a key/value page: [pages, kv heads, page_size tokens, head_dim].
// One head's tokens of one page are one contiguous run, so an attention kernel
// fetches them with a single bulk copy.  When `swizzle` is set (bfloat16 pages
// with head_dim % 64 == 0), the 16-byte chunks of every token row are stored
// permuted: chunk c of the row of token r lives at chunk position c ^ (r & 7).
// Copied as they are into shared memory, eight consecutive rows then put any
// one logical chunk into eight different bank groups, so the tensor-core loads
// (ldmatrix) are free of bank conflicts without padding.  elem_per_chunk is 8
// for bfloat16.  Everyone who touches a page goes through this function.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ int pb_kv_elem_offset(int elem, int token_in_page, int swizzle) {
    return swizzle ? ((((elem >> 3) ^ (token_in_page & 7)) << 3) | (elem & 7)) : elem;
}

// Dispatch a launcher body on an element type code.
#define PB_DISPATCH_DTYPE(code, T, ...)                              \
    do {                                                             \
        if ((code) == PB_F32) { using T = float; __VA_ARGS__; }      \
        else if ((code) == PB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return pb_fail("unknown element type code %d", (int)(code)); \
    } while (0)
