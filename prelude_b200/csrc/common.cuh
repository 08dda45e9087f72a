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

// ---------------------------------------------------------------------------
// A timeline of a step's kernels, for looking at what happens between them
// (compiled in with -DPB_TIMELINE, which PRELUDE_TIMELINE=1 asks the build
// for; without it the marks are nothing).  A source file that has marks says
// PB_TIMELINE_UNIT(name) once: that gives it the pointer to the record and
// the exported setter pb_timeline_set_<name>.  PB_TL(kernel, mark) then stores
// the device-wide nanosecond clock, by thread 0 of the grid's first and of
// its last block: word 0 of the record counts the entries, entry = kernel (8
// bits) | mark (4) | last block (1) | time (51 bits).
// ---------------------------------------------------------------------------
#ifdef PB_TIMELINE
#define PB_TL_CAP 8192
__device__ __forceinline__ void pb_tl_mark(unsigned long long* tl, int kernel, int mark) {
    if (tl == nullptr || threadIdx.x != 0) return;
    const bool first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    const bool last = blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1 && blockIdx.z == gridDim.z - 1;
    if (!first && !last) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    const unsigned i = atomicAdd(reinterpret_cast<unsigned*>(tl), 1u);
    if (i < PB_TL_CAP)
        tl[1 + i] = ((unsigned long long)(kernel & 0xff) << 56) | ((unsigned long long)(mark & 0xf) << 52) |
                    ((unsigned long long)(first ? 0 : 1) << 51) | (t & 0x7FFFFFFFFFFFFull);
}
#define PB_TIMELINE_UNIT(name)                                                                   \
    static __device__ unsigned long long* g_pb_tl = nullptr;                                     \
    PB_API int pb_timeline_set_##name(unsigned long long* record) {                              \
        return cudaMemcpyToSymbol(g_pb_tl, &record, sizeof(record)) == cudaSuccess ? 0 : 1;      \
    }
#define PB_TL(kernel, mark) pb_tl_mark(g_pb_tl, kernel, mark)
#else
#define PB_TIMELINE_UNIT(name)
#define PB_TL(kernel, mark) do { } while (0)
#endif
enum PbTimelineKernel : int { PB_TL_NORM = 1, PB_TL_GEMM_STREAM = 2, PB_TL_ROPE = 3, PB_TL_ATTN_DECODE = 4 };
enum PbTimelineMark : int { PB_TL_ENTRY = 0, PB_TL_AFTER_WAIT = 1, PB_TL_INPUT = 2, PB_TL_DONE = 3, PB_TL_EXIT = 4 };

// Dispatch a launcher body on an element type code.
#define PB_DISPATCH_DTYPE(code, T, ...)                              \
    do {                                                             \
        if ((code) == PB_F32) { using T = float; __VA_ARGS__; }      \
        else if ((code) == PB_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return pb_fail("unknown element type code %d", (int)(code)); \
    } while (0)
