// SiLU-gated product on a merged gate/up projection:
//   out[t, i] = silu(gu[t, i]) * gu[t, I + i],  silu(g) = g / (1 + exp(-g))
// computed in float32 (crates/prelude-cuda/src/kernels/kernels_src/elementwise/silu_mul.cu:27-32).
// The merged layout is the reference's gate_up projection, gate rows first
// (crates/prelude-core/src/models/qwen3.rs:411-447).
#include "common.cuh"

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = n_tokens * inter;
    if (idx >= total) return;
    long long t = idx / inter;
    int i = (int)(idx % inter);
    float g = pb_ld(gu + t * 2 * inter + i);
    float u = pb_ld(gu + t * 2 * inter + inter + i);
    pb_st(out + idx, g / (1.0f + expf(-g)) * u);
}

// bfloat16, 8 elements per thread; inter % 8 == 0.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       long long n_tokens, int inter) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = inter / 8;
    if (idx >= n_tokens * per_row) return;
    long long t = idx / per_row;
    int c = (int)(idx % per_row) * 8;
    uint4 graw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + c);
    uint4 uraw = *reinterpret_cast<const uint4*>(gu + t * 2 * inter + inter + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + t * inter + c) = oraw;
}

PB_API int pb_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int inter, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && inter > 0, "silu_mul: bad sizes T=%d I=%d", n_tokens, inter);
    if (n_tokens == 0) return 0;
    const int threads = 256;
    if (dtype == PB_BF16 && inter % 8 == 0 && pb_aligned(gate_up, 16) && pb_aligned(out, 16)) {
        long long n = (long long)n_tokens * (inter / 8);
        pb_launch(silu_mul_bf16x8_kernel, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream, 
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_tokens, inter);
    } else {
        long long n = (long long)n_tokens * inter;
        PB_REQUIRE((n + threads - 1) / threads < (1ll << 31), "silu_mul: too many elements");
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(silu_mul_kernel<T>, dim3((unsigned)((n + threads - 1) / threads)), dim3(threads), 0, stream, 
                (const T*)gate_up, (T*)out, n_tokens, inter)));
    }
    PB_CHECK_LAUNCH("silu_mul");
    return 0;
}
