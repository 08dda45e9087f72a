// Embedding gather: res[t, :] = table[ids[t], :], written as float32 because
// it opens the residual stream, which is kept in 32-bit.
//
// Counterpart in the reference: index_select of the embedding table
// (crates/prelude-core/src/models/commons/embedding.rs:29-35).
#include "common.cuh"

template <typename T>
__global__ void embed_gather_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                    float* __restrict__ out, int n_tokens, int width, int vocab) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    int t = blockIdx.x;
    if (t >= n_tokens) return;
    int id = ids[t];
    float* dst = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {   // the host validates ids; never read out of bounds
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const T* src = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = pb_ld(src + i);
}

// bfloat16 rows, 8 elements per thread and access; needs width % 8 == 0.
__global__ void embed_gather_bf16x8_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                           float* __restrict__ out, int n_tokens, int width, int vocab) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    int t = blockIdx.x;
    if (t >= n_tokens) return;
    int id = ids[t];
    bool ok = id >= 0 && id < vocab;
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * width);
    float4* dst = reinterpret_cast<float4*>(out + (size_t)t * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
        uint4 raw = ok ? src[i] : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
        dst[2 * i] = make_float4(a.x, a.y, b.x, b.y);
        dst[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
}

PB_API int pb_embed_gather(const int32_t* ids, const void* table, int table_dtype, float* out,
                           int n_tokens, int width, int vocab, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && width > 0 && vocab > 0, "embed_gather: bad sizes T=%d H=%d V=%d", n_tokens, width, vocab);
    if (n_tokens == 0) return 0;
    int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == PB_BF16 && width % 8 == 0 && pb_aligned(table, 16) && pb_aligned(out, 16)) {
        pb_launch(embed_gather_bf16x8_kernel, dim3(n_tokens), dim3(threads), 0, stream, 
            ids, (const __nv_bfloat16*)table, out, n_tokens, width, vocab);
    } else {
        PB_DISPATCH_DTYPE(table_dtype, T,
            (pb_launch(embed_gather_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, ids, (const T*)table, out, n_tokens, width, vocab)));
    }
    PB_CHECK_LAUNCH("embed_gather");
    return 0;
}
