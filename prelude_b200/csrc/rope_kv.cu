// Fused per-head q/k RMSNorm + rotary position encoding + paged key/value write.
//
// For every token t and head h of the projected q, k and v rows:
//   q' = rope(rmsnorm_D(q) * wq, pos_t)   -> q_out[t, h, :]
//   k' = rope(rmsnorm_D(k) * wk, pos_t)   -> k_pages[page, h, pos % page_size, :]
//   v                                      -> v_pages[page, h, pos % page_size, :]
// with page = block_table[seq_t, pos / page_size].  Norm and rotation are in
// float32 with one rounding at the end, like the reference's fused kernels
// (crates/prelude-cuda/src/kernels/kernels_src/rope/qknorm_rope.cu:49-90,
//  crates/prelude-cuda/src/kernels/kernels_src/kvcache/knorm_rope_kv_write.cu:17-113,
//  crates/prelude-cuda/src/kernels/kernels_src/kvcache/scatter_kv_cache.cu:32-46);
// here q, k and v are handled by one launch.  The rotation pairs element j with
// j + rotary_dim/2 (crates/prelude-core/src/models/commons/attn_utils.rs:52-59);
// elements from rotary_dim on pass through.  cos/sin are float32 tables
// [max_positions, rotary_dim/2].
//
// One warp per (token, head).  Norm weights and the tables may be null: no
// norm, no rotation.  A page id outside [0, num_pages) is never written; the
// kernel raises *status instead.
#include "common.cuh"

template <typename T>
__global__ void qknorm_rope_kvwrite_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long token_stride,
    T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim, int max_positions,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
    int n_tokens, int n_heads, int n_kv_heads, int head_dim, int write_kv, int swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    const int heads_per_token = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp_id >= (long long)n_tokens * heads_per_token) return;
    const int t = (int)(warp_id / heads_per_token);
    const int slot = (int)(warp_id % heads_per_token);
    const int pos = positions[t];

    const T* src;
    T* dst;
    const float* weight;
    bool rotate;
    int swz = 0, in_page = 0;           // page rows may be stored with permuted 16-byte chunks
    if (slot < n_heads) {
        src = q + (size_t)t * token_stride + (size_t)slot * head_dim;
        dst = q_out + ((size_t)t * n_heads + slot) * head_dim;
        weight = q_weight;
        rotate = true;
    } else {
        const bool is_k = slot < n_heads + n_kv_heads;
        const int h = is_k ? slot - n_heads : slot - n_heads - n_kv_heads;
        const int seq = token_seq[t];
        const int page = block_table[(size_t)seq * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages || pos < 0) {
            if (lane == 0 && status) atomicExch(status, 2);
            return;
        }
        in_page = pos % page_size;
        swz = swizzle;
        const size_t row = (((size_t)page * n_kv_heads + h) * page_size + in_page) * head_dim;
        src = (is_k ? k : v) + (size_t)t * token_stride + (size_t)h * head_dim;
        dst = (is_k ? k_pages : v_pages) + row;
        weight = is_k ? k_weight : nullptr;
        rotate = is_k;
        if (!is_k) {   // values: plain copy
            for (int i = lane; i < head_dim; i += 32) dst[pb_kv_elem_offset(i, in_page, swz)] = src[i];
            return;
        }
    }

    float inv = 1.f;
    if (weight != nullptr) {
        float ss = 0.f;
        for (int i = lane; i < head_dim; i += 32) {
            float a = pb_ld(src + i);
            ss += a * a;
        }
        ss = pb_warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
    }
    const bool do_rope = rotate && cos_table != nullptr && rotary_dim > 0;
    const int half = do_rope ? rotary_dim / 2 : 0;
    if (do_rope && (pos < 0 || pos >= max_positions)) {
        if (lane == 0 && status) atomicExch(status, 3);
        return;
    }
    for (int j = lane; j < half; j += 32) {
        float a = pb_ld(src + j) * inv, b = pb_ld(src + j + half) * inv;
        if (weight != nullptr) { a *= weight[j]; b *= weight[j + half]; }
        float c = cos_table[(size_t)pos * half + j], s = sin_table[(size_t)pos * half + j];
        pb_st(dst + pb_kv_elem_offset(j, in_page, swz), a * c - b * s);
        pb_st(dst + pb_kv_elem_offset(j + half, in_page, swz), b * c + a * s);
    }
    for (int i = 2 * half + lane; i < head_dim; i += 32) {
        float a = pb_ld(src + i) * inv;
        if (weight != nullptr) a *= weight[i];
        pb_st(dst + pb_kv_elem_offset(i, in_page, swz), a);
    }
}

PB_API int pb_qknorm_rope_kvwrite(
    const void* q, const void* k, const void* v, long long token_stride, void* q_out, void* k_pages, void* v_pages,
    int dtype, const float* q_weight, const float* k_weight, float eps, const float* cos_table,
    const float* sin_table, int rotary_dim, int max_positions, const int32_t* positions, const int32_t* token_seq,
    const int32_t* block_table, int table_stride, int page_size, int num_pages, int n_tokens, int n_heads,
    int n_kv_heads, int head_dim, int write_kv, int swizzle, int* status, cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0, "qknorm_rope_kvwrite: bad sizes");
    PB_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
               "qknorm_rope_kvwrite: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    PB_REQUIRE(q && q_out && positions, "qknorm_rope_kvwrite: null pointer");
    PB_REQUIRE(!swizzle || (dtype == PB_BF16 && head_dim % 64 == 0), "qknorm_rope_kvwrite: permuted pages are bfloat16 with head_dim %% 64 == 0");
    if (write_kv)
        PB_REQUIRE(k && v && k_pages && v_pages && token_seq && block_table && page_size > 0 && num_pages > 0,
                   "qknorm_rope_kvwrite: cache write asked for without cache arguments");
    if (n_tokens == 0) return 0;
    long long warps = (long long)n_tokens * (n_heads + (write_kv ? 2 * n_kv_heads : 0));
    const int threads = 256;
    long long blocks = (warps * 32 + threads - 1) / threads;
    PB_REQUIRE(blocks < (1ll << 31), "qknorm_rope_kvwrite: too many rows");
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(qknorm_rope_kvwrite_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, stream, 
            (const T*)q, (const T*)k, (const T*)v, token_stride, (T*)q_out, (T*)k_pages, (T*)v_pages, q_weight,
            k_weight, eps, cos_table, sin_table, rotary_dim, max_positions, positions, token_seq, block_table,
            table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, head_dim, write_kv, swizzle, status)));
    PB_CHECK_LAUNCH("qknorm_rope_kvwrite");
    return 0;
}
