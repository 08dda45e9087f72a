// Plain paged attention: one warp per (query token, query head), any head size
// up to 256, float32 or bfloat16 storage, float32 arithmetic throughout.
//
// It is the attention of the 32-bit path, the fallback of the bfloat16 path
// for shapes the tensor-core kernels refuse, and the oracle the fast kernels
// are tested against.  It serves prompt portions and decoded tokens alike: a
// query at absolute position p of request r sees the keys of r at positions
// max(0, p - window + 1) .. p, which are all in the cache because a step
// writes its keys before it attends
// (crates/prelude-core/src/models/qwen3.rs:191-222; mask and softmax after
//  crates/prelude-core/src/ops/traits/attention.rs:30-81).
//
// Keys are visited in blocks of 32 aligned to absolute positions, in ascending
// order, with a running maximum and sum.  The blocks, and so the order of every
// floating-point operation, depend on the query's position and the window only:
// not on how the tokens were cut into steps, not on the batch, not on the pages.
#include "common.cuh"

#include <math.h>

#define ATTN_REF_MAX_D 256
#define ATTN_REF_WARPS 4

template <typename T>
__global__ void paged_attention_warp_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ out,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages, int n_tokens,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float q_s[ATTN_REF_WARPS][ATTN_REF_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * ATTN_REF_WARPS + warp;
    if (item >= (long long)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item % n_heads);
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int seq = token_seq[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int32_t* table = block_table + (size_t)seq * table_stride;

    const T* qrow = q + ((size_t)t * n_heads + h) * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_s[warp][i] = pb_ld(qrow + i);
    __syncwarp();

    float o[ATTN_REF_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < ATTN_REF_MAX_D / 32; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool bad = false;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j >= lo && j <= pos;
        float s = -INFINITY;
        int slot = -1;
        if (valid) {
            const int page = table[j / page_size];
            if (page < 0 || page >= num_pages) {
                bad = true;
            } else {
                slot = (page * n_kv_heads + kvh) * page_size + j % page_size;    // row of this head's run in the page
                const T* kr = k_pages + (size_t)slot * head_dim;
                float acc = 0.f;
                const int in_page = j % page_size;
                for (int d = 0; d < head_dim; ++d) acc = fmaf(q_s[warp][d], pb_ld(kr + pb_kv_elem_offset(d, in_page, swizzle)), acc);
                s = acc * scale;
            }
        }
        const float bm = pb_warp_max(s);
        const float m_new = fmaxf(m, bm);
        if (m_new == -INFINITY) continue;   // only when every page id of the block was bad
        const float p = (slot >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + pb_warp_sum(p);
#pragma unroll
        for (int i = 0; i < ATTN_REF_MAX_D / 32; ++i) o[i] *= corr;
        const int n_in_block = min(32, pos - base + 1);
        for (int jj = 0; jj < n_in_block; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int sj = __shfl_sync(0xffffffffu, slot, jj);
            if (sj < 0) continue;
            const T* vr = v_pages + (size_t)sj * head_dim;
            const int vin = (base + jj) % page_size;
#pragma unroll
            for (int i = 0; i < ATTN_REF_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) o[i] = fmaf(pj, pb_ld(vr + pb_kv_elem_offset(d, vin, swizzle)), o[i]);
            }
        }
        m = m_new;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0 && status) atomicExch(status, 4);
    T* orow = out + ((size_t)t * n_heads + h) * head_dim;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < ATTN_REF_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) pb_st(orow + d, o[i] * inv);
    }
}

// q, out: [n_tokens, n_heads, head_dim]; pages: [num_pages, n_kv_heads, page_size, head_dim];
// positions, token_seq: [n_tokens]; block_table: [n_seqs, table_stride]; window <= 0: all keys.
PB_API int pb_paged_attention_ref(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                  const int32_t* positions, const int32_t* token_seq, const int32_t* block_table,
                                  int table_stride, int page_size, int num_pages, int n_tokens, int n_heads,
                                  int n_kv_heads, int head_dim, float scale, int window, int swizzle, int* status,
                                  cudaStream_t stream) {
    PB_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
               "paged_attention_ref: %d query heads over %d key/value heads", n_heads, n_kv_heads);
    PB_REQUIRE(head_dim > 0 && head_dim <= ATTN_REF_MAX_D, "paged_attention_ref: head_dim=%d not in 1..%d", head_dim,
               ATTN_REF_MAX_D);
    PB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "paged_attention_ref: bad cache geometry");
    if (n_tokens == 0) return 0;
    long long items = (long long)n_tokens * n_heads;
    long long blocks = (items + ATTN_REF_WARPS - 1) / ATTN_REF_WARPS;
    PB_REQUIRE(blocks < (1ll << 31), "paged_attention_ref: too many rows");
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(paged_attention_warp_kernel<T>, dim3((unsigned)blocks), dim3(ATTN_REF_WARPS * 32), 0, stream, 
            (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, positions, token_seq, block_table,
            table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, head_dim, scale, window, swizzle, status)));
    PB_CHECK_LAUNCH("paged_attention_ref");
    return 0;
}
