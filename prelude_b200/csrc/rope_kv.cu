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
// j + rotary_dim/2 (crates/prelude-core/src/models/commons/attn_utils.rs:52-59),
// or, with `interleaved`, element 2j with 2j + 1 (what architectures with
// adjacent pairs need; the position part says which); elements from rotary_dim
// on pass through.  cos/sin are float32 tables [max_positions, rotary_dim/2].
//
// One warp per (token, head) in the general kernel.  bfloat16 rows whose head
// size is a power of two up to 256 take the vector kernel: 16 bytes per lane,
// head_dim / 8 lanes per (token, head) and several of those per warp; the two
// halves of a rotation pair sit in two lanes of the group and are exchanged by
// a shuffle; every row is read once.  Norm weights and the tables may be null:
// no norm, no rotation.  A page id outside [0, num_pages) is never written; the
// kernel raises *status instead.  A token whose token_seq entry is negative is a
// padding row (a captured step is as long as its bucket): nothing is written for it.
#include "common.cuh"

template <typename T>
__global__ void qknorm_rope_kvwrite_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long token_stride,
    T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim, int interleaved, int max_positions,
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
    if (token_seq != nullptr && token_seq[t] < 0) return;      // a padding row of a captured step: nothing to do
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
        const int ia = interleaved ? 2 * j : j, ib = interleaved ? 2 * j + 1 : j + half;      // the pair that angle j turns
        float a = pb_ld(src + ia) * inv, b = pb_ld(src + ib) * inv;
        if (weight != nullptr) { a *= weight[ia]; b *= weight[ib]; }
        float c = cos_table[(size_t)pos * half + j], s = sin_table[(size_t)pos * half + j];
        pb_st(dst + pb_kv_elem_offset(ia, in_page, swz), a * c - b * s);
        pb_st(dst + pb_kv_elem_offset(ib, in_page, swz), b * c + a * s);
    }
    for (int i = 2 * half + lane; i < head_dim; i += 32) {
        float a = pb_ld(src + i) * inv;
        if (weight != nullptr) a *= weight[i];
        pb_st(dst + pb_kv_elem_offset(i, in_page, swz), a);
    }
}

PB_TIMELINE_UNIT(rope)

// The vector kernel: LANES = head_dim / 8 lanes per (token, head), 8 elements each.
template <int LANES>
__global__ void __launch_bounds__(256) qknorm_rope_kvwrite_vec_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    long long token_stride, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
    __nv_bfloat16* __restrict__ v_pages, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim, int interleaved, int max_positions,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
    int n_tokens, int n_heads, int n_kv_heads, int write_kv, int swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_ROPE, PB_TL_ENTRY);
    constexpr int D = LANES * 8;
    const int heads_per_token = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;     // (token, head) of this lane
    const int c = threadIdx.x % LANES;                                                       // its 16-byte chunk
    const bool live = group < (long long)n_tokens * heads_per_token;
    // lanes without a row keep going (the shuffles below are warp-wide) on row 0 and store nothing
    const int t = live ? (int)(group / heads_per_token) : 0;
    const int slot = live ? (int)(group % heads_per_token) : 0;
    // Positions, block tables, norm scales and the rotation tables were written before this step's first kernel
    // started: everything that depends on them alone is fetched before the wait for the kernel ahead (which
    // writes q, k and v).
    const int pos = positions[t];
    const bool padding = token_seq != nullptr && token_seq[t] < 0;                           // a padding row of a captured step
    const bool is_q = slot < n_heads, is_k = !is_q && slot < n_heads + n_kv_heads;
    const int h = is_q ? slot : (is_k ? slot - n_heads : slot - n_heads - n_kv_heads);
    const __nv_bfloat16* src = (is_q ? q : is_k ? k : v) + (size_t)t * token_stride + (size_t)h * D + c * 8;
    __nv_bfloat16* dst = nullptr;
    bool store = live && !padding;
    if (is_q) {
        dst = q_out + ((size_t)t * n_heads + h) * D + c * 8;
    } else if (!padding) {
        const int seq = token_seq[t];
        const int page = pos >= 0 ? block_table[(size_t)seq * table_stride + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (live && c == 0 && status) atomicExch(status, 2);
            store = false;
        } else {
            const int in_page = pos % page_size;
            const int cc = swizzle ? (c ^ (in_page & 7)) : c;                                // chunks of a page row may be permuted
            dst = (is_k ? k_pages : v_pages) + (((size_t)page * n_kv_heads + h) * page_size + in_page) * D + cc * 8;
        }
    }
    const float* weight = is_q ? q_weight : (is_k ? k_weight : nullptr);
    float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
    if (weight != nullptr) {
        w0 = *reinterpret_cast<const float4*>(weight + c * 8);
        w1 = *reinterpret_cast<const float4*>(weight + c * 8 + 4);
    }
    // rotation: element j of the first half pairs with j + half; the partner chunk sits half / 8 lanes away
    const int half = (cos_table != nullptr) ? rotary_dim / 2 : 0;
    const int hc = half / 8;                                                                 // chunks per half (0: no rotation)
    // interleaved pairs (2j, 2j + 1) lie inside one lane's chunk: the chunk of elements 8c.. takes angles 4c..4c+3
    const bool first = interleaved ? (c * 8 < 2 * half) : (c < hc), second = !interleaved && c >= hc && c < 2 * hc;
    const bool rotates = (first || second) && (is_q || is_k);
    float4 c0 = make_float4(1.f, 1.f, 1.f, 1.f), c1 = c0, s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (rotates && !padding) {
        if (pos < 0 || pos >= max_positions) {
            if (live && c == 0 && status) atomicExch(status, 3);
            store = false;
        } else if (interleaved) {
            c0 = *reinterpret_cast<const float4*>(cos_table + (size_t)pos * half + c * 4);   // four angles for four pairs
            s0 = *reinterpret_cast<const float4*>(sin_table + (size_t)pos * half + c * 4);
        } else {
            const int j0 = (first ? c : c - hc) * 8;
            const float* cp = cos_table + (size_t)pos * half + j0;
            const float* sp = sin_table + (size_t)pos * half + j0;
            c0 = *reinterpret_cast<const float4*>(cp); c1 = *reinterpret_cast<const float4*>(cp + 4);
            s0 = *reinterpret_cast<const float4*>(sp); s1 = *reinterpret_cast<const float4*>(sp + 4);
        }
    }
    pb_grid_dep_wait();
    PB_TL(PB_TL_ROPE, PB_TL_AFTER_WAIT);
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    if (!is_q && !is_k) {                                                                    // values: plain copy
        if (store) *reinterpret_cast<uint4*>(dst) = raw;
        // no return: the lanes of this warp that hold q or k rows need all lanes at the shuffles
    }
    float x[8];
    {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h2[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);       // over the lanes of the row
    if (weight != nullptr) {
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
        x[0] *= inv * w0.x; x[1] *= inv * w0.y; x[2] *= inv * w0.z; x[3] *= inv * w0.w;
        x[4] *= inv * w1.x; x[5] *= inv * w1.y; x[6] *= inv * w1.z; x[7] *= inv * w1.w;
    }
    const int partner = interleaved ? c : (first ? c + hc : (second ? c - hc : c));
    const int src_lane = (threadIdx.x & 31) - c + partner;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = __shfl_sync(0xffffffffu, x[i], src_lane);
    if (rotates && interleaved) {
        const float cs[4] = {c0.x, c0.y, c0.z, c0.w}, sn[4] = {s0.x, s0.y, s0.z, s0.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float a = x[2 * m], b = x[2 * m + 1];
            x[2 * m] = a * cs[m] - b * sn[m];
            x[2 * m + 1] = b * cs[m] + a * sn[m];
        }
    } else if (rotates) {
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = first ? x[i] * cs[i] - y[i] * sn[i] : x[i] * cs[i] + y[i] * sn[i];
    }
    if (store && (is_q || is_k)) {
        uint4 out;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst) = out;
    }
    PB_TL(PB_TL_ROPE, PB_TL_DONE);
}

// The vector kernel for the many tokens of a prompt step: LANES lanes per (token, G consecutive heads).  What
// depends on the token alone - position, page, angles - is looked up once for the G heads, and their G loads are in
// flight together; with one head per lane group (the kernel above) a step of 2,048 tokens spends its time in the
// chains of dependent look-ups of 1.5 million threads (23.7 us for 50 MB), which is what a decode step's few rows
// want but not this.
template <int LANES, int G>
__global__ void __launch_bounds__(256) qknorm_rope_kvwrite_heads_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    long long token_stride, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
    __nv_bfloat16* __restrict__ v_pages, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rotary_dim, int interleaved, int max_positions,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int table_stride, int page_size, int num_pages,
    int n_tokens, int n_heads, int n_kv_heads, int write_kv, int swizzle, int* __restrict__ status) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_ROPE, PB_TL_ENTRY);
    constexpr int D = LANES * 8;
    const int heads_per_token = n_heads + (write_kv ? 2 * n_kv_heads : 0);
    const int groups_per_token = (heads_per_token + G - 1) / G;
    const long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;      // (token, group of heads) of this lane
    const int c = threadIdx.x % LANES;                                                       // its 16-byte chunk
    const bool live = unit < (long long)n_tokens * groups_per_token;
    // lanes without a unit keep going (the shuffles below are warp-wide) on token 0 and store nothing
    const int t = live ? (int)(unit / groups_per_token) : 0;
    const int slot0 = live ? (int)(unit % groups_per_token) * G : 0;
    const int pos = positions[t];
    const bool padding = token_seq != nullptr && token_seq[t] < 0;                           // a padding row of a captured step
    // the token's place in the cache, if this group has keys or values
    bool page_ok = false;
    size_t page_row = 0;
    int in_page = 0;
    if (write_kv && slot0 + G > n_heads && !padding) {
        const int seq = token_seq[t];
        const int page = pos >= 0 ? block_table[(size_t)seq * table_stride + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (live && c == 0 && status) atomicExch(status, 2);
        } else {
            page_ok = true;
            in_page = pos % page_size;
            page_row = (size_t)page * n_kv_heads;
        }
    }
    const int cc = swizzle ? (c ^ (in_page & 7)) : c;                                        // chunks of a page row may be permuted
    // rotation: element j of the first half pairs with j + half; the partner chunk sits half / 8 lanes away
    const int half = (cos_table != nullptr) ? rotary_dim / 2 : 0;
    const int hc = half / 8;
    const bool first = interleaved ? (c * 8 < 2 * half) : (c < hc), second = !interleaved && c >= hc && c < 2 * hc;
    const bool rotates = first || second;
    bool pos_ok = true;
    float4 c0 = make_float4(1.f, 1.f, 1.f, 1.f), c1 = c0, s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
    if (rotates && !padding && slot0 < n_heads + (write_kv ? n_kv_heads : 0)) {              // the group has queries or keys
        if (pos < 0 || pos >= max_positions) {
            if (live && c == 0 && status) atomicExch(status, 3);
            pos_ok = false;
        } else if (interleaved) {
            c0 = *reinterpret_cast<const float4*>(cos_table + (size_t)pos * half + c * 4);
            s0 = *reinterpret_cast<const float4*>(sin_table + (size_t)pos * half + c * 4);
        } else {
            const int j0 = (first ? c : c - hc) * 8;
            const float* cp = cos_table + (size_t)pos * half + j0;
            const float* sp = sin_table + (size_t)pos * half + j0;
            c0 = *reinterpret_cast<const float4*>(cp); c1 = *reinterpret_cast<const float4*>(cp + 4);
            s0 = *reinterpret_cast<const float4*>(sp); s1 = *reinterpret_cast<const float4*>(sp + 4);
        }
    }
    const int partner = interleaved ? c : (first ? c + hc : (second ? c - hc : c));
    const int src_lane = (threadIdx.x & 31) - c + partner;
    pb_grid_dep_wait();
    PB_TL(PB_TL_ROPE, PB_TL_AFTER_WAIT);
    uint4 raw[G];
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int slot = slot0 + i < heads_per_token ? slot0 + i : slot0;
        const bool is_q = slot < n_heads, is_k = !is_q && slot < n_heads + n_kv_heads;
        const int h = is_q ? slot : (is_k ? slot - n_heads : slot - n_heads - n_kv_heads);
        raw[i] = *reinterpret_cast<const uint4*>((is_q ? q : is_k ? k : v) + (size_t)t * token_stride + (size_t)h * D + c * 8);
    }
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const bool valid = slot0 + i < heads_per_token;
        const int slot = valid ? slot0 + i : slot0;
        const bool is_q = slot < n_heads, is_k = !is_q && slot < n_heads + n_kv_heads;
        const int h = is_q ? slot : (is_k ? slot - n_heads : slot - n_heads - n_kv_heads);
        bool store = live && valid && !padding;
        __nv_bfloat16* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * n_heads + h) * D + c * 8;
        } else {
            store = store && page_ok;
            dst = (is_k ? k_pages : v_pages) + ((page_row + h) * page_size + in_page) * D + cc * 8;
        }
        if (!is_q && !is_k) {                                                                // values: plain copy
            if (store) *reinterpret_cast<uint4*>(dst) = raw[i];
            store = false;                           // no `continue`: the shuffles below are warp-wide
        }
        float x[8];
        {
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
            for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h2[j]); x[2 * j] = f.x; x[2 * j + 1] = f.y; }
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // over the lanes of the row
        const float* weight = is_q ? q_weight : (is_k ? k_weight : nullptr);
        if (weight != nullptr) {
            const float4 w0 = *reinterpret_cast<const float4*>(weight + c * 8), w1 = *reinterpret_cast<const float4*>(weight + c * 8 + 4);
            const float inv = 1.0f / sqrtf(ss / (float)D + eps);
            x[0] *= inv * w0.x; x[1] *= inv * w0.y; x[2] *= inv * w0.z; x[3] *= inv * w0.w;
            x[4] *= inv * w1.x; x[5] *= inv * w1.y; x[6] *= inv * w1.z; x[7] *= inv * w1.w;
        }
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = __shfl_sync(0xffffffffu, x[j], src_lane);
        if (rotates && (is_q || is_k)) {
            if (!pos_ok) store = false;
            if (interleaved) {
                const float cs[4] = {c0.x, c0.y, c0.z, c0.w}, sn[4] = {s0.x, s0.y, s0.z, s0.w};
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const float a = x[2 * m], b = x[2 * m + 1];
                    x[2 * m] = a * cs[m] - b * sn[m];
                    x[2 * m + 1] = b * cs[m] + a * sn[m];
                }
            } else {
                const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = first ? x[j] * cs[j] - y[j] * sn[j] : x[j] * cs[j] + y[j] * sn[j];
            }
        }
        if (store) {
            uint4 out;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
            *reinterpret_cast<uint4*>(dst) = out;
        }
    }
    PB_TL(PB_TL_ROPE, PB_TL_DONE);
}

#define PB_ROPE_HEADS_PER_UNIT 8
// tokens from which a step takes the form above; below, one head per lane group: a decode step's rows are few and
// want every lane
static int g_rope_heads_min_tokens = 256;
PB_API int pb_rope_set_heads_min_tokens(int n) {
    const int before = g_rope_heads_min_tokens;
    if (n > 0) g_rope_heads_min_tokens = n;
    return before;
}

template <int LANES, typename... Args>
static void launch_rope_heads(int n_tokens, int heads_per_token, cudaStream_t stream, Args... args) {
    const int threads = 256;
    const long long units = (long long)n_tokens * ((heads_per_token + PB_ROPE_HEADS_PER_UNIT - 1) / PB_ROPE_HEADS_PER_UNIT);
    const long long blocks = (units * LANES + threads - 1) / threads;
    pb_launch(qknorm_rope_kvwrite_heads_kernel<LANES, PB_ROPE_HEADS_PER_UNIT>, dim3((unsigned)blocks), dim3(threads), 0, stream, args...);
}

template <int LANES, typename... Args>
static void launch_rope_vec(long long rows, cudaStream_t stream, Args... args) {
    const int threads = 256;
    const long long blocks = (rows * LANES + threads - 1) / threads;
    pb_launch(qknorm_rope_kvwrite_vec_kernel<LANES>, dim3((unsigned)blocks), dim3(threads), 0, stream, args...);
}

PB_API int pb_qknorm_rope_kvwrite(
    const void* q, const void* k, const void* v, long long token_stride, void* q_out, void* k_pages, void* v_pages,
    int dtype, const float* q_weight, const float* k_weight, float eps, const float* cos_table,
    const float* sin_table, int rotary_dim, int interleaved, int max_positions, const int32_t* positions, const int32_t* token_seq,
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
    // the vector kernel: bfloat16, a power-of-two head size from 16 to 256, rotation halves of whole 16-byte
    // chunks, everything 16-byte aligned
    const bool pow2 = head_dim >= 16 && head_dim <= 256 && (head_dim & (head_dim - 1)) == 0;
    const bool rot_ok = cos_table == nullptr || rotary_dim % 16 == 0;
    const bool aligned = pb_aligned(q, 16) && pb_aligned(q_out, 16) && token_stride % 8 == 0 &&
                         (!write_kv || (pb_aligned(k, 16) && pb_aligned(v, 16) && pb_aligned(k_pages, 16) && pb_aligned(v_pages, 16))) &&
                         (q_weight == nullptr || pb_aligned(q_weight, 16)) && (k_weight == nullptr || pb_aligned(k_weight, 16)) &&
                         (cos_table == nullptr || (pb_aligned(cos_table, 16) && pb_aligned(sin_table, 16) && (rotary_dim / 2) % 4 == 0));
    if (dtype == PB_BF16 && pow2 && rot_ok && aligned && warps * (head_dim / 8) < (1ll << 38)) {
        typedef const __nv_bfloat16* CB;
        typedef __nv_bfloat16* B;
#define PB_ROPE_VEC(L)                                                                                                  \
        launch_rope_vec<L>(warps, stream, (CB)q, (CB)k, (CB)v, token_stride, (B)q_out, (B)k_pages, (B)v_pages, q_weight,   \
                           k_weight, eps, cos_table, sin_table, rotary_dim, interleaved, max_positions, positions, token_seq, \
                           block_table, table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, write_kv,        \
                           swizzle, status)
        const int heads_per_token = n_heads + (write_kv ? 2 * n_kv_heads : 0);
        if (n_tokens >= g_rope_heads_min_tokens && heads_per_token >= PB_ROPE_HEADS_PER_UNIT && (head_dim == 64 || head_dim == 128)) {
#define PB_ROPE_HEADS(L)                                                                                                \
            launch_rope_heads<L>(n_tokens, heads_per_token, stream, (CB)q, (CB)k, (CB)v, token_stride, (B)q_out, (B)k_pages, \
                                 (B)v_pages, q_weight, k_weight, eps, cos_table, sin_table, rotary_dim, interleaved,       \
                                 max_positions, positions, token_seq, block_table, table_stride, page_size, num_pages,     \
                                 n_tokens, n_heads, n_kv_heads, write_kv, swizzle, status)
            if (head_dim == 64) PB_ROPE_HEADS(8);
            else PB_ROPE_HEADS(16);
#undef PB_ROPE_HEADS
            PB_CHECK_LAUNCH("qknorm_rope_kvwrite");
            return 0;
        }
        if (head_dim == 16) PB_ROPE_VEC(2);
        else if (head_dim == 32) PB_ROPE_VEC(4);
        else if (head_dim == 64) PB_ROPE_VEC(8);
        else if (head_dim == 128) PB_ROPE_VEC(16);
        else PB_ROPE_VEC(32);
#undef PB_ROPE_VEC
        PB_CHECK_LAUNCH("qknorm_rope_kvwrite");
        return 0;
    }
    const int threads = 256;
    long long blocks = (warps * 32 + threads - 1) / threads;
    PB_REQUIRE(blocks < (1ll << 31), "qknorm_rope_kvwrite: too many rows");
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(qknorm_rope_kvwrite_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, stream, 
            (const T*)q, (const T*)k, (const T*)v, token_stride, (T*)q_out, (T*)k_pages, (T*)v_pages, q_weight,
            k_weight, eps, cos_table, sin_table, rotary_dim, interleaved, max_positions, positions, token_seq, block_table,
            table_stride, page_size, num_pages, n_tokens, n_heads, n_kv_heads, head_dim, write_kv, swizzle, status)));
    PB_CHECK_LAUNCH("qknorm_rope_kvwrite");
    return 0;
}
