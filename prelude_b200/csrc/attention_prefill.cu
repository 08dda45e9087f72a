// Tensor-core paged attention for bfloat16: one kernel for prompt portions, one
// for decode steps with the key range split over several blocks, and the merge
// of the splits.
//
// Both kernels compute, for a query at absolute position p of request r and
// query head h (key/value head h / G):
//     o = softmax_j( (q . k_j) * scale ) v_j    over  max(0, p - window + 1) <= j <= p
// with k_j, v_j read from the request's pages through its block table
// (crates/prelude-core/src/models/qwen3.rs:191-222; the reference hands this to
// FlashAttention-4 / FlashInfer, crates/prelude-cuda/src/attn/flash_v4.rs:125-278).
// Scores and the running softmax (maximum, sum, rescaling) are float32; the
// probabilities are rounded to bfloat16 for the second product, whose
// accumulator is float32.
//
// Layout of the work.  The G query heads that share a key/value head are packed
// into the rows of the tensor-core tile, so keys and values are read once per
// group.  Keys and values come through shared memory in tiles of 64 keys,
// gathered page by page with 16-byte asynchronous copies, double buffered.
//   prefill: a block owns 64 rows = 64/G tokens x G heads of one request and one
//            key/value head; each of its 4 warps owns 16 rows and walks all keys.
//   decode:  a block owns the G rows of one token and one key/value head and a
//            contiguous share of the key tiles; its 4 warps take 16 keys each of
//            every tile and are merged at the end.  With more than one split the
//            block writes an unnormalised partial result (float32) and its
//            running maximum and sum to scratch memory; a merge kernel adds the
//            splits up in ascending order.
// Head sizes: multiples of 16 up to 256 (register arrays are sized for 64, 128
// or 256).  Row strides in shared memory are padded by 16 bytes so that the
// 8 x 16-byte rows of an ldmatrix fall into different banks.
#include "attention_common.cuh"

// ---------------------------------------------------------------------------------------
// prefill: 64 rows (tokens x heads of a group) against all visible keys
// ---------------------------------------------------------------------------------------
template <int DMAX>
__global__ void __launch_bounds__(ATT_THREADS) attn_prefill_kernel(AttnParams p) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    constexpr int STRIDE = DMAX + 8;
    constexpr int KSTEPS = DMAX / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sKV = sQ + 64 * STRIDE;                 // 2 stages x (K, V) x BN rows

    const int G = p.group, d = p.head_dim;
    const int tpt = 64 / G;                                // tokens per tile
    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int r = p.tile_seq[tile], tok0 = p.tile_tok0[tile];
    const int q_base = p.cu_q[r], q_len = p.cu_q[r + 1] - q_base, pos0 = p.q_start[r];
    const int n_tok = min(tpt, q_len - tok0);              // tokens of this tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int32_t* table = p.block_table + (size_t)p.token_seq[q_base + tok0] * p.table_stride;

    // Q rows: row i -> token tok0 + i / G, head kvh * G + i % G
    {
        const int chunks = d >> 3;
        for (int c = threadIdx.x; c < 64 * chunks; c += ATT_THREADS) {
            const int row = c / chunks, ch = c - row * chunks;
            const int tl = row / G, hg = row - tl * G;
            const bool ok = tl < n_tok;
            const size_t src = ok ? (((size_t)(q_base + tok0 + tl) * p.n_heads + kvh * G + hg) * d + ch * 8) : 0;
            cp_async16(sQ + row * STRIDE + ch * 8, p.q + src, ok);
        }
    }
    const int p_min = pos0 + tok0, p_max = pos0 + tok0 + n_tok - 1;
    const int lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt0 = lo / BN, kt1 = p_max / BN;
    const int kv_end = p_max + 1;
    load_kv_tile<DMAX>(sKV, sKV + BN * STRIDE, p, table, kvh, kt0 * BN, lo, kv_end);
    cp_async_commit();

    // this thread's two rows
    int row_pos[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + 8 * h;
        const int tl = row / G;
        row_pos[h] = tl < n_tok ? pos0 + tok0 + tl : -1;    // -1: no key is visible
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int kt = kt0; kt <= kt1; ++kt) {
        const int stage = (kt - kt0) & 1;
        __nv_bfloat16* sK = sKV + stage * 2 * BN * STRIDE;
        __nv_bfloat16* sV = sK + BN * STRIDE;
        if (kt < kt1) {
            __nv_bfloat16* nK = sKV + (stage ^ 1) * 2 * BN * STRIDE;
            load_kv_tile<DMAX>(nK, nK + BN * STRIDE, p, table, kvh, (kt + 1) * BN, lo, kv_end);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        // S = Q K^T : 16 rows x 64 keys per warp
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            if (kk * 16 < d) {
                unsigned a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], sQ + (warp * 16 + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int n2 = 0; n2 < 4; ++n2) {
                    unsigned b0, b1, b2, b3;
                    const int key = n2 * 16 + (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b0, b1, b2, b3, sK + key * STRIDE + col);
                    mma_bf16(s[2 * n2], a, b0, b1);
                    mma_bf16(s[2 * n2 + 1], a, b2, b3);
                }
            }
        }
        // mask, running maximum and sum
        float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kt * BN + nt * 8 + 2 * t4 + (e & 1);
                const int pr = row_pos[e >> 1];
                const bool vis = j <= pr && (p.window <= 0 || j > pr - p.window);
                const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
                s[nt][e] = v;
                rmax[e >> 1] = fmaxf(rmax[e >> 1], v);
            }
        }
        float corr[2], mref[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
            rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
            const float m_new = fmaxf(m[h], rmax[h]);
            corr[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
            mref[h] = (m_new == -INFINITY) ? 0.f : m_new;   // exp2f(-inf - 0) = 0 for rows that see nothing yet
            m[h] = m_new;
            l[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - mref[e >> 1]);
                s[nt][e] = pv;
                l[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < DMAX / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            unsigned a[4] = {pack_bf16(s[2 * ks][0], s[2 * ks][1]), pack_bf16(s[2 * ks][2], s[2 * ks][3]),
                             pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]), pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
            for (int d2 = 0; d2 < KSTEPS; ++d2) {
                if (d2 * 16 < d) {
                    unsigned b0, b1, b2, b3;
                    const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = d2 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sV + key * STRIDE + col);
                    mma_bf16(o[2 * d2], a, b0, b1);
                    mma_bf16(o[2 * d2 + 1], a, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    // normalise and store
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        const int row = warp * 16 + g + 8 * h;
        const int tl = row / G, hg = row - tl * G;
        if (tl >= n_tok) continue;
        const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
        __nv_bfloat16* dst = p.out + ((size_t)(q_base + tok0 + tl) * p.n_heads + kvh * G + hg) * d;
#pragma unroll
        for (int i = 0; i < DMAX / 8; ++i) {
            const int col = i * 8 + 2 * t4;
            if (col < d)
                *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
        }
    }
}

template <int DMAX> static size_t prefill_smem() { return (size_t)(64 + 4 * BN) * (DMAX + 8) * 2; }

template <int DMAX>
static int launch_prefill(const AttnParams& p, int n_tiles, cudaStream_t stream) {
    static bool configured = false;
    size_t smem = prefill_smem<DMAX>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(attn_prefill_kernel<DMAX>, dim3(n_tiles, p.n_kv_heads), dim3(ATT_THREADS), smem, stream, p);
    return 0;
}


PB_API int pb_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                     const int32_t* block_table, int table_stride, const int32_t* positions,
                                     const int32_t* token_seq, const int32_t* cu_q, const int32_t* q_start,
                                     const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size,
                                     int num_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     float scale, int window, int swizzle, int* status, cudaStream_t stream) {
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.cu_q = cu_q; p.q_start = q_start; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0; p.n_splits = 1;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.swizzle = swizzle;
    if (int e = attn_check_common("attention_prefill", p)) return e;
    p.group = n_heads / n_kv_heads;
    PB_REQUIRE(p.group <= 64, "attention_prefill: %d query heads per key/value head; at most 64 fit a tile", p.group);
    PB_REQUIRE(n_tiles >= 0 && n_kv_heads < 65536, "attention_prefill: bad grid");
    if (n_tiles == 0 || n_tokens == 0) return 0;
    int e = head_dim <= 64 ? launch_prefill<64>(p, n_tiles, stream)
          : head_dim <= 128 ? launch_prefill<128>(p, n_tiles, stream) : launch_prefill<256>(p, n_tiles, stream);
    if (e) return e;
    PB_CHECK_LAUNCH("attention_prefill");
    return 0;
}

