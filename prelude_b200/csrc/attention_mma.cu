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
#include "common.cuh"

#include <math.h>

#define BN 64                 // keys per tile
#define ATT_THREADS 128

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int n = pred ? 16 : 0;     // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q;        // [T, nH, D]
    const __nv_bfloat16* k_pages;  // [pages, page_size, nKV, D]
    const __nv_bfloat16* v_pages;
    __nv_bfloat16* out;            // [T, nH, D]
    const int32_t* block_table;    // [rows, table_stride]
    const int32_t* positions;      // [T]
    const int32_t* token_seq;      // [T] row of block_table for each token
    // prefill plan
    const int32_t* cu_q;           // [R + 1]
    const int32_t* q_start;        // [R]
    const int32_t* tile_seq;       // [n_tiles] request of each tile
    const int32_t* tile_tok0;      // [n_tiles] first token of the tile within the request's portion
    // decode splits
    float* part_o;                 // [T, nH, n_splits, D]
    float* part_ml;                // [T, nH, n_splits, 2]
    int n_splits;
    int table_stride, page_size, num_pages;
    int n_tokens, n_heads, n_kv_heads, head_dim, group, window;
    float scale_log2;              // scale * log2(e)
    int* status;
};

// One tile of BN keys and values of one key/value head into shared memory;
// rows outside [kv_begin, kv_end) (and rows whose page id is bad) are zero-filled.
// Pages below kv_begin may have been given back already and are never looked up.
template <int DMAX>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV, const AttnParams& p,
                                             const int32_t* table, int kvh, int key0, int kv_begin, int kv_end) {
    constexpr int STRIDE = DMAX + 8;
    const int chunks = p.head_dim >> 3;                    // 16-byte chunks in a row
    const int total = BN * chunks;
    for (int c = threadIdx.x; c < total; c += ATT_THREADS) {
        const int row = c / chunks, ch = c - row * chunks;
        const int j = key0 + row;
        bool ok = j >= kv_begin && j < kv_end;
        size_t src = 0;
        if (ok) {
            const int page = table[j / p.page_size];
            if (page < 0 || page >= p.num_pages) {
                ok = false;
                if (p.status) atomicExch(p.status, 6);
            } else {
                src = (((size_t)page * p.page_size + j % p.page_size) * p.n_kv_heads + kvh) * p.head_dim + ch * 8;
            }
        }
        cp_async16(sK + row * STRIDE + ch * 8, p.k_pages + src, ok);
        cp_async16(sV + row * STRIDE + ch * 8, p.v_pages + src, ok);
    }
}

// ---------------------------------------------------------------------------------------
// prefill: 64 rows (tokens x heads of a group) against all visible keys
// ---------------------------------------------------------------------------------------
template <int DMAX>
__global__ void __launch_bounds__(ATT_THREADS) attn_prefill_kernel(AttnParams p) {
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

// ---------------------------------------------------------------------------------------
// decode: the G rows of one token, a share of the key tiles, 16 keys of each tile per warp
// ---------------------------------------------------------------------------------------
template <int DMAX>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(AttnParams p) {
    constexpr int STRIDE = DMAX + 8;
    constexpr int KSTEPS = DMAX / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sKV = sQ + 16 * STRIDE;

    const int G = p.group, d = p.head_dim;
    const int split = blockIdx.x, kvh = blockIdx.y, tok = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int pos = p.positions[tok];
    const int32_t* table = p.block_table + (size_t)p.token_seq[tok] * p.table_stride;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int kt_lo = lo / BN, kt_hi = pos / BN;
    const int per_split = (kt_hi - kt_lo + 1 + p.n_splits - 1) / p.n_splits;
    const int kt0 = kt_lo + split * per_split, kt1 = min(kt_hi, kt0 + per_split - 1);
    const int kv_end = pos + 1;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    if (kt0 <= kt1) {
        const int chunks = d >> 3;
        for (int c = threadIdx.x; c < 16 * chunks; c += ATT_THREADS) {
            const int row = c / chunks, ch = c - row * chunks;
            const bool ok = row < G;
            const size_t src = ok ? (((size_t)tok * p.n_heads + kvh * G + row) * d + ch * 8) : 0;
            cp_async16(sQ + row * STRIDE + ch * 8, p.q + src, ok);
        }
        load_kv_tile<DMAX>(sKV, sKV + BN * STRIDE, p, table, kvh, kt0 * BN, lo, kv_end);
        cp_async_commit();
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
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                if (kk * 16 < d) {
                    unsigned a[4], b0, b1, b2, b3;
                    ldmatrix_x4(a[0], a[1], a[2], a[3], sQ + (lane & 15) * STRIDE + kk * 16 + (lane >> 4) * 8);
                    const int key = warp * 16 + (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(b0, b1, b2, b3, sK + key * STRIDE + col);
                    mma_bf16(s[0], a, b0, b1);
                    mma_bf16(s[1], a, b2, b3);
                }
            }
            float rmax = -INFINITY;                         // every row of the tile has the same visible keys
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = kt * BN + warp * 16 + nt * 8 + 2 * t4 + (e & 1);
                    const float v = (j >= lo && j <= pos) ? s[nt][e] * p.scale_log2 : -INFINITY;
                    s[nt][e] = v;
                }
            }
            float corr[2], mref[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                rmax = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
                const float m_new = fmaxf(m[h], rmax);
                corr[h] = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
                mref[h] = (m_new == -INFINITY) ? 0.f : m_new;
                m[h] = m_new;
                l[h] *= corr[h];
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
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
            unsigned a[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                             pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
            for (int d2 = 0; d2 < KSTEPS; ++d2) {
                if (d2 * 16 < d) {
                    unsigned b0, b1, b2, b3;
                    const int key = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = d2 * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(b0, b1, b2, b3, sV + key * STRIDE + col);
                    mma_bf16(o[2 * d2], a, b0, b1);
                    mma_bf16(o[2 * d2 + 1], a, b2, b3);
                }
            }
            __syncthreads();
        }
    }
    // merge the four warps through shared memory (the tile buffers are free now)
    float* sO = reinterpret_cast<float*>(sKV);              // [4][16][DMAX]
    float* sM = sO + 4 * 16 * DMAX;                         // [4][16]
    float* sL = sM + 64;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        const int row = g + 8 * h;
        if (t4 == 0) { sM[warp * 16 + row] = m[h]; sL[warp * 16 + row] = l[h]; }
#pragma unroll
        for (int i = 0; i < DMAX / 8; ++i) {
            const int col = i * 8 + 2 * t4;
            sO[(warp * 16 + row) * DMAX + col] = o[i][2 * h];
            sO[(warp * 16 + row) * DMAX + col + 1] = o[i][2 * h + 1];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * d; idx += ATT_THREADS) {
        const int row = idx / d, col = idx - row * d;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sM[w * 16 + row]);
        float acc = 0.f, ls = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sM[w * 16 + row];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mm);
            acc += f * sO[(w * 16 + row) * DMAX + col];
            ls += f * sL[w * 16 + row];
        }
        const size_t th = (size_t)tok * p.n_heads + kvh * G + row;
        if (p.n_splits == 1) {
            p.out[th * d + col] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
        } else {
            p.part_o[(th * p.n_splits + split) * d + col] = acc;
            if (col == 0) {
                p.part_ml[(th * p.n_splits + split) * 2] = mm;
                p.part_ml[(th * p.n_splits + split) * 2 + 1] = ls;
            }
        }
    }
}

// Sum of the splits of one (token, head), in ascending split order.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  __nv_bfloat16* __restrict__ out, int n_splits, int head_dim) {
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * n_splits * 2;
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, ml[2 * s]);
    float ls = 0.f;
    for (int s = 0; s < n_splits; ++s) ls += (ml[2 * s] == -INFINITY) ? 0.f : exp2f(ml[2 * s] - mm) * ml[2 * s + 1];
    const float inv = ls > 0.f ? 1.0f / ls : 0.f;
    for (int col = threadIdx.x; col < head_dim; col += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float f = (ml[2 * s] == -INFINITY) ? 0.f : exp2f(ml[2 * s] - mm);
            acc += f * part_o[(th * n_splits + s) * head_dim + col];
        }
        out[th * head_dim + col] = __float2bfloat16_rn(acc * inv);
    }
}

template <int DMAX> static size_t prefill_smem() { return (size_t)(64 + 4 * BN) * (DMAX + 8) * 2; }
template <int DMAX> static size_t decode_smem() {
    size_t tiles = (size_t)(16 + 4 * BN) * (DMAX + 8) * 2;
    size_t merge = (size_t)16 * (DMAX + 8) * 2 + (size_t)(4 * 16 * DMAX + 128) * 4;
    return tiles > merge ? tiles : merge;
}

template <int DMAX>
static int launch_prefill(const AttnParams& p, int n_tiles, cudaStream_t stream) {
    static bool configured = false;
    size_t smem = prefill_smem<DMAX>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_prefill_kernel<DMAX><<<dim3(n_tiles, p.n_kv_heads), ATT_THREADS, smem, stream>>>(p);
    return 0;
}

template <int DMAX>
static int launch_decode(const AttnParams& p, cudaStream_t stream) {
    static bool configured = false;
    size_t smem = decode_smem<DMAX>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_decode: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_decode_kernel<DMAX><<<dim3(p.n_splits, p.n_kv_heads, p.n_tokens), ATT_THREADS, smem, stream>>>(p);
    return 0;
}

static int check_common(const char* name, const AttnParams& p) {
    PB_REQUIRE(p.n_heads > 0 && p.n_kv_heads > 0 && p.n_heads % p.n_kv_heads == 0,
               "%s: %d query heads over %d key/value heads", name, p.n_heads, p.n_kv_heads);
    PB_REQUIRE(p.head_dim >= 16 && p.head_dim <= 256 && p.head_dim % 16 == 0,
               "%s: head_dim=%d; the tensor-core kernels take multiples of 16 up to 256", name, p.head_dim);
    PB_REQUIRE(p.page_size > 0 && p.num_pages > 0 && p.table_stride > 0, "%s: bad cache geometry", name);
    PB_REQUIRE(pb_aligned(p.q, 16) && pb_aligned(p.k_pages, 16) && pb_aligned(p.v_pages, 16) && pb_aligned(p.out, 4),
               "%s: q and the pages must be 16-byte aligned", name);
    return 0;
}

// Prompt portions (and any mix of portions and single tokens).  Tiles are listed by the host:
// tile i covers tokens [tile_tok0[i], tile_tok0[i] + 64 / group) of request tile_seq[i].
PB_API int pb_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                     const int32_t* block_table, int table_stride, const int32_t* positions,
                                     const int32_t* token_seq, const int32_t* cu_q, const int32_t* q_start,
                                     const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size,
                                     int num_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     float scale, int window, int* status, cudaStream_t stream) {
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.cu_q = cu_q; p.q_start = q_start; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0; p.n_splits = 1;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    if (int e = check_common("attention_prefill", p)) return e;
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

// Scratch floats a decode call needs for its splits: (head_dim + 2) per token, head and split.
PB_API long long pb_attention_decode_scratch_floats(int n_tokens, int n_heads, int head_dim, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (head_dim + 2);
}

// Decode step: token i is the one new token of block-table row token_seq[i], at positions[i].
// scratch: pb_attention_decode_scratch_floats(...) floats, or null when n_splits == 1.
PB_API int pb_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                    const int32_t* block_table, int table_stride, const int32_t* positions,
                                    const int32_t* token_seq, int page_size, int num_pages, int n_tokens,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                    float* scratch, int* status, cudaStream_t stream) {
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.n_splits = n_splits; p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages;
    p.n_tokens = n_tokens; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    if (int e = check_common("attention_decode", p)) return e;
    p.group = n_heads / n_kv_heads;
    PB_REQUIRE(p.group <= 16, "attention_decode: %d query heads per key/value head; at most 16 fit a tile", p.group);
    PB_REQUIRE(n_splits >= 1 && n_splits <= 1024, "attention_decode: n_splits=%d", n_splits);
    PB_REQUIRE(n_tokens < 65536 && n_kv_heads < 65536, "attention_decode: bad grid");
    PB_REQUIRE(n_splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", n_splits);
    if (n_tokens == 0) return 0;
    if (n_splits > 1) {
        p.part_o = scratch;
        p.part_ml = scratch + (size_t)n_tokens * n_heads * n_splits * head_dim;
    }
    int e = head_dim <= 64 ? launch_decode<64>(p, stream)
          : head_dim <= 128 ? launch_decode<128>(p, stream) : launch_decode<256>(p, stream);
    if (e) return e;
    PB_CHECK_LAUNCH("attention_decode");
    if (n_splits > 1) {
        attn_merge_kernel<<<n_tokens * n_heads, head_dim <= 64 ? 32 : 64, 0, stream>>>(p.part_o, p.part_ml, p.out, n_splits, head_dim);
        PB_CHECK_LAUNCH("attention_merge");
    }
    return 0;
}
