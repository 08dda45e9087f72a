// Tensor-core paged attention for decode steps (one new token per request),
// bfloat16, with the key range of a request split over several blocks.
//
// For token i (the one new token of block-table row token_seq[i], at position
// p = positions[i]) and query head h (key/value head h / G):
//     o = softmax_j( (q . k_j) * scale ) v_j    over  max(0, p - window + 1) <= j <= p
// (crates/prelude-core/src/models/qwen3.rs:191-222; the reference runs decode
// through the same FlashAttention-4 / FlashInfer calls as prefill,
// crates/prelude-cuda/src/attn/flash_v4.rs:125-278, flashinfer.rs:766-793).
//
// A decode step is a stream over the cache: every key and value of every live
// request is read once, so the kernel is arranged to keep many bytes in flight.
//  * A block owns one (token, key/value head) and a contiguous share of that
//    request's 64-key tiles.  The G query heads of the group are the rows of the
//    tensor-core tile, so the group's keys and values are read once.
//  * Tiles come through a ring of three shared-memory stages, two tiles ahead of
//    the one being used.  Every thread brings one row (one token's key or value
//    of this head, head_dim * 2 bytes) per tile with one bulk asynchronous copy
//    that completes on the stage's shared-memory barrier; the page ids of the
//    block's whole share are fetched into shared memory first, so the copies do
//    not wait on the block table.  Waits on a barrier are bounded: a block that
//    gives up raises the step's status word and returns.
//  * Each of the 4 warps takes 16 keys of every tile (scores, running maximum
//    and sum in float32, probabilities rounded to bfloat16 for the second
//    product); the warps are merged through shared memory at the end.
//  * With more than one split, every block writes its unnormalised partial
//    result with its maximum and sum to scratch memory and counts itself in;
//    the block that arrives last for a (token, key/value head) adds the splits
//    up in ascending order and writes the output.  The counters are left at
//    zero for the next call.
#include "attention_common.cuh"

#define DEC_MAX_PAGES 512       // page ids of one block's share kept in shared memory (else read from the table)

struct DecodeParams {
    AttnParams a;
    int* counters;              // [n_tokens * n_kv_heads], zero on entry and on exit
    int page_shift;             // log2(page_size) when it is a power of two, else -1
};

// BNW keys per warp tile, WST stages per warp
template <int DMAX, int BNW, int WST>
__global__ void __launch_bounds__(ATT_THREADS) attn_decode_kernel(DecodeParams dp) {
    pb_grid_dep_launch();
    const AttnParams& p = dp.a;
    constexpr int STRIDE = DMAX + 8;
    constexpr int KSTEPS = DMAX / 16;
    constexpr int NT = BNW / 8;                              // 8-key score tiles per warp tile
    constexpr int STAGE_ELEMS = 2 * BNW * STRIDE;            // K rows then V rows
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sKV = sQ + 16 * STRIDE;                   // [4 warps][WST stages][K, V][BNW rows]
    int32_t* s_pages = reinterpret_cast<int32_t*>(sKV + 4 * WST * STAGE_ELEMS);
    __shared__ __align__(8) uint64_t bars[4][WST];
    __shared__ int s_last;

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
    const int ps = p.page_size;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    bool healthy = true;

    if (kt0 <= kt1) {
        if (threadIdx.x == 0) {
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int s = 0; s < WST; ++s) mbar_init(&bars[w][s], 1);
            mbar_fence_init();
        }
        // page ids of keys [key_first, key_last] of this block
        const int key_first = max(lo, kt0 * BN), key_last = min(pos, kt1 * BN + BN - 1);
        const int page_first = key_first / ps, n_pages = key_last / ps - page_first + 1;
        const bool pages_in_smem = n_pages <= DEC_MAX_PAGES;
        if (pages_in_smem)
            for (int i = threadIdx.x; i < n_pages; i += ATT_THREADS) s_pages[i] = table[page_first + i];
        // positions and block tables were written before the previous kernel started; q and the
        // newest keys and values are that kernel's output
        pb_grid_dep_wait();
        // q rows of the group (rows from G on are zero)
        const int chunks = d >> 3;
        for (int c = threadIdx.x; c < 16 * chunks; c += ATT_THREADS) {
            const int row = c / chunks, ch = c - row * chunks;
            const bool ok = row < G;
            const size_t src = ok ? (((size_t)tok * p.n_heads + kvh * G + row) * d + ch * 8) : 0;
            cp_async16(sQ + row * STRIDE + ch * 8, p.q + src, ok);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();                                    // barriers, s_pages and q are ready

        // From here on the four warps run on their own: warp w takes the BNW-key tiles w, w + 4, ...
        // of the block's share, brings them in itself (lane i copies key row i and value row i of a
        // tile with one bulk copy each) and waits on its own barriers.
        const int first_wt = kt0 * (BN / BNW), last_wt = kt1 * (BN / BNW) + (BN / BNW) - 1;
        const size_t slot_elems = (size_t)p.n_kv_heads * d;
        const unsigned row_bytes = (unsigned)d * 2;
        __nv_bfloat16* my_stages = sKV + warp * WST * STAGE_ELEMS;
        auto issue_tile = [&](int wt, int use) {
            const int stage = use % WST;
            uint64_t* bar = &bars[warp][stage];
            const int key0 = wt * BNW;
            const int n_valid = max(0, min(kv_end, key0 + BNW) - max(lo, key0));
            if (lane == 0) mbar_arrive_expect_tx(bar, (unsigned)n_valid * row_bytes * 2);
            __nv_bfloat16* dk = my_stages + stage * STAGE_ELEMS + lane * STRIDE;
            __nv_bfloat16* dv = dk + BNW * STRIDE;
            const int j = key0 + lane;
            if (lane < BNW) {
                if (j >= lo && j < kv_end) {
                    const int pi = dp.page_shift >= 0 ? (j >> dp.page_shift) : (j / ps);
                    int page = pages_in_smem ? s_pages[pi - page_first] : table[pi];
                    int slot = page * ps + (j - pi * ps);
                    if (page < 0 || page >= p.num_pages) {  // never read outside the pool; the step is reported as bad
                        slot = 0;
                        if (p.status) atomicExch(p.status, 6);
                    }
                    const size_t off = (size_t)slot * slot_elems + (size_t)kvh * d;
                    fence_proxy_async();
                    bulk_copy_g2s(dk, p.k_pages + off, row_bytes, bar);
                    bulk_copy_g2s(dv, p.v_pages + off, row_bytes, bar);
                } else {
                    // a value row that no key stands for: zeros, so that 0 * (whatever was there) cannot make a NaN
                    for (int c = 0; c < chunks; ++c) *reinterpret_cast<uint4*>(dv + c * 8) = make_uint4(0, 0, 0, 0);
                }
            }
            __syncwarp();
        };
        // tiles that hold no visible key at all (before the window, after the last key) are skipped
        int wt = first_wt + warp, use = 0, ahead_wt = wt, ahead_use = 0;
        auto tile_has_keys = [&](int t) { return t * BNW + BNW > lo && t * BNW < kv_end; };
        while (wt <= last_wt && !tile_has_keys(wt)) wt += 4;
        ahead_wt = wt;
#pragma unroll 1
        for (int i = 0; i < WST - 1 && ahead_wt <= last_wt; ++i) {
            issue_tile(ahead_wt, ahead_use++);
            do { ahead_wt += 4; } while (ahead_wt <= last_wt && !tile_has_keys(ahead_wt));
        }
#pragma unroll 1
        for (; wt <= last_wt; ++use) {
            if (ahead_wt <= last_wt) {
                issue_tile(ahead_wt, ahead_use++);
                do { ahead_wt += 4; } while (ahead_wt <= last_wt && !tile_has_keys(ahead_wt));
            }
            const bool landed = mbar_wait_bounded(&bars[warp][use % WST], (use / WST) & 1);
            if (!__all_sync(0xffffffffu, landed)) {         // gave up waiting: report, do not hang
                healthy = false;
                break;
            }
            const __nv_bfloat16* sK = my_stages + (use % WST) * STAGE_ELEMS;
            const __nv_bfloat16* sV = sK + BNW * STRIDE;
            float s[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                if (kk * 16 < d) {
                    unsigned a[4];
                    ldmatrix_x4(a[0], a[1], a[2], a[3], sQ + (lane & 15) * STRIDE + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                    for (int n2 = 0; n2 < NT / 2; ++n2) {
                        unsigned b0, b1, b2, b3;
                        const int key = n2 * 16 + (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
                        ldmatrix_x4(b0, b1, b2, b3, sK + key * STRIDE + col);
                        mma_bf16(s[2 * n2], a, b0, b1);
                        mma_bf16(s[2 * n2 + 1], a, b2, b3);
                    }
                }
            }
            const int key0 = wt * BNW;
            const bool edge = key0 < lo || key0 + BNW - 1 > pos;           // some key of the tile is not visible
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t4 + (e & 1);
                    s[nt][e] = (!edge || (j >= lo && j <= pos)) ? s[nt][e] * p.scale_log2 : -INFINITY;
                }
            }
            float corr[2], mref[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float rmax = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) rmax = fmaxf(rmax, fmaxf(s[nt][2 * h], s[nt][2 * h + 1]));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
                const float m_new = fmaxf(m[h], rmax);
                corr[h] = (m[h] == m_new) ? 1.f : ((m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new));
                mref[h] = (m_new == -INFINITY) ? 0.f : m_new;
                m[h] = m_new;
                l[h] *= corr[h];
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[nt][e] - mref[e >> 1]);
                    s[nt][e] = pv;
                    l[e >> 1] += pv;
                }
            }
            // the accumulator is rescaled only when some row's maximum moved
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < DMAX / 8; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
                }
            }
#pragma unroll
            for (int ks = 0; ks < BNW / 16; ++ks) {
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
            __syncwarp();                                   // the stage may be refilled by this warp
            do { wt += 4; } while (wt <= last_wt && !tile_has_keys(wt));
        }
        if (!healthy) {
            if (lane == 0 && p.status) atomicExch(p.status, 7);
            // copies that were issued may still be in flight: give them a bounded time to land before
            // shared memory is used for something else
            for (int u = use; u < ahead_use; ++u) mbar_wait_bounded(&bars[warp][u % WST], (u / WST) & 1);
        }
        __syncthreads();                                    // all warps are done with the tile buffers
    }
    pb_grid_dep_wait();                                     // blocks without keys come here directly
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
    if (p.n_splits == 1) return;
    // count this split in; the last one adds all splits up, in ascending order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = dp.counters + (size_t)tok * p.n_kv_heads + kvh;
        const int old = atomicAdd(counter, 1);
        s_last = (old == p.n_splits - 1);
        if (s_last) *counter = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * d; idx += ATT_THREADS) {
        const int row = idx / d, col = idx - row * d;
        const size_t th = (size_t)tok * p.n_heads + kvh * G + row;
        const float* ml = p.part_ml + th * p.n_splits * 2;
        float mm = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) mm = fmaxf(mm, __ldcg(ml + 2 * s));
        float acc = 0.f, ls = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float ms = __ldcg(ml + 2 * s);
            const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
            ls += f * __ldcg(ml + 2 * s + 1);
            acc += f * __ldcg(p.part_o + (th * p.n_splits + s) * d + col);
        }
        p.out[th * d + col] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
    }
}

// keys per warp tile and stages per warp, by head size: as much in flight as shared memory holds
template <int DMAX> struct DecodeTiling { static constexpr int BNW = 32, WST = 3; };
template <> struct DecodeTiling<256> { static constexpr int BNW = 16, WST = 3; };

template <int DMAX> static size_t decode_smem() {
    using T = DecodeTiling<DMAX>;
    size_t tiles = (size_t)(16 + 4 * T::WST * 2 * T::BNW) * (DMAX + 8) * 2 + DEC_MAX_PAGES * 4;
    size_t merge = (size_t)16 * (DMAX + 8) * 2 + (size_t)(4 * 16 * DMAX + 128) * 4;
    return tiles > merge ? tiles : merge;
}

template <int DMAX>
static int launch_decode(const DecodeParams& dp, cudaStream_t stream) {
    static bool configured = false;
    size_t smem = decode_smem<DMAX>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DMAX, DecodeTiling<DMAX>::BNW, DecodeTiling<DMAX>::WST>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_decode: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(attn_decode_kernel<DMAX, DecodeTiling<DMAX>::BNW, DecodeTiling<DMAX>::WST>, dim3(dp.a.n_splits, dp.a.n_kv_heads, dp.a.n_tokens), dim3(ATT_THREADS), smem, stream, dp);
    return 0;
}

// Blocks of this kernel that one multiprocessor holds at a time (for choosing the number of splits).
PB_API int pb_attention_decode_blocks_per_sm(int head_dim) {
    size_t smem = head_dim <= 64 ? decode_smem<64>() : head_dim <= 128 ? decode_smem<128>() : decode_smem<256>();
    int n = (int)((227 * 1024) / (smem + 1024));
    return n < 1 ? 1 : n;
}

// Scratch floats a call needs for its splits: (head_dim + 2) per token, head and split.
PB_API long long pb_attention_decode_scratch_floats(int n_tokens, int n_heads, int head_dim, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (head_dim + 2);
}

// scratch: pb_attention_decode_scratch_floats(...) floats, or null when n_splits == 1.
// counters: n_tokens * n_kv_heads ints, zero before the first call; every call leaves them
// zero, so calls that follow one another on a stream may share them.  Null when n_splits == 1.
PB_API int pb_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                    const int32_t* block_table, int table_stride, const int32_t* positions,
                                    const int32_t* token_seq, int page_size, int num_pages, int n_tokens,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_splits,
                                    float* scratch, int* counters, int* status, cudaStream_t stream) {
    DecodeParams dp{};
    AttnParams& p = dp.a;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.n_splits = n_splits; p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages;
    p.n_tokens = n_tokens; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    if (int e = attn_check_common("attention_decode", p)) return e;
    p.group = n_heads / n_kv_heads;
    PB_REQUIRE(p.group <= 16, "attention_decode: %d query heads per key/value head; at most 16 fit a tile", p.group);
    PB_REQUIRE(n_splits >= 1 && n_splits <= 1024, "attention_decode: n_splits=%d", n_splits);
    PB_REQUIRE(n_tokens < 65536 && n_kv_heads < 65536, "attention_decode: bad grid");
    PB_REQUIRE(n_splits == 1 || (scratch != nullptr && counters != nullptr),
               "attention_decode: %d splits need scratch memory and counters", n_splits);
    if (n_tokens == 0) return 0;
    if (n_splits > 1) {
        p.part_o = scratch;
        p.part_ml = scratch + (size_t)n_tokens * n_heads * n_splits * head_dim;
    }
    dp.counters = counters;
    dp.page_shift = -1;
    for (int s = 0; s < 31; ++s)
        if ((1 << s) == page_size) dp.page_shift = s;
    int e = head_dim <= 64 ? launch_decode<64>(dp, stream)
          : head_dim <= 128 ? launch_decode<128>(dp, stream) : launch_decode<256>(dp, stream);
    if (e) return e;
    PB_CHECK_LAUNCH("attention_decode");
    return 0;
}
