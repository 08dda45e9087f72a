// Paged attention for prompt portions on the fifth-generation tensor cores (tcgen05), bfloat16.
//
// The same function as attention_prefill.cu computes (for a query at absolute position p of request r and
// query head h, o = softmax_j((q . k_j) * scale) v_j over max(0, p - window + 1) <= j <= p, keys and values
// read from the request's pages; crates/prelude-core/src/models/qwen3.rs:191-222, which the reference hands
// to FlashAttention-4, crates/prelude-cuda/src/attn/flash_v4.rs:125-278), with both products issued as
// tcgen05.mma and their accumulators in tensor memory.
//
// Work of a block: 256 query rows = 256/G tokens of one request x the G query heads that share one
// key/value head (G a power of two), as two row tiles of 128; row R is head R / (256/G), token R % (256/G),
// so every head's tokens are one box of the query tensor for TMA.  The block walks the visible keys in
// tiles of 128; both row tiles use every key and value tile, which is fetched once.
//
// Shared memory: the query rows and a ring of key and value tiles, each tile as 64-column slabs of 128 rows
// x 128 bytes with 128-byte swizzle - what the tensor cores read directly.  The cache stores the 16-byte
// chunks of every token row already permuted that way (pb_kv_elem_offset), so a tensor map WITHOUT swizzle
// over [page][kv head][token][half][64] brings one page's run of one head into a slab as it is; keys are the
// K-major B operand of the first product, values the MN-major B operand of the second.  The query tensor is
// dense and its map swizzles.
//
// Tensor memory (512 columns): S_0, S_1 (128 float32 columns each: scores of the two row tiles), O_0, O_1
// (head_dim columns each).  The probabilities, rounded to bfloat16, overwrite the first 64 columns of their
// scores and are the A operand of the second product straight from tensor memory.
//
// Warps: 0-3 and 4-7 are the softmax groups of row tile 0 and 1 (thread = row = tensor-memory lane: the
// maximum and the sum of a row need no exchange), warp 8 issues the TMA loads, warp 9 owns the tensor-memory
// allocation and issues the products.  The products of one row tile run while the other group is in its
// softmax:  S_0(0) S_1(0) | PV_0(j) S_0(j+1) PV_1(j) S_1(j+1) | ...
// The running maximum is kept in scaled log2 units and the accumulator is rescaled (by the row's own
// thread, in tensor memory) only when a maximum grew by more than 2^8; the sum and the accumulator stay
// relative to that slightly stale maximum and the final division cancels it.  Softmax, maximum, sum and
// rescaling are float32.  Every wait on a barrier is bounded in time; a block that gives up raises the status
// word, and all its warps still meet at the end, where the tensor memory is freed.  No load uses cluster
// multicast.
#include "attention_common.cuh"
#include "tcgen05.cuh"

#define PT_KEYS 128                 // keys per tile
#define PT_THREADS 320
#define PT_SLAB (128 * 128)         // bytes of a slab: 128 rows x 64 bfloat16
#define PT_S_COLS 128

template <int D> struct PtTiling {
    static constexpr int HALVES = D / 64;
    static constexpr int TILE_BYTES = HALVES * PT_SLAB;          // 128 rows x D
    static constexpr int Q_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = D == 64 ? 4 : 2;
    static constexpr int SMEM_BYTES = Q_BYTES + STAGES * 2 * TILE_BYTES + 1024;
    static constexpr int O_COL = 2 * PT_S_COLS;                  // O_m starts at O_COL + m * D
    static constexpr int TMEM_COLS = 512;
};

struct PtParams {
    AttnParams a;
    int tok;                        // tokens of a block: 256 / group
    int q_rows;                     // rows of a query box: min(tok, 128)
    int kv_rows;                    // rows of a key/value box: min(page_size, 128)
};

template <int D>
__global__ void __launch_bounds__(PT_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, PtParams pp) {
    pb_grid_dep_launch();
    using T = PtTiling<D>;
    constexpr int S = T::STAGES;
    const AttnParams& p = pp.a;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;
    unsigned char* sKV = smem + T::Q_BYTES;                      // stage s: keys at s * 2 * TILE_BYTES, values TILE_BYTES later
    __shared__ __align__(8) uint64_t q_full, k_full[S], v_full[S], k_empty[S], v_empty[S], s_full[2], p_full[2], o_full[2];
    __shared__ uint32_t tmem_holder;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.group, TOK = pp.tok, ps = p.page_size;
    const int tile = blockIdx.x / p.n_kv_heads, kvh = blockIdx.x - tile * p.n_kv_heads;
    const int r = p.tile_seq[tile], tok0 = p.tile_tok0[tile];
    const int q_base = p.cu_q[r], q_len = p.cu_q[r + 1] - q_base, pos0 = p.q_start[r];
    const int n_tok = min(TOK, q_len - tok0);                    // tokens of this block
    const int p_min = pos0 + tok0, p_max = p_min + n_tok - 1;
    const int lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt0 = lo / PT_KEYS;
    const int lo_run = lo / pp.kv_rows * pp.kv_rows;             // first key of the first run that holds a visible key
    // key tiles of each row tile: row tile m holds tokens (m * 128) % TOK .. ; with one head per block
    // (TOK = 256) the second row tile holds the later 128 tokens and may be empty
    int n_m[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const int tl_first = (m * 128) % TOK, tl_last = min(tl_first + min(TOK, 128), n_tok) - 1;
        n_m[m] = tl_first < n_tok ? (pos0 + tok0 + tl_last) / PT_KEYS - kt0 + 1 : 0;
    }
    const int n_tiles = max(n_m[0], n_m[1]);

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < S; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1); }
        for (int m = 0; m < 2; ++m) { mbar_init(&s_full[m], 1); mbar_init(&p_full[m], 128); mbar_init(&o_full[m], 1); }
        mbar_fence_init();
    }
    if (warp == 9) tc_tmem_alloc(&tmem_holder, T::TMEM_COLS);
    if (warp == 8 && lane == 0) { tc_prefetch_map(&map_q); tc_prefetch_map(&map_k); tc_prefetch_map(&map_v); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 8) {
        // ---------------- loads ----------------
        // The whole warp walks the loop.  It keeps 32 consecutive entries
        // of the request's block table in registers, one per lane, and the 32 after them: a page number is then a
        // shuffle away, not a trip to memory per copy.
        const int32_t* table = p.block_table + (size_t)p.token_seq[q_base + tok0] * p.table_stride;
        const int runs = PT_KEYS / pp.kv_rows;
        const int last_pi = p_max / ps;                          // the last page the block reads; the request holds it for sure
        const int hi_run = p_max / pp.kv_rows * pp.kv_rows;      // first key of the last run that holds a visible key
        int win_pi = (kt0 * PT_KEYS) / ps;                       // table index that lane 0 of `cur` holds
        int cur = table[min(win_pi + lane, last_pi)], nxt = table[min(win_pi + 32 + lane, last_pi)];
        // The page and the row in it where the u-th run of key tile j starts.  Runs without a visible key (before the
        // window, after the last key) are read from the nearest run that has one: their probabilities are zero, and
        // the value rows are cleared by the softmax threads.
        auto locate = [&](int j, int u, int& page, int& row) {
            int j0 = (kt0 + j) * PT_KEYS + u * pp.kv_rows;
            j0 = min(max(j0, lo_run), hi_run);
            const int pi = j0 / ps;
            row = j0 - pi * ps;
            const int idx = pi - win_pi;                         // 0 .. 47: the tile starts inside `cur` and spans at most 16 pages
            const int a = __shfl_sync(0xffffffffu, cur, idx & 31), b = __shfl_sync(0xffffffffu, nxt, idx & 31);
            page = idx < 32 ? a : b;
            if (page < 0 || page >= p.num_pages) {               // never read outside the pool; the step is reported as bad
                page = 0;
                if (p.status) atomicExch(p.status, 6);
            }
        };
        // q and the newest keys and values are the output of the kernel before this one
        pb_grid_dep_wait();
        if (tc_elect_one()) {
            mbar_arrive_expect_tx(&q_full, T::Q_BYTES);
            for (int i = 0; i < 256 / pp.q_rows; ++i) {
                const int R0 = i * pp.q_rows, hg = R0 / TOK, tl0 = R0 - hg * TOK;
                unsigned char* dst = sQ + (R0 >> 7) * T::TILE_BYTES + (R0 & 127) * 128;
#pragma unroll
                for (int h = 0; h < T::HALVES; ++h)
                    tc_tma_load_3d(dst + h * PT_SLAB, &map_q, h * 64, kvh * G + hg, q_base + tok0 + tl0, &q_full);
            }
        }
        __syncwarp();
        bool ok = true;
        int stage = 0, phase = 0;
#pragma unroll 1
        for (int j = 0; j < n_tiles; ++j) {
            unsigned char* sK = sKV + stage * 2 * T::TILE_BYTES;
            unsigned char* sV = sK + T::TILE_BYTES;
            while (((kt0 + j) * PT_KEYS) / ps - win_pi >= 32) {  // slide the window of table entries
                cur = nxt;
                win_pi += 32;
                nxt = table[min(win_pi + 32 + lane, last_pi)];
            }
            // lane u brings the u-th run of the tile, its keys and then its values: the copies of a tile are issued
            // side by side, not one after the other
            int page, row;
            locate(j, lane < runs ? lane : 0, page, row);
#pragma unroll 1
            for (int kv = 0; kv < 2 && ok; ++kv) {
                uint64_t* full = kv ? &v_full[stage] : &k_full[stage];
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(kv ? &v_empty[stage] : &k_empty[stage], phase ^ 1));
                if (!ok) break;
                if (lane == 0) mbar_arrive_expect_tx(full, T::TILE_BYTES);
                __syncwarp();
                if (lane < runs) {
#pragma unroll
                    for (int h = 0; h < T::HALVES; ++h)
                        tc_tma_load_5d((kv ? sV : sK) + h * PT_SLAB + lane * pp.kv_rows * 128, kv ? &map_v : &map_k, 0, h, row, kvh, page, full);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 7);
    } else if (warp == 9) {
        // ---------------- products: reads shared and tensor memory only ----------------
        // The whole warp walks the loop and waits; one elected lane issues.  (Issued from a branch on the lane
        // number instead, every tcgen05.mma cost the thread about 100 cycles, more than the product itself takes;
        // under elect.sync the descriptors stay in uniform registers and a 128 x 128 x 16 product issues every 64.)
        const uint32_t idesc_s = tc_instr_desc(PT_KEYS), idesc_o = tc_instr_desc(D, true);
        bool ok = true;
        auto wait_all = [&](uint64_t* bar, unsigned parity) {
            ok = __all_sync(0xffffffffu, ok && mbar_wait_bounded(bar, parity));
            return ok;
        };
        // S_m = Q_m K^T for the key tile in `stage`; release_k: the key stage is free once these have finished
        auto issue_s = [&](int m, int stage, bool release_k) {
            tc_fence_after();
            if (tc_elect_one()) {
                const uint64_t dq = tc_smem_desc(sQ + m * T::TILE_BYTES), dk = tc_smem_desc(sKV + stage * 2 * T::TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const unsigned off = ((ks >> 2) * PT_SLAB + (ks & 3) * 32) >> 4;
                    tc_mma(tmem_base + m * PT_S_COLS, dq + off, dk + off, idesc_s, ks > 0 ? 1u : 0u);
                }
                tc_commit(&s_full[m]);
                if (release_k) tc_commit(&k_empty[stage]);
            }
            __syncwarp();
        };
        // O_m (+)= P_m V for the value tile in `stage`
        auto issue_o = [&](int m, int stage, bool first, bool last, bool release_v) {
            tc_fence_after();
            if (tc_elect_one()) {
                const uint64_t dv = tc_smem_desc_mn(sKV + stage * 2 * T::TILE_BYTES + T::TILE_BYTES, PT_SLAB);
#pragma unroll
                for (int ks = 0; ks < PT_KEYS / 16; ++ks)
                    tc_mma_ts(tmem_base + T::O_COL + m * D, tmem_base + m * PT_S_COLS + ks * 8, dv + ((ks * 16 * 128) >> 4), idesc_o,
                              (!first || ks > 0) ? 1u : 0u);
                if (last) tc_commit(&o_full[m]);
                if (release_v) tc_commit(&v_empty[stage]);
            }
            __syncwarp();
        };
        const auto first_active = [&](int j) { return j < n_m[0] ? 0 : 1; };
        const auto last_active = [&](int j) { return j < n_m[1] ? 1 : 0; };
        if (wait_all(&q_full, 0) && wait_all(&k_full[0], 0)) {
            for (int m = 0; m < 2; ++m)
                if (n_m[m] > 0) issue_s(m, 0, m == last_active(0));
        }
        int stage = 0, phase = 0;
#pragma unroll 1
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int nstage = stage + 1 == S ? 0 : stage + 1, nphase = stage + 1 == S ? phase ^ 1 : phase;
            for (int m = 0; m < 2 && ok; ++m) {
                if (j >= n_m[m]) continue;
                if (!wait_all(&p_full[m], j & 1)) break;
                if (m == first_active(j) && !wait_all(&v_full[stage], phase)) break;
                issue_o(m, stage, j == 0, j == n_m[m] - 1, m == last_active(j));
                if (j + 1 < n_m[m]) {
                    if (m == first_active(j + 1) && !wait_all(&k_full[nstage], nphase)) break;
                    issue_s(m, nstage, m == last_active(j + 1));
                }
            }
            stage = nstage; phase = nphase;
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 9);
    } else {
        // ---------------- softmax: thread = row ----------------
        const int m = warp >> 2;                                  // row tile
        const int R = m * 128 + (warp & 3) * 32 + lane;           // row of the block
        const int hg = R / TOK, tl = R - hg * TOK;
        const bool valid = tl < n_tok;
        const int row_pos = pos0 + tok0 + min(tl, n_tok - 1);      // rows without a token behave like the last token
        const int row_lo = p.window > 0 ? row_pos - p.window + 1 : 0;
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + m * PT_S_COLS, o_addr = lane_base + T::O_COL + m * D;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < n_m[m]; ++j) {
            ok = mbar_wait_bounded(&s_full[m], j & 1);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[PT_KEYS];
#pragma unroll
            for (int c = 0; c < PT_KEYS; c += 32) tc_tmem_ld32(s_addr + c, sr + c);
            tc_tmem_ld_wait();
            const int key0 = (kt0 + j) * PT_KEYS;
            if (key0 + PT_KEYS - 1 > row_pos || key0 < row_lo) {
#pragma unroll
                for (int c = 0; c < PT_KEYS; ++c) {
                    const int kj = key0 + c;
                    if (kj > row_pos || kj < row_lo) sr[c] = __float_as_uint(-INFINITY);
                }
            }
            // eight chains side by side: one chain of 128 dependent operations would take their latency 128 times
            float mx[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx[i] = __uint_as_float(sr[i]);
#pragma unroll
            for (int c = 8; c < PT_KEYS; ++c) mx[c & 7] = fmaxf(mx[c & 7], __uint_as_float(sr[c]));
            const float rmax = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
            const float cand = fmaxf(m_ref, rmax * p.scale_log2);  // scale > 0: the maximum commutes with it
            const bool grow = cand > m_ref + ATT_RESCALE_STEP;      // also true for -inf -> finite
            if (__any_sync(0xffffffffu, grow)) {
                const float corr = (m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - cand);
                m_ref = cand;
                l *= corr;
                if (j > 0) {                                       // the accumulator holds something: no product is writing it now
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t orr[32];
                        tc_tmem_ld32(o_addr + c, orr);
                        tc_tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * corr);
                        tc_tmem_st32(o_addr + c, orr);
                    }
                }
            }
            // exp2(s * scale - m); a row that has seen nothing yet has m = -inf and only -inf scores: exp2(-inf - 0) = 0
            const float mref = m_ref == -INFINITY ? 0.f : m_ref;
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < PT_KEYS; c += 32) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(sr[c + 2 * i]), p.scale_log2, -mref));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(sr[c + 2 * i + 1]), p.scale_log2, -mref));
                    ls[i & 3] += p0 + p1;
                    pk[i] = pack_bf16(p0, p1);
                }
                tc_tmem_st16(s_addr + (c >> 1), pk);
            }
            l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
            // Value rows of keys that nobody may see (before the first visible run, after the last key) hold whatever
            // their page holds, and 0 x NaN is NaN: this group clears them once the tile has landed and before it
            // lets its product start.  Only the first and the last tile of the block have such rows.
            const int clear_below = j == 0 ? lo_run - key0 : 0, clear_from = j == n_tiles - 1 ? p_max + 1 - key0 : PT_KEYS;
            if (clear_below > 0 || clear_from < PT_KEYS) {
                const int stage = j % S;
                ok = mbar_wait_bounded(&v_full[stage], (j / S) & 1);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                unsigned char* sV = sKV + stage * 2 * T::TILE_BYTES + T::TILE_BYTES;
                const int t = (warp & 3) * 32 + lane;
                for (int idx = t; idx < PT_KEYS * T::HALVES * 8; idx += 128) {
                    const int row = idx / (T::HALVES * 8), rest = idx - row * (T::HALVES * 8);
                    if (row < clear_below || row >= clear_from)
                        *reinterpret_cast<uint4*>(sV + (rest >> 3) * PT_SLAB + row * 128 + (rest & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async();
            }
            tc_tmem_st_wait();
            tc_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&p_full[m])) : "memory");
        }
        if (n_m[m] > 0) {
            if (ok) ok = mbar_wait_bounded(&o_full[m], 0);
            if (__all_sync(0xffffffffu, ok)) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                __nv_bfloat16* dst = p.out + ((size_t)(q_base + tok0 + (valid ? tl : 0)) * p.n_heads + kvh * G + hg) * D;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t orr[32];
                    tc_tmem_ld32(o_addr + c, orr);
                    tc_tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 w;
                            w.x = pack_bf16(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv);
                            w.y = pack_bf16(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
                            w.z = pack_bf16(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv);
                            w.w = pack_bf16(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c + i) = w;
                        }
                    }
                }
            } else if (lane == 0 && p.status) {
                atomicExch(p.status, 10);
            }
        }
    }
    // everybody is done with tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        tc_fence_after();
        tc_tmem_dealloc(tmem_base, T::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static int pt_encode(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                     const cuuint32_t* box, CUtensorMapSwizzle swizzle, const char* what) {
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pb_fail("attention_prefill_tc: cuTensorMapEncodeTiled failed with code %d for %s", (int)r, what);
    return 0;
}

template <int D>
static int pt_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PtParams& pp, int n_tiles,
                     cudaStream_t stream) {
    using T = PtTiling<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess)
            return pb_fail("attention_prefill_tc: cannot get %d bytes of shared memory: %s", T::SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(attn_prefill_tc_kernel<D>, dim3((unsigned)n_tiles * pp.a.n_kv_heads), dim3(PT_THREADS), (size_t)T::SMEM_BYTES, stream,
              mq, mk, mv, pp);
    return 0;
}

static bool pt_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Whether the kernel takes the shape: permuted bfloat16 pages, head_dim 64 or 128, a power of two of at most
// 32 query heads per key/value head, and pages whose runs tile a 128-key tile evenly.
PB_API int pb_attention_prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim, int page_size, int swizzle) {
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int g = n_heads / n_kv_heads;
    if (!pt_pow2(g) || g > 32) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (!swizzle || page_size % 8 || !(PT_KEYS % page_size == 0 || page_size % PT_KEYS == 0)) return 0;
    return 1;
}

// Tokens of one tile of the host's list for this kernel.
PB_API int pb_attention_prefill_tc_tile_tokens(int n_heads, int n_kv_heads) { return 256 / (n_heads / n_kv_heads); }

// Tiles are listed by the host: tile t covers tokens tile_tok0[t] .. of request tile_seq[t]'s portion,
// 256 / (n_heads / n_kv_heads) tokens each.  q and out are dense [n_tokens, n_heads, head_dim].
PB_API int pb_attention_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                        const int32_t* block_table, int table_stride, const int32_t* positions,
                                        const int32_t* token_seq, const int32_t* cu_q, const int32_t* q_start,
                                        const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size,
                                        int num_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                        float scale, int window, int swizzle, int* status, cudaStream_t stream) {
    PtParams pp{};
    AttnParams& p = pp.a;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.cu_q = cu_q; p.q_start = q_start; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0; p.n_splits = 1;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.swizzle = swizzle;
    if (int e = attn_check_common("attention_prefill_tc", p)) return e;
    PB_REQUIRE(pb_attention_prefill_tc_supported(n_heads, n_kv_heads, head_dim, page_size, swizzle),
               "attention_prefill_tc: n_heads=%d n_kv_heads=%d head_dim=%d page_size=%d swizzle=%d not taken (permuted pages, "
               "head_dim 64 or 128, a power of two of query heads per key/value head, page_size dividing or divided by 128)",
               n_heads, n_kv_heads, head_dim, page_size, swizzle);
    PB_REQUIRE(scale > 0.f, "attention_prefill_tc: scale=%g; the kernel takes the row maximum before scaling", (double)scale);
    PB_REQUIRE(pb_aligned(out, 16), "attention_prefill_tc: out must be 16-byte aligned");
    PB_REQUIRE(n_tiles >= 0 && (long long)n_tiles * n_kv_heads < (1ll << 31), "attention_prefill_tc: bad grid");
    if (n_tiles == 0 || n_tokens == 0) return 0;
    p.group = n_heads / n_kv_heads;
    pp.tok = 256 / p.group;
    pp.q_rows = pp.tok < 128 ? pp.tok : 128;
    pp.kv_rows = page_size < PT_KEYS ? page_size : PT_KEYS;
    if (int e = get_encode()) return e;
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)n_heads, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)n_heads * head_dim * 2};
        cuuint32_t box[3] = {64, 1, (cuuint32_t)pp.q_rows};
        if (int e = pt_encode(&mq, q, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "q")) return e;
    }
    {
        const cuuint64_t row = (cuuint64_t)head_dim * 2;
        cuuint64_t dims[5] = {64, (cuuint64_t)head_dim / 64, (cuuint64_t)page_size, (cuuint64_t)n_kv_heads, (cuuint64_t)num_pages};
        cuuint64_t strides[4] = {128, row, row * page_size, row * page_size * n_kv_heads};
        cuuint32_t box[5] = {64, 1, (cuuint32_t)pp.kv_rows, 1, 1};
        if (int e = pt_encode(&mk, k_pages, 5, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "the key pages")) return e;
        if (int e = pt_encode(&mv, v_pages, 5, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE, "the value pages")) return e;
    }
    int e = head_dim == 64 ? pt_launch<64>(mq, mk, mv, pp, n_tiles, stream) : pt_launch<128>(mq, mk, mv, pp, n_tiles, stream);
    if (e) return e;
    PB_CHECK_LAUNCH("attention_prefill_tc");
    return 0;
}
