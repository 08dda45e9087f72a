// Tensor-core paged attention for prompt portions (and any mix of portions and
// single tokens), bfloat16.
//
// For a query at absolute position p of request r and query head h (key/value
// head h / G):
//     o = softmax_j( (q . k_j) * scale ) v_j    over  max(0, p - window + 1) <= j <= p
// with k_j, v_j read from the request's pages through its block table
// (crates/prelude-core/src/models/qwen3.rs:191-222; the reference hands this to
// FlashAttention-4 / FlashInfer, crates/prelude-cuda/src/attn/flash_v4.rs:125-278).
// Scores and the running softmax (maximum, sum, rescaling) are float32; the
// probabilities are rounded to bfloat16 for the second product, whose
// accumulator is float32.
//
// Layout of the work.  The host lists tiles: a tile is 64 rows = 64/G tokens x
// the G query heads that share a key/value head, of one request, so keys and
// values are read once per group.  A block owns one tile and one key/value head;
// each of its four compute warps owns 16 rows and walks all visible keys in
// tiles of 64.  Two ways of bringing the key and value tiles into shared memory:
//   bulk - a fifth warp fetches, per tile, each page's run of one head with a
//          single bulk copy (cp.async.bulk) into a ring of stages, each with a
//          full and an empty barrier; the runs are stored with permuted 16-byte
//          chunks (pb_kv_elem_offset), so they land ready for conflict-free
//          ldmatrix.  No block-wide barrier in the loop.  Taken when pages are
//          permuted, head_dim is 64, 128 or 256 and a page's run tiles a
//          64-key tile evenly.
//   lsu  - the four warps copy 16 bytes per lane (cp.async) into padded rows,
//          double buffered, with a block-wide barrier per tile; any head size
//          (multiples of 16 up to 256) and page size.
// The inner loops are written for few instructions per tensor-core product:
// the byte offsets of every ldmatrix are per-thread constants plus immediates,
// masking runs only in tiles that hold an invisible key, the scale is folded
// into the exponent's multiply-add, and the accumulator is rescaled only when
// a row's maximum grew by more than 2^8 (the sum and the accumulator then stay
// relative to a slightly stale maximum, which the final division cancels).
#include "attention_common.cuh"

#define PF_ROWS 64              // rows of a block's tile
#define PF_COMPUTE_THREADS 128

template <int DMAX, bool BULK> struct PrefillTiling {
    static constexpr int STRIDE = BULK ? DMAX : DMAX + 8;     // elements per row in shared memory
    static constexpr int ROW_BYTES = STRIDE * 2;
    static constexpr int TILE_BYTES = BN * ROW_BYTES;          // one tile of keys (or of values)
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int STAGES = BULK ? (DMAX <= 128 ? 3 : 2) : 2;
    static constexpr int Q_BYTES = PF_ROWS * ROW_BYTES;
    static constexpr int SMEM_BYTES = Q_BYTES + STAGES * STAGE_BYTES;
    static constexpr int THREADS = BULK ? PF_COMPUTE_THREADS + 32 : PF_COMPUTE_THREADS;
    static constexpr int BLOCKS_PER_SM = (2 * (SMEM_BYTES + 1024) <= 227 * 1024) ? 2 : 1;
};

struct PrefillParams {
    AttnParams a;
    int page_shift;             // log2(page_size) when it is a power of two, else -1
};

__device__ __forceinline__ void pf_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// Keys and values of one tile through the load/store path: thread `tid` of 128 copies 16-byte chunk
// `ch` of rows row0, row0 + rows_per_pass, ...; rows outside [kv_begin, kv_end) are zero-filled.
// Pages below kv_begin may have been given back already and are never looked up.
template <int DMAX>
__device__ __forceinline__ void load_kv_tile_lsu(unsigned char* sK, unsigned char* sV, const AttnParams& p,
                                                 const int32_t* table, int kvh, int key0, int kv_begin, int kv_end,
                                                 int row0, int ch, int rows_per_pass) {
    constexpr int ROW_BYTES = (DMAX + 8) * 2;
    if (row0 >= rows_per_pass) return;                     // threads beyond the last whole row of a pass
    const int ps = p.page_size, d = p.head_dim;
    int j = key0 + row0;
    int pi = j / ps, in_page = j - pi * ps;
    for (int row = row0; row < BN; row += rows_per_pass) {
        bool ok = j >= kv_begin && j < kv_end;
        size_t src = 0;
        if (ok) {
            const int page = table[pi];
            if (page < 0 || page >= p.num_pages) {
                ok = false;
                if (p.status) atomicExch(p.status, 6);
            } else {
                src = (((size_t)page * p.n_kv_heads + kvh) * ps + in_page) * d + (p.swizzle ? ((ch ^ (in_page & 7)) * 8) : ch * 8);
            }
        }
        cp_async16(sK + row * ROW_BYTES + ch * 16, p.k_pages + src, ok);
        cp_async16(sV + row * ROW_BYTES + ch * 16, p.v_pages + src, ok);
        j += rows_per_pass;
        in_page += rows_per_pass;
        while (in_page >= ps) { in_page -= ps; ++pi; }
    }
}

template <int DMAX, bool BULK>
__global__ void __launch_bounds__(PrefillTiling<DMAX, BULK>::THREADS, PrefillTiling<DMAX, BULK>::BLOCKS_PER_SM)
attn_prefill_kernel(PrefillParams pp) {
    pb_grid_dep_launch();
    using T = PrefillTiling<DMAX, BULK>;
    const AttnParams& p = pp.a;
    constexpr int S = T::STAGES;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* sQ = smem_raw;
    unsigned char* stages = smem_raw + T::Q_BYTES;
    __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S];
    __shared__ int s_issued;

    const int G = p.group, d = p.head_dim, ps = p.page_size;
    const int tpt = PF_ROWS / G;                           // tokens per tile
    const int tile = blockIdx.x / p.n_kv_heads, kvh = blockIdx.x - tile * p.n_kv_heads;
    const int r = p.tile_seq[tile], tok0 = p.tile_tok0[tile];
    const int q_base = p.cu_q[r], q_len = p.cu_q[r + 1] - q_base, pos0 = p.q_start[r];
    const int n_tok = min(tpt, q_len - tok0);              // tokens of this tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int32_t* table = p.block_table + (size_t)p.token_seq[q_base + tok0] * p.table_stride;
    const int p_min = pos0 + tok0, p_max = pos0 + tok0 + n_tok - 1;
    const int lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt0 = lo / BN, kt1 = p_max / BN;
    const int n_tiles = kt1 - kt0 + 1;
    const int kv_end = p_max + 1;

    if (BULK && threadIdx.x == 0) {
        s_issued = 0;
#pragma unroll
        for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], PF_COMPUTE_THREADS / 32); }
        mbar_fence_init();
    }
    // the batch's index arrays were written before the previous kernel started; q and the newest keys
    // and values are that kernel's output
    pb_grid_dep_wait();

    // Q rows: row i -> token tok0 + i / G, head kvh * G + i % G; rows without a token are zero
    {
        const int chunks = d >> 3;
        for (int c = threadIdx.x; c < PF_ROWS * chunks; c += T::THREADS) {
            const int row = c / chunks, ch = c - row * chunks;
            const int tl = row / G, hg = row - tl * G;
            const bool ok = tl < n_tok;
            const size_t src = ok ? (((size_t)(q_base + tok0 + tl) * p.n_heads + kvh * G + hg) * d + ch * 8) : 0;
            cp_async16(sQ + row * T::ROW_BYTES + ((BULK ? (ch ^ (row & 7)) : ch) << 4), p.q + src, ok);
        }
        cp_async_commit();
    }

    if (BULK && warp == PF_COMPUTE_THREADS / 32) {
        cp_async_wait<0>();
        __syncthreads();                                   // barriers and q are ready
        // ---------------- loader warp: lane u fetches the u-th run of keys and of values of every tile ----------------
        const int run_rows = min(ps, BN);                  // tokens one copy brings: a page's run, or 64 of it
        const int runs = BN / run_rows;
        const unsigned run_bytes = (unsigned)run_rows * T::ROW_BYTES;
        auto page_of = [&](int j0, bool& want, size_t& src) {
            want = lane < runs && j0 <= p_max && j0 + run_rows > lo;       // the run holds a visible key
            src = 0;
            if (want) {
                const int pi = pp.page_shift >= 0 ? (j0 >> pp.page_shift) : (j0 / ps);
                const int page = table[pi];
                if (page < 0 || page >= p.num_pages) {
                    want = false;                          // never read outside the pool; the step is reported as bad
                    if (p.status) atomicExch(p.status, 6);
                } else {
                    src = (((size_t)page * p.n_kv_heads + kvh) * ps + (j0 - pi * ps)) * d;
                }
            }
        };
        bool want, ok = true;
        size_t src;
        page_of(kt0 * BN + lane * run_rows, want, src);
        int stage = 0, phase = 0;
#pragma unroll 1
        for (int i = 0; i < n_tiles; ++i) {
            ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            if (lane == 0) *(volatile int*)&s_issued = i + 1;              // the stage's previous tenant has been consumed
            unsigned char* sK = stages + stage * T::STAGE_BYTES;
            unsigned char* sV = sK + T::TILE_BYTES;
            const unsigned n_want = __popc(__ballot_sync(0xffffffffu, want));
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], n_want * run_bytes * 2);
            __syncwarp();
            if (want) {
                bulk_copy_g2s(sK + lane * run_bytes, p.k_pages + src, run_bytes, &full_bar[stage]);
                bulk_copy_g2s(sV + lane * run_bytes, p.v_pages + src, run_bytes, &full_bar[stage]);
            }
            if (i + 1 < n_tiles) page_of((kt0 + i + 1) * BN + lane * run_rows, want, src);   // the next tile's page, ahead of its turn
            if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 7);
        return;
    }

    // ---------------- compute warps ----------------
    // this thread's two rows, and what the warp's 16 rows can see
    int row_pos[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int tl = (warp * 16 + g + 8 * h) / G;
        row_pos[h] = tl < n_tok ? pos0 + tok0 + tl : -1;   // -1: no key is visible
    }
    const int tl_first = (warp * 16) / G, tl_last = (warp * 16 + 15) / G;
    const bool warp_has_rows = tl_first < n_tok;
    const bool warp_full = tl_last < n_tok;
    const int wp_min = pos0 + tok0 + tl_first, wp_max = pos0 + tok0 + min(tl_last, n_tok - 1);

    FragOffsets<DMAX, BULK> f;
    attn_frag_offsets<DMAX, BULK>(f, warp * 16, lane);
    const unsigned sQ_a = smem_u32(sQ);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    auto tile_edge = [&](int key0) {                       // some key of the tile is invisible to some row of the warp
        return !warp_full || key0 + BN - 1 > wp_min || (p.window > 0 && key0 < wp_max - p.window + 1);
    };
    auto tile_unseen = [&](int key0) {                     // no row of the warp sees any key of the tile
        return !warp_has_rows || key0 > wp_max || (p.window > 0 && key0 + BN - 1 < wp_min - p.window + 1);
    };

    if constexpr (BULK) {
        cp_async_wait<0>();
        __syncthreads();                                   // barriers and q are ready
        int stage = 0, phase = 0;
#pragma unroll 1
        for (int i = 0; i < n_tiles; ++i) {
            bool landed = true;
            if (*(volatile int*)&s_issued <= i) {          // not announced yet: the barrier may still be in an older phase
                const long long t0 = clock64();
                while (*(volatile int*)&s_issued <= i)
                    if (clock64() - t0 > (1ll << 31)) { landed = false; break; }
            }
            landed = landed && mbar_wait_bounded(&full_bar[stage], phase);
            if (!__all_sync(0xffffffffu, landed)) {        // gave up waiting: report, do not hang
                if (lane == 0 && p.status) atomicExch(p.status, 7);
                break;
            }
            unsigned char* sK = stages + stage * T::STAGE_BYTES;
            unsigned char* sV = sK + T::TILE_BYTES;
            const int key0 = (kt0 + i) * BN;
            if (!tile_unseen(key0)) {
                if (key0 + BN - 1 > p_max || key0 < lo) {
                    // value rows that no visible key stands for hold whatever the page (or the stage) held: zeros
                    // instead, so that 0 * (whatever is there) cannot make a NaN.  Every warp writes the same zeros.
                    for (int rr = lane; rr < BN; rr += 32) {
                        const int j = key0 + rr;
                        if (j < lo || j > p_max)
                            for (int c = 0; c < DMAX / 8; ++c)
                                *reinterpret_cast<uint4*>(sV + rr * T::ROW_BYTES + c * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();                   // these ordinary stores come before the bulk copy that refills the stage
                    __syncwarp();
                }
                attn_tile<DMAX, BULK>(o, m, l, f, sQ_a, smem_u32(sK), smem_u32(sV), d, key0, row_pos, tile_edge(key0),
                                         p.window, p.scale_log2, t4);
            }
            __syncwarp();
            if (lane == 0) pf_mbar_arrive(&empty_bar[stage]);              // this warp is done with the stage
            if (++stage == S) { stage = 0; phase ^= 1; }
        }
    } else {
        const int chunks = d >> 3;
        const int rows_per_pass = PF_COMPUTE_THREADS / chunks;
        const int row0 = threadIdx.x / chunks, ch = threadIdx.x - row0 * chunks;
        load_kv_tile_lsu<DMAX>(stages, stages + T::TILE_BYTES, p, table, kvh, kt0 * BN, lo, kv_end, row0, ch, rows_per_pass);
        cp_async_commit();
#pragma unroll 1
        for (int i = 0; i < n_tiles; ++i) {
            unsigned char* sK = stages + (i & 1) * T::STAGE_BYTES;
            unsigned char* sV = sK + T::TILE_BYTES;
            if (i + 1 < n_tiles) {
                unsigned char* nK = stages + ((i + 1) & 1) * T::STAGE_BYTES;
                load_kv_tile_lsu<DMAX>(nK, nK + T::TILE_BYTES, p, table, kvh, (kt0 + i + 1) * BN, lo, kv_end, row0, ch, rows_per_pass);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            const int key0 = (kt0 + i) * BN;
            if (!tile_unseen(key0))
                attn_tile<DMAX, BULK>(o, m, l, f, sQ_a, smem_u32(sK), smem_u32(sV), d, key0, row_pos, tile_edge(key0),
                                         p.window, p.scale_log2, t4);
            __syncthreads();
        }
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

template <int DMAX, bool BULK>
static int launch_prefill(const PrefillParams& pp, int n_tiles, cudaStream_t stream) {
    using T = PrefillTiling<DMAX, BULK>;
    static bool configured = false;
    const size_t smem = T::SMEM_BYTES;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<DMAX, BULK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(attn_prefill_kernel<DMAX, BULK>, dim3((unsigned)n_tiles * pp.a.n_kv_heads), dim3(T::THREADS), smem, stream, pp);
    return 0;
}

// Tiles are listed by the host: tile t covers tokens tile_tok0[t] .. of request tile_seq[t]'s portion,
// 64 / (n_heads / n_kv_heads) tokens each; listing the tiles that see the most keys first shortens the tail.
PB_API int pb_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                     const int32_t* block_table, int table_stride, const int32_t* positions,
                                     const int32_t* token_seq, const int32_t* cu_q, const int32_t* q_start,
                                     const int32_t* tile_seq, const int32_t* tile_tok0, int n_tiles, int page_size,
                                     int num_pages, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     float scale, int window, int swizzle, int* status, cudaStream_t stream) {
    PrefillParams pp{};
    AttnParams& p = pp.a;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.cu_q = cu_q; p.q_start = q_start; p.tile_seq = tile_seq; p.tile_tok0 = tile_tok0; p.n_splits = 1;
    p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages; p.n_tokens = n_tokens;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.swizzle = swizzle;
    if (int e = attn_check_common("attention_prefill", p)) return e;
    PB_REQUIRE(scale > 0.f, "attention_prefill: scale=%g; the kernel takes the row maximum before scaling", (double)scale);
    PB_REQUIRE(!swizzle || head_dim % 64 == 0, "attention_prefill: permuted pages need head_dim %% 64 == 0");
    p.group = n_heads / n_kv_heads;
    PB_REQUIRE(p.group <= 64, "attention_prefill: %d query heads per key/value head; at most 64 fit a tile", p.group);
    PB_REQUIRE(n_tiles >= 0 && (long long)n_tiles * n_kv_heads < (1ll << 31), "attention_prefill: bad grid");
    if (n_tiles == 0 || n_tokens == 0) return 0;
    pp.page_shift = -1;
    for (int s = 0; s < 31; ++s)
        if ((1 << s) == page_size) pp.page_shift = s;
    // bulk copies bring whole runs of a page: a run must tile the 64-key tile evenly and start at a multiple
    // of 8 tokens (the rows then sit at the row numbers their permutation was made for)
    const bool bulk = swizzle && page_size % 8 == 0 && (BN % page_size == 0 || page_size % BN == 0) &&
                      (head_dim == 64 || head_dim == 128 || head_dim == 256);
    int e = bulk ? (head_dim == 64 ? launch_prefill<64, true>(pp, n_tiles, stream)
                    : head_dim == 128 ? launch_prefill<128, true>(pp, n_tiles, stream) : launch_prefill<256, true>(pp, n_tiles, stream))
                 : (head_dim <= 64 ? launch_prefill<64, false>(pp, n_tiles, stream)
                    : head_dim <= 128 ? launch_prefill<128, false>(pp, n_tiles, stream) : launch_prefill<256, false>(pp, n_tiles, stream));
    if (e) return e;
    PB_CHECK_LAUNCH("attention_prefill");
    return 0;
}
