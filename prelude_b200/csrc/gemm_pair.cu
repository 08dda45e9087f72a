// C = A * B^T for prompt steps on the fifth-generation tensor cores with PAIRED blocks: two multiprocessors
// share one 256 x 256 output tile (tcgen05.mma.cta_group::2).
//
//   A: [rows_a, K] bfloat16, K contiguous (the step's tokens)     B: [rows_b, K] bfloat16 (a weight matrix)
//   C[i, j] = sum_k A[i, k] * B[j, k], float32 accumulation, bfloat16 out
//
// Why pairs.  A 128 x 256 tile on one multiprocessor needs 48 KB of operands for every 512 cycles of products,
// 94 bytes a cycle, more than a multiprocessor draws from the L2 cache while all the others do the same; its tensor
// cores then wait.  In a pair each block holds 128 rows of A and HALF of the tile's 256 rows of B (32 KB per 512
// cycles), the instruction reads both blocks' shared memory, and each block's tensor memory receives its 128 rows of
// the result.  Measured on B200 at 2,048 x 6,144 x 2,560: 527 cycles for every 64 of K against the tensor cores' own
// 512.  No load is multicast: every block fetches its own halves with plain tensor-map copies
// (cp.async.bulk.tensor ... cta_group::2 only routes the completion to the leading block's barrier).
// (The reference sends these products to DeepGEMM / CUTLASS, both with 2-block tiles on sm_100:
// crates/prelude-cuda/deepgemm/src/sm100_bf16.cuh:10-205, crates/prelude-cuda/cutlass-gemm/src/cutlass_wrapper.cu:166-262.)
//
// The gated form serves a feed-forward's merged gate/up projection: B holds the N gate rows, then the N up rows;
// the leading block loads 128 gate rows, its partner the 128 up rows of the same features, so columns 0..127 of the
// accumulator are gate sums and 128..255 the up sums of those features, and the epilogue writes silu(gate) * up:
// the activation costs no kernel and the 2N-wide intermediate never exists.
//
// The q/k/v form serves the merged projection of an attention layer whose heads are 64, 128 or 256 wide: a tile
// holds whole heads and a thread a whole row of each, so the epilogue does what otherwise a kernel of its own does
// after the product - the per-head RMSNorm of queries and keys, the rotation by the token's position (the pair
// (j, j + head/2)), queries to their dense tensor and keys and values into the token's place in the cache pages -
// from the float32 sums, without the merged projection ever being written or read.
//
// Work.  Persistent pairs: pair p of P takes tiles p, p + P, ...; tiles run down the rows of A first, so that the
// pairs of a wave share a panel of B in the L2 cache.  (Dealing the last wave out in units of (tile, 64 of K), with
// the parts of a split tile summed through the L2 cache, was measured: the products are bound by power here, not by
// idle pairs - 64 pairs take as long as 74 - and the summing cost 10 us, so it did not pay.)
//
// In each block: warp 8 issues the tensor-map copies of its halves (six 32 KB stages), warp 9 of the LEADING block
// issues the products for both and commits to the barriers of both (tcgen05.commit ... multicast::cluster), warps
// 0..7 read the block's 128 accumulator rows out of tensor memory (two accumulators of 256 columns: one's stores
// overlap the next one's products; a warp reads the lanes of its number modulo four, so two warps share a row's
// columns) and store.  Every wait is bounded in time; a block that gives up raises the
// status word, and both blocks leave through the cluster's last barrier with their tensor memory freed.
#include "tcgen05.cuh"

#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define GP_BM 128                   // rows of A per block (256 per pair)
#define GP_BN 256                   // columns of the pair's tile (each block loads 128 rows of B)
#define GP_HALF 128
#define GP_BK 64
#define GP_STAGES 6
#define GP_THREADS 320                  // eight epilogue warps, one that copies, one that issues the products
#define GP_EPI_WARPS 8
#define GP_A_BYTES (GP_BM * GP_BK * 2)              // a stage's tile of A in one block
#define GP_STAGE_BYTES (2 * GP_A_BYTES)             // and as much of B

// What the q/k/v form needs beside the product (the arguments of the norm/rotary/cache-write kernel).
struct GpHeads {
    __nv_bfloat16* q_out;           // [tokens, n_heads, head_dim]
    __nv_bfloat16* k_pages;         // [pages, n_kv_heads, page_size, head_dim]
    __nv_bfloat16* v_pages;
    const float* q_weight;          // per-head norm scales, or null
    const float* k_weight;
    const float* cos_table;         // [max_positions, head_dim / 2]
    const float* sin_table;
    const int32_t* positions;
    const int32_t* token_seq;       // row of the block table per token; negative: a padding row
    const int32_t* block_table;
    float eps;
    int max_positions, table_stride, page_size, num_pages;
    int n_heads, n_kv_heads, head_dim, swizzle;
};

struct GpParams {
    GpHeads heads;
    __nv_bfloat16* out;             // [rows_a, out_cols]
    const float* bias;              // per output column, or null
    int* status;
    long long ldo;
    int rows_a, rows_b, K;          // rows_b: rows of B (2 * out_cols when gated)
    int out_cols;
    int tiles_m, tiles_n, kblocks;
    int gated;                      // 0: plain; 1: silu(gate) * up; 2: q/k/v heads
    int b_is_constant;
};

// ---- what the paired form adds to tcgen05.cuh ----
__device__ __forceinline__ uint32_t gp_map_to_rank(uint32_t smem_addr, uint32_t rank) {   // the same variable in another block of the cluster
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void gp_tmem_alloc2(uint32_t* holder, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(holder)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void gp_tmem_dealloc2(uint32_t taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
// a tile copy into this block's shared memory whose bytes are counted on a barrier of the LEADING block
// (`leader_bar`: a cluster-wide address); both blocks of the pair issue it, each for its own halves
__device__ __forceinline__ void gp_tma_load_2d(void* smem, const CUtensorMap* map, int c0, int c1, uint32_t leader_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(tc_smem(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void gp_mma2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// one arrival on the barrier at this address in BOTH blocks when the products issued so far have finished
__device__ __forceinline__ void gp_commit_both(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(tc_smem(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void gp_arrive_cluster(uint32_t bar) {      // `bar`: a cluster-wide address
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// bfloat16 x bfloat16 -> float32, M = 256 over the pair, N = 256, both operands K-major
__device__ __forceinline__ uint32_t gp_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GP_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

__device__ __forceinline__ void gp_bar_epilogue() { asm volatile("bar.sync 1, 256;\n" ::: "memory"); }
// 32 columns of this thread's row of the accumulator
__device__ __forceinline__ void gp_row_chunk(uint32_t taddr, float* v) {
    uint32_t r[32];
    tc_tmem_ld32(taddr, r);
    tc_tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}
// 32 values to bfloat16 at dst, of which `valid` exist
__device__ __forceinline__ void gp_store_chunk(__nv_bfloat16* dst, const float* v, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            unsigned w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
                w[j] = *reinterpret_cast<unsigned*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

// 32 values to bfloat16 as four 16-byte chunks of a head's row, chunk c of the row at position c ^ flip (the pages'
// permutation; 0 for none)
__device__ __forceinline__ void gp_store_head_chunks(__nv_bfloat16* row, int col, const float* v, int flip) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        unsigned w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
            w[j] = *reinterpret_cast<unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(row + (((col >> 3) + q) ^ flip) * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// The epilogue of the q/k/v form for one tile: this thread's token, the 256 / head_dim heads of the tile.
// (Norm, rotation and the cache write as crates/prelude-core/src/models/qwen3.rs:161-231 orders them; the same
// arithmetic as the kernel in rope_kv.cu, on the float32 sums instead of their bfloat16 rounding.)
__device__ __forceinline__ void gp_heads_epilogue(const GpParams& p, uint32_t taddr, int tn, int t, bool live, int side) {
    const GpHeads& r = p.heads;
    const int D = r.head_dim, half = D >> 1;
    const int pos = live ? r.positions[t] : 0;
    const int seq = (live && r.token_seq) ? r.token_seq[t] : 0;
    const bool padding = seq < 0;
    const bool pos_ok = pos >= 0 && pos < r.max_positions;
    bool page_known = false, page_ok = false;
    size_t page_row = 0;
    int in_page = 0;
    const int heads_per_tile = GP_BN / D, total_heads = r.n_heads + 2 * r.n_kv_heads;
    // the tile's heads are shared out between the two sets of epilogue warps (a single 256-wide head goes to the first)
    const int per_side = heads_per_tile > 1 ? heads_per_tile / 2 : 1;
    if (heads_per_tile == 1 && side == 1) return;
    for (int hh = side * per_side; hh < (side + 1) * per_side; ++hh) {
        const int slot = tn * heads_per_tile + hh;
        if (slot >= total_heads) break;                                     // the same for the whole block
        const bool is_q = slot < r.n_heads, is_k = !is_q && slot < r.n_heads + r.n_kv_heads;
        const int h = is_q ? slot : (is_k ? slot - r.n_heads : slot - r.n_heads - r.n_kv_heads);
        const uint32_t tcol = taddr + hh * D;
        bool store = live && !padding;
        __nv_bfloat16* dst = nullptr;
        int flip = 0;
        if (is_q) {
            dst = r.q_out + ((size_t)t * r.n_heads + h) * D;
        } else {
            if (!page_known && store) {                                     // the token's place in the cache, once
                page_known = true;
                const int page = pos >= 0 ? r.block_table[(size_t)seq * r.table_stride + pos / r.page_size] : -1;
                if (page < 0 || page >= r.num_pages) {
                    if (p.status) atomicExch(p.status, 2);
                } else {
                    page_ok = true;
                    in_page = pos % r.page_size;
                    page_row = (size_t)page * r.n_kv_heads;
                }
            }
            store = store && page_ok;
            dst = (is_k ? r.k_pages : r.v_pages) + ((page_row + h) * r.page_size + in_page) * D;
            flip = r.swizzle ? (in_page & 7) : 0;
        }
        if (!is_q && !is_k) {                                               // values: as they are
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                gp_row_chunk(tcol + c0, v);
                if (store) gp_store_head_chunks(dst, c0, v, flip);
            }
            continue;
        }
        const float* weight = is_q ? r.q_weight : r.k_weight;
        float inv = 1.0f;
        if (weight != nullptr) {
            float ss = 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                gp_row_chunk(tcol + c0, v);
#pragma unroll
                for (int j = 0; j < 32; ++j) ss += v[j] * v[j];
            }
            inv = 1.0f / sqrtf(ss / (float)D + r.eps);
        }
        if (store && !pos_ok) {
            if (p.status) atomicExch(p.status, 3);
            store = false;
        }
#pragma unroll 1
        for (int c0 = 0; c0 < half; c0 += 32) {
            float a[32], b[32];
            gp_row_chunk(tcol + c0, a);
            gp_row_chunk(tcol + half + c0, b);
            if (store) {
                if (weight != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 wa = *reinterpret_cast<const float4*>(weight + c0 + j), wb = *reinterpret_cast<const float4*>(weight + half + c0 + j);
                        a[j] *= inv * wa.x; a[j + 1] *= inv * wa.y; a[j + 2] *= inv * wa.z; a[j + 3] *= inv * wa.w;
                        b[j] *= inv * wb.x; b[j + 1] *= inv * wb.y; b[j + 2] *= inv * wb.z; b[j + 3] *= inv * wb.w;
                    }
                }
                const float4* cs = reinterpret_cast<const float4*>(r.cos_table + (size_t)pos * half + c0);
                const float4* sn = reinterpret_cast<const float4*>(r.sin_table + (size_t)pos * half + c0);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 c = cs[j], s = sn[j];
                    const float cc[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float x = a[4 * j + u], y = b[4 * j + u];
                        a[4 * j + u] = x * cc[u] - y * ss4[u];
                        b[4 * j + u] = y * cc[u] + x * ss4[u];
                    }
                }
                gp_store_head_chunks(dst, c0, a, flip);
                gp_store_head_chunks(dst, half + c0, b, flip);
            }
        }
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GP_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GpParams p) {
    pb_grid_dep_launch();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[GP_STAGES], empty_bar[GP_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_holder;
    __shared__ int s_ok;

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();             // 0: the leading block of the pair
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        s_ok = 1;
        for (int s = 0; s < GP_STAGES; ++s) { tc_mbar_init(&full_bar[s], 1); tc_mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { tc_mbar_init(&acc_full[a], 1); tc_mbar_init(&acc_empty[a], 2 * GP_EPI_WARPS); }   // the epilogue warps of both blocks
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 9) gp_tmem_alloc2(&tmem_holder, 512);       // one warp of each block, the same warp in both
    if (warp == 8 && lane == 0) { tc_prefetch_map(&map_a); tc_prefetch_map(&map_b); }
    tc_fence_before();
    cluster.sync();                                         // both blocks' barriers and tensor memory are set up
    tc_fence_after();
    const uint32_t tmem_base = tmem_holder;

    if (warp == 8) {
        // ---------------- copies: this block's 128 rows of A and its 128 rows of B for every stage ----------------
        if (lane == 0) {
            bool ok = true;
            int fill = 0;
            bool waited = false;
            if (!p.b_is_constant) { pb_grid_dep_wait(); waited = true; }
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int a_row = tm * 256 + rank * GP_BM;
                const int b_row = p.gated == 1 ? (rank == 0 ? tn * GP_HALF : p.out_cols + tn * GP_HALF) : tn * GP_BN + rank * GP_HALF;
                for (int kb = 0; kb < p.kblocks; ++kb, ++fill) {
                    const int stage = fill % GP_STAGES;
                    ok = tc_mbar_wait(&empty_bar[stage], ((fill / GP_STAGES) & 1) ^ 1);
                    if (!ok) break;
                    unsigned char* sa = smem + stage * GP_STAGE_BYTES;
                    const uint32_t leader_full = gp_map_to_rank(tc_smem(&full_bar[stage]), 0);
                    if (rank == 0) tc_mbar_expect_tx(&full_bar[stage], 2 * GP_STAGE_BYTES);   // both blocks' halves land on this barrier
                    // the weights are written by no kernel: their first copy need not wait for the kernel before this one
                    gp_tma_load_2d(sa + GP_A_BYTES, &map_b, kb * GP_BK, b_row, leader_full);
                    if (!waited) { pb_grid_dep_wait(); waited = true; }
                    gp_tma_load_2d(sa, &map_a, kb * GP_BK, a_row, leader_full);
                }
            }
            if (!ok && p.status) atomicExch(p.status, 8);
        }
    } else if (warp == 9) {
        // ---------------- products: the leading block issues for the pair ----------------
        if (rank == 0) {
            const uint32_t idesc = gp_idesc();
            int fill = 0, seg = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++seg) {
                const int acc = seg & 1;
                ok = __all_sync(0xffffffffu, tc_mbar_wait(&acc_empty[acc], ((seg >> 1) & 1) ^ 1));
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * GP_BN;
                for (int kb = 0; kb < p.kblocks; ++kb, ++fill) {
                    const int stage = fill % GP_STAGES;
                    ok = __all_sync(0xffffffffu, tc_mbar_wait(&full_bar[stage], (fill / GP_STAGES) & 1));
                    if (!ok) break;
                    tc_fence_after();
                    if (tc_elect_one()) {
                        const unsigned char* sa = smem + stage * GP_STAGE_BYTES;
                        const uint64_t da = tc_smem_desc(sa), db = tc_smem_desc(sa + GP_A_BYTES);
#pragma unroll
                        for (int k = 0; k < GP_BK / 16; ++k)
                            gp_mma2(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        gp_commit_both(&empty_bar[stage]);               // the stage is free in both blocks when these finish
                        if (kb + 1 == p.kblocks) gp_commit_both(&acc_full[acc]);
                    }
                    __syncwarp();
                }
            }
            if (!ok && lane == 0 && p.status) atomicExch(p.status, 9);
        }
    } else {
        // ---------------- epilogue: eight warps, this block's 128 accumulator rows ----------------
        // A warp reads the 32 tensor-memory lanes of its number modulo four; warps 0..3 take the first half of a
        // tile's columns (features, heads), warps 4..7 the second.
        pb_grid_dep_wait();                                 // the output may still be in use by the kernel before
        const int quarter = warp & 3, side = warp >> 2;
        const int row = quarter * 32 + lane;                // row of the block's half = tensor-memory lane
        int seg = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++seg) {
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int acc = seg & 1;
            if (ok) ok = tc_mbar_wait(&acc_full[acc], (seg >> 1) & 1);
            if (!ok) s_ok = 0;
            gp_bar_epilogue();
            if (!s_ok) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + acc * GP_BN + ((uint32_t)(quarter * 32) << 16);
            const int gi = tm * 256 + rank * GP_BM + row;
            const bool live = gi < p.rows_a;
            __nv_bfloat16* orow = p.out + (size_t)(live ? gi : 0) * p.ldo;
            if (p.gated == 2) {
                gp_heads_epilogue(p, taddr, tn, gi, live, side);
            } else if (p.gated) {
                const int col0 = tn * GP_HALF;
#pragma unroll 1
                for (int c0 = side * (GP_HALF / 2); c0 < (side + 1) * (GP_HALF / 2); c0 += 32) {
                    float g[32], up[32];
                    gp_row_chunk(taddr + c0, g);
                    gp_row_chunk(taddr + GP_HALF + c0, up);
#pragma unroll
                    for (int j = 0; j < 32; ++j) g[j] = g[j] / (1.0f + __expf(-g[j])) * up[j];
                    if (live && col0 + c0 < p.out_cols) gp_store_chunk(orow + col0 + c0, g, p.out_cols - (col0 + c0));
                    __syncwarp();
                }
            } else {
                const int col0 = tn * GP_BN;
#pragma unroll 1
                for (int c0 = side * (GP_BN / 2); c0 < (side + 1) * (GP_BN / 2); c0 += 32) {
                    float v[32];
                    gp_row_chunk(taddr + c0, v);
                    if (live && col0 + c0 < p.out_cols) {
                        if (p.bias) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + c0 + j < p.out_cols) v[j] += p.bias[col0 + c0 + j];
                        }
                        gp_store_chunk(orow + col0 + c0, v, p.out_cols - (col0 + c0));
                    }
                    __syncwarp();
                }
            }
            // the accumulator may be overwritten: tell the leading block, which issues the products
            tc_fence_before();
            __syncwarp();
            if (lane == 0) gp_arrive_cluster(gp_map_to_rank(tc_smem(&acc_empty[acc]), 0));
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 10);
    }
    // nobody touches the other block's shared memory, barriers or tensor memory after this
    tc_fence_before();
    cluster.sync();
    if (warp == 9) {
        __syncwarp();
        tc_fence_after();
        gp_tmem_dealloc2(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static int gp_make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {GP_BK, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pb_fail("gemm_pair: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d ld=%lld)", (int)r, rows, K, ld);
    return 0;
}

static int gp_max_pairs() {
    static int pairs = 0;
    if (pairs == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        pairs = sms > 1 ? sms / 2 : 74;
    }
    return pairs;
}

static int gp_launch(const void* A, const void* B, long long lda, long long ldb, GpParams& p, int max_pairs, cudaStream_t stream) {
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    PB_REQUIRE(tiles < (1ll << 30), "gemm_pair: %lld tiles are too many", tiles);
    long long pairs = gp_max_pairs();
    if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
    if (tiles < pairs) pairs = tiles;
    CUtensorMap ma, mb;
    if (int e = gp_make_map(&ma, A, p.rows_a, p.K, lda)) return e;
    if (int e = gp_make_map(&mb, B, p.rows_b, p.K, ldb)) return e;
    const size_t smem = (size_t)GP_STAGES * GP_STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("gemm_pair: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(gemm_pair_kernel, dim3((unsigned)(2 * pairs)), dim3(GP_THREADS), smem, stream, ma, mb, p);
    PB_CHECK_LAUNCH("gemm_pair");
    return 0;
}

// Whether the kernel takes the shape: 16-byte aligned rows (K and the strides multiples of 8 elements); the gated
// form needs an even number of rows of B.
PB_API int pb_gemm_pair_supported(int rows_a, int rows_b, int K, long long lda, long long ldb, int gated) {
    if (rows_a < 1 || rows_b < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8) return 0;
    if (gated && rows_b % 2) return 0;
    return 1;
}

// out[i * ldo + j] = sum_k A[i, k] B[j, k] (+ bias[j]), bfloat16; gated: B is [2 N, K], N gate rows then N up rows, and
// out[i * ldo + j] = silu(sum_k A[i, k] B[j, k]) * (sum_k A[i, k] B[N + j, k]) for j < N (no bias).
// b_is_constant: no kernel writes B (a weight matrix).  max_pairs: 0, or fewer pairs than the device has (tests).
PB_API int pb_gemm_pair_bf16(const void* A, const void* B, const float* bias, void* out, int rows_a, int rows_b, int K,
                             long long lda, long long ldb, long long ldo, int gated, int b_is_constant, int max_pairs,
                             int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_gemm_pair_supported(rows_a, rows_b, K, lda, ldb, gated),
               "gemm_pair: rows_a=%d rows_b=%d K=%d lda=%lld ldb=%lld not taken (rows must be 16-byte aligned)", rows_a, rows_b, K, lda, ldb);
    PB_REQUIRE(A && B && out && pb_aligned(A, 16) && pb_aligned(B, 16), "gemm_pair: null or unaligned pointer");
    PB_REQUIRE(!gated || bias == nullptr, "gemm_pair: the gated form takes no bias");
    if (int e = get_encode()) return e;
    GpParams p{};
    p.out = (__nv_bfloat16*)out; p.bias = bias; p.status = status; p.ldo = ldo;
    p.rows_a = rows_a; p.rows_b = rows_b; p.K = K; p.gated = gated ? 1 : 0; p.b_is_constant = b_is_constant;
    p.out_cols = gated ? rows_b / 2 : rows_b;
    p.tiles_m = (rows_a + 255) / 256;
    p.tiles_n = gated ? (p.out_cols + GP_HALF - 1) / GP_HALF : (p.out_cols + GP_BN - 1) / GP_BN;
    p.kblocks = (K + GP_BK - 1) / GP_BK;
    return gp_launch(A, B, lda, ldb, p, max_pairs, stream);
}

// Whether the q/k/v form takes the layer: heads of 64, 128 or 256, rotation of the whole head by halves.
PB_API int pb_gemm_pair_heads_supported(int rows_a, int K, long long lda, long long ldb, int n_heads, int n_kv_heads, int head_dim, int rotary_dim) {
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return 0;
    if (rotary_dim != head_dim || n_heads < 1 || n_kv_heads < 0) return 0;
    return pb_gemm_pair_supported(rows_a, (n_heads + 2 * n_kv_heads) * head_dim, K, lda, ldb, 0);
}

// x [rows_a, K] against the merged q/k/v weight [(n_heads + 2 n_kv_heads) head_dim, K]; then per head what
// pb_qknorm_rope_kvwrite does with the projection, in the product's epilogue: queries (normalised with q_weight
// if given, rotated) to q_out [rows_a, n_heads, head_dim], keys (k_weight) and values into the pages at
// block_table[token_seq[t]][positions[t] / page_size].  n_kv_heads == 0: queries only (a layer that reads another
// layer's cache).  Status 2: a token without a page; 3: a position outside the tables.
PB_API int pb_gemm_pair_heads_bf16(const void* A, const void* B, int rows_a, int K, long long lda, long long ldb,
                                   void* q_out, void* k_pages, void* v_pages, const float* q_weight, const float* k_weight, float eps,
                                   const float* cos_table, const float* sin_table, int max_positions, const int32_t* positions,
                                   const int32_t* token_seq, const int32_t* block_table, int table_stride, int page_size, int num_pages,
                                   int n_heads, int n_kv_heads, int head_dim, int swizzle, int max_pairs, int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_gemm_pair_heads_supported(rows_a, K, lda, ldb, n_heads, n_kv_heads, head_dim, head_dim),
               "gemm_pair: q/k/v form: rows_a=%d K=%d heads %d + 2 x %d of %d not taken", rows_a, K, n_heads, n_kv_heads, head_dim);
    PB_REQUIRE(A && B && q_out && cos_table && sin_table && positions && pb_aligned(A, 16) && pb_aligned(B, 16) && pb_aligned(q_out, 16) &&
               pb_aligned(cos_table, 16) && pb_aligned(sin_table, 16) && (!q_weight || pb_aligned(q_weight, 16)) && (!k_weight || pb_aligned(k_weight, 16)),
               "gemm_pair: q/k/v form: null or unaligned pointer");
    if (n_kv_heads > 0)
        PB_REQUIRE(k_pages && v_pages && token_seq && block_table && page_size > 0 && num_pages > 0 && pb_aligned(k_pages, 16) && pb_aligned(v_pages, 16),
                   "gemm_pair: q/k/v form: cache write asked for without cache arguments");
    PB_REQUIRE(!swizzle || head_dim % 64 == 0, "gemm_pair: permuted pages have head_dim %% 64 == 0");
    if (int e = get_encode()) return e;
    GpParams p{};
    p.status = status;
    p.rows_a = rows_a; p.rows_b = (n_heads + 2 * n_kv_heads) * head_dim; p.K = K; p.gated = 2; p.b_is_constant = 1;
    p.out_cols = p.rows_b;
    p.tiles_m = (rows_a + 255) / 256;
    p.tiles_n = (p.out_cols + GP_BN - 1) / GP_BN;
    p.kblocks = (K + GP_BK - 1) / GP_BK;
    GpHeads& r = p.heads;
    r.q_out = (__nv_bfloat16*)q_out; r.k_pages = (__nv_bfloat16*)k_pages; r.v_pages = (__nv_bfloat16*)v_pages;
    r.q_weight = q_weight; r.k_weight = k_weight; r.cos_table = cos_table; r.sin_table = sin_table;
    r.positions = positions; r.token_seq = token_seq; r.block_table = block_table; r.eps = eps;
    r.max_positions = max_positions; r.table_stride = table_stride; r.page_size = page_size; r.num_pages = num_pages;
    r.n_heads = n_heads; r.n_kv_heads = n_kv_heads; r.head_dim = head_dim; r.swizzle = swizzle;
    return gp_launch(A, B, lda, ldb, p, max_pairs, stream);
}
