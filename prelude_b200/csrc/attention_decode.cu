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
// request is read once, so the kernel is arranged to keep many bytes in flight
// and to keep the arithmetic out of the way of the loads.
//  * A block owns one (token, key/value head) and a contiguous share of that
//    request's 64-key tiles.  The G query heads of the group are the rows of the
//    tensor-core tile, so the group's keys and values are read once.
//  * Tiles go into a ring of shared-memory stages with a full and an empty
//    barrier each; as many tiles are in flight as shared memory holds.  The page
//    ids of the block's whole share are fetched into shared memory first.
//    Two ways of bringing a tile in:
//      bulk - one head's tokens of one page are one contiguous run of memory
//             (a few KB), stored with permuted 16-byte chunks (pb_kv_elem_offset);
//             one lane fetches each run with a single bulk copy
//             (cp.async.bulk) that completes on the stage's barrier, and the run
//             lands in shared memory ready for conflict-free ldmatrix.  Measured
//             on B200: 4 KB bulk copies reach the full memory bandwidth (42 GB/s
//             per multiprocessor), 256-byte ones 9 GB/s, tensor-map boxes of 16
//             rows x 128 bytes 22 GB/s, 16-byte copies through the load/store path
//             about 25 GB/s.  Used when pages are permuted and page_size % 8 == 0.
//      lsu  - four loader warps copy 16 bytes per lane (cp.async) into padded
//             rows; any head size and page size.
//  * Consumer warps (four; as many as there are stages when fewer fit) take whole
//    64-key tiles in turn (tile i goes to warp i mod 4):
//    scores, running maximum and sum in float32, probabilities rounded to
//    bfloat16 for the second product.  No block-wide barrier in the loop.  The
//    warps are merged through shared memory at the end.
//  * With more than one split, the blocks of a (token, key/value head) are
//    launched as one thread-block cluster where the device can place it (up to
//    16 blocks): every block leaves its unnormalised partial result with its
//    maximum and sum in its own shared memory, the cluster meets at its
//    barrier, and every block adds up a slice of the output elements over all
//    blocks, in ascending order, reading the others' parts through distributed
//    shared memory.  No scratch memory, no fence, no counter, no reload: the
//    end of the kernel is two cluster barriers and one remote read.
//  * Splits that do not fit a cluster go through scratch memory: every block
//    writes its part there and counts itself in; the block that arrives last
//    adds the splits up in ascending order and writes the output.  The
//    counters are left at zero for the next call.
//  * All keys and values but the newest were written by earlier steps, so the
//    loaders start the stream before the kernel that precedes this one on the
//    stream (it writes q and the newest key and value) has finished, and wait
//    for it only before the request's last tile; the consumers wait for it
//    before they fetch q.
//  * Waits on barriers are bounded in time: a warp that gives up raises the
//    step's status word and goes on to the end.
#include "attention_common.cuh"

#include <stdlib.h>
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

PB_TIMELINE_UNIT(attention_decode)

#define DEC_LOADERS 128         // threads of the lsu path's four loader warps
#define DEC_MAX_CLUSTER 16      // blocks of one (token, key/value head) that may form a thread-block cluster
#define DEC_MAX_PAGES 512       // page ids of one block's share kept in shared memory (else read from the table)

struct DecodeParams {
    AttnParams a;
    int* counters;              // [n_tokens * n_kv_heads], zero on entry and on exit
    int page_shift;             // log2(page_size) when it is a power of two, else -1
    int cluster;                // the blocks of a (token, key/value head) are one thread-block cluster: they add
                                // their parts up through each other's shared memory instead of scratch memory
};

#define BNW 64                  // keys per consumer tile

// One ring of stages shared by all warps; tile i lives in stage i % STAGES and is consumed by warp i % NC.
// A barrier wait can tell only the current phase from the one before it, so a consumer must not start
// to wait for tile i before tile i - STAGES (the stage's previous tenant) has been consumed: it first
// waits until the loaders have announced tile i (s_issued), which they do only after that.
// PAIR: two blocks per multiprocessor with half the ring each, for steps with more (token, head) pairs than
// multiprocessors - one block's start and end then overlap the other's stream.  (Bulk path, head sizes up to 128.)
template <int DMAX, bool BULK, bool PAIR> struct DecodeTiling {
    static constexpr int STRIDE = BULK ? DMAX : DMAX + 8;    // lsu: padded rows; bulk: dense rows with permuted chunks
    static constexpr int STAGE_ELEMS = 2 * BNW * STRIDE;     // K rows then V rows
    static constexpr int FIT = ((PAIR ? 98 : 200) * 1024) / (STAGE_ELEMS * 2);
    static constexpr int STAGES = FIT > 8 ? 8 : FIT;
    static constexpr int NC = STAGES < 4 ? STAGES : 4;       // consumer warps
    static constexpr int THREADS = PAIR ? 160 : 256;         // four consumer warps and one loader warp (two blocks share the registers), or four
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// the barrier gets this thread's arrival when all its earlier asynchronous copies have landed
__device__ __forceinline__ void cp_async_arrive_on(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

template <int DMAX, bool BULK, bool PAIR>
__global__ void __launch_bounds__((DecodeTiling<DMAX, BULK, PAIR>::THREADS), (PAIR ? 2 : 1)) attn_decode_kernel(DecodeParams dp) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_ATTN_DECODE, PB_TL_ENTRY);
    using T = DecodeTiling<DMAX, BULK, PAIR>;
    constexpr int DEC_THREADS = T::THREADS;
    const AttnParams& p = dp.a;
    constexpr int STRIDE = T::STRIDE;
    constexpr int S = T::STAGES, NC = T::NC;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    using TG = AttnTileGeom<DMAX, BULK>;                     // q rows are laid out like key rows: padded, or dense with permuted chunks
    constexpr int QSTRIDE = TG::STRIDE;
    __nv_bfloat16* sQ = stages + S * T::STAGE_ELEMS;
    int32_t* s_pages = reinterpret_cast<int32_t*>(sQ + 16 * (DMAX + 8));
    __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S];
    __shared__ int s_last, s_issued;

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

    if (kt0 <= kt1) {
        if (threadIdx.x == 0) {
            s_issued = 0;
#pragma unroll
            for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], BULK ? 1 : DEC_LOADERS); mbar_init(&empty_bar[s], 1); }
            mbar_fence_init();
        }
        // page ids of keys [key_first, key_last] of this block
        const int key_first = max(lo, kt0 * BN), key_last = min(pos, kt1 * BN + BN - 1);
        const int page_first = key_first / ps, n_pages = key_last / ps - page_first + 1;
        const bool pages_in_smem = n_pages <= DEC_MAX_PAGES;
        if (pages_in_smem)
            for (int i = threadIdx.x; i < n_pages; i += DEC_THREADS) s_pages[i] = table[page_first + i];
        __syncthreads();                                    // barriers and s_pages are ready
        // Positions and block tables were written before this step's first kernel started, and so were all keys
        // and values but the newest: the kernel before this one writes those (and q).  The loaders therefore
        // start the stream at once and wait for that kernel only before the tile that holds the newest key; the
        // consumers wait for it before they fetch q.
        const int chunks = d >> 3;
        const bool holds_newest = kt1 == kt_hi;             // this block's last tile is the request's last
        if (warp < 4) {
            pb_grid_dep_wait();
            PB_TL(PB_TL_ATTN_DECODE, PB_TL_AFTER_WAIT);
            // q rows of the group (rows from G on are zero)
            for (int c = threadIdx.x; c < 16 * chunks; c += 128) {
                const int row = c / chunks, ch = c - row * chunks;
                const bool ok = row < G;
                const size_t src = ok ? (((size_t)tok * p.n_heads + kvh * G + row) * d + ch * 8) : 0;
                cp_async16(sQ + row * QSTRIDE + (BULK ? (ch ^ (row & 7)) : ch) * 8, p.q + src, ok);
            }
            cp_async_commit();
            cp_async_wait<0>();
            asm volatile("bar.sync 1, 128;\n" ::: "memory");   // q is ready (the four consumer warps only)
            PB_TL(PB_TL_ATTN_DECODE, PB_TL_INPUT);
        }

        const int n_tiles = (kt1 - kt0 + 1) * (BN / BNW);   // consumer tiles of BNW keys; tile i belongs to warp i % NC
        const int key_base = kt0 * BN;
        const int row_elems = BULK ? d : STRIDE;            // elements between rows of a key or value tile
        if (BULK && warp >= 4) {
            // ---------------- bulk loader: lane u of warp 4 fetches the u-th run of keys and of values ----------------
            if (warp == 4) {
                const int run_rows = min(ps, BNW);          // tokens one copy brings: a page's run, or BNW of it
                const int runs = BNW / run_rows;
                const unsigned run_bytes = (unsigned)run_rows * d * 2;
                bool ok = true;
#pragma unroll 1
                for (int i = 0; i < n_tiles; ++i) {
                    const int stage = i % S;
                    if (holds_newest && i == n_tiles - 1) pb_grid_dep_wait();
                    ok = mbar_wait_bounded(&empty_bar[stage], ((i / S) & 1) ^ 1);
                    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    if (lane == 0) *(volatile int*)&s_issued = i + 1;       // the stage's previous tenant has been consumed
                    __nv_bfloat16* sK = stages + stage * T::STAGE_ELEMS;
                    __nv_bfloat16* sV = sK + BNW * STRIDE;
                    const int j0 = key_base + i * BNW + lane * run_rows;
                    size_t src = 0;
                    bool want = lane < runs && j0 <= pos && j0 + run_rows > lo;   // the run holds a visible key
                    if (want) {
                        const int pi = dp.page_shift >= 0 ? (j0 >> dp.page_shift) : (j0 / ps);
                        const int page = pages_in_smem ? s_pages[pi - page_first] : table[pi];
                        if (page < 0 || page >= p.num_pages) {
                            want = false;                   // never read outside the pool; the step is reported as bad
                            if (p.status) atomicExch(p.status, 6);
                        } else {
                            src = (((size_t)page * p.n_kv_heads + kvh) * ps + (j0 - pi * ps)) * d;
                        }
                    }
                    const unsigned n_want = __popc(__ballot_sync(0xffffffffu, want));
                    if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], n_want * run_bytes * 2);
                    __syncwarp();
                    if (want) {
                        bulk_copy_g2s(sK + lane * run_rows * d, p.k_pages + src, run_bytes, &full_bar[stage]);
                        bulk_copy_g2s(sV + lane * run_rows * d, p.v_pages + src, run_bytes, &full_bar[stage]);
                    }
                }
                if (!ok && lane == 0 && p.status) atomicExch(p.status, 7);
            }
        } else if (warp >= 4) {
            // ---------------- loaders: thread lt copies 16-byte chunk `ch` of rows row0, row0 + rows_per_pass, ... ----------------
            const int lt = threadIdx.x - DEC_LOADERS;
            const int rows_per_pass = DEC_LOADERS / chunks;
            const int row0 = lt / chunks, ch = lt - row0 * chunks;
            const bool copier = row0 < rows_per_pass;
            const size_t head_elems = (size_t)ps * d;        // one head's run of a page
            bool ok = true;
#pragma unroll 1
            for (int i = 0; i < n_tiles; ++i) {
                const int stage = i % S;
                if (holds_newest && i == n_tiles - 1) pb_grid_dep_wait();
                ok = mbar_wait_bounded(&empty_bar[stage], ((i / S) & 1) ^ 1);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                if (lt == 0) *(volatile int*)&s_issued = i + 1;             // the stage's previous tenant has been consumed
                __nv_bfloat16* sK = stages + stage * T::STAGE_ELEMS;
                __nv_bfloat16* sV = sK + BNW * STRIDE;
                if (copier) {
                    for (int row = row0; row < BNW; row += rows_per_pass) {
                        const int j = key_base + i * BNW + row;
                        bool valid = j >= lo && j < kv_end;
                        size_t src = 0;
                        if (valid) {
                            const int pi = dp.page_shift >= 0 ? (j >> dp.page_shift) : (j / ps);
                            const int page = pages_in_smem ? s_pages[pi - page_first] : table[pi];
                            if (page < 0 || page >= p.num_pages) {
                                valid = false;              // never read outside the pool; the step is reported as bad
                                if (p.status) atomicExch(p.status, 6);
                            } else {
                                const int in_page = j - pi * ps;
                                src = ((size_t)page * p.n_kv_heads + kvh) * head_elems + (size_t)in_page * d +
                                      ((p.swizzle ? (ch ^ (in_page & 7)) : ch) << 3);
                            }
                        }
                        cp_async16(sK + row * STRIDE + ch * 8, p.k_pages + src, valid);   // rows without a key are zero-filled
                        cp_async16(sV + row * STRIDE + ch * 8, p.v_pages + src, valid);
                    }
                }
                cp_async_arrive_on(&full_bar[stage]);
            }
            if (!ok && lane == 0 && p.status) atomicExch(p.status, 7);
            cp_async_wait<0>();                             // nothing of this thread is in flight when shared memory changes its use
        } else {
            // ---------------- consumers: warp w takes tiles w, w + NC, ... ----------------
            FragOffsets<DMAX, BULK> frag;
            attn_frag_offsets<DMAX, BULK>(frag, 0, lane);
            const unsigned sQ_a = smem_u32(sQ);
            const int row_pos[2] = {pos, pos};              // every row of the tile is a head of the one new token
#pragma unroll 1
            for (int i = warp; warp < NC && i < n_tiles; i += NC) {
                const int stage = i % S;
                bool landed = true;
                if (*(volatile int*)&s_issued <= i) {       // not announced yet: the barrier may still be in an older phase
                    const long long t0 = clock64();
                    while (*(volatile int*)&s_issued <= i)
                        if (clock64() - t0 > (1ll << 31)) { landed = false; break; }
                }
                landed = landed && mbar_wait_bounded(&full_bar[stage], (i / S) & 1);
                if (!__all_sync(0xffffffffu, landed)) {     // gave up waiting: report, do not hang
                    if (lane == 0 && p.status) atomicExch(p.status, 7);
                    break;
                }
                const __nv_bfloat16* sK = stages + stage * T::STAGE_ELEMS;
                const __nv_bfloat16* sV = sK + BNW * STRIDE;
                const int key0 = key_base + i * BNW;
                const bool edge = key0 < lo || key0 + BNW - 1 > pos;         // some key of the tile is not visible
                if (BULK && edge) {
                    // value rows that no visible key stands for hold whatever the page (or the stage) held:
                    // zeros instead, so that 0 * (whatever is there) cannot make a NaN
                    for (int r = lane; r < BNW; r += 32) {
                        const int j = key0 + r;
                        if (j < lo || j > pos)
                            for (int c = 0; c < (d >> 3); ++c)
                                *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(sV) + r * row_elems + c * 8) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();                    // these ordinary stores come before the bulk copy that refills the stage
                    __syncwarp();
                }
                attn_tile<DMAX, BULK>(o, m, l, frag, sQ_a, smem_u32(sK), smem_u32(sV), d, key0, row_pos, edge, p.window,
                                      p.scale_log2, t4);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[stage]);               // the stage may be refilled
            }
        }
        __syncthreads();                                    // all warps are done with the tile buffers
    }
    pb_grid_dep_wait();                                     // blocks without keys come here directly
    // merge the four warps through shared memory (the tile buffers are free now)
    float* sO = reinterpret_cast<float*>(stages);           // [4][16][DMAX]
    float* sM = sO + 4 * 16 * DMAX;                         // [4][16]
    float* sL = sM + 64;
    float* sC = sL + 64 + 2 * 16 * 64 + 16;                 // [16][DMAX] this block's part, for the cluster's other blocks
    float* sCml = sC + 16 * DMAX;                           // [16][2] its maxima and sums
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        if (warp >= 4) continue;                            // the loader warps hold no partial result
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
    for (int idx = threadIdx.x; idx < G * d; idx += DEC_THREADS) {
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
        } else if (dp.cluster) {
            sC[idx] = acc;                                  // this block's part stays in its shared memory
            if (col == 0) { sCml[row * 2] = mm; sCml[row * 2 + 1] = ls; }
        } else {
            p.part_o[(th * p.n_splits + split) * d + col] = acc;
            if (col == 0) {
                p.part_ml[(th * p.n_splits + split) * 2] = mm;
                p.part_ml[(th * p.n_splits + split) * 2 + 1] = ls;
            }
        }
    }
    PB_TL(PB_TL_ATTN_DECODE, PB_TL_DONE);
    if (p.n_splits == 1) return;
    if (dp.cluster) {
        // The cluster is the (token, key/value head)'s splits, in order: block rank = split.  After the barrier every
        // block's part is in place; block r adds up the r-th slice of the output elements over all parts, in
        // ascending order, and the second barrier keeps every block's shared memory alive until all have read it.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int ns = p.n_splits, rank = (int)cluster.block_rank();
        const int per = (G * d + ns - 1) / ns;
        const size_t th0 = (size_t)tok * p.n_heads + kvh * G;
        for (int idx = rank * per + threadIdx.x; idx < min(G * d, (rank + 1) * per); idx += DEC_THREADS) {
            const int row = idx / d;
            float ms[16], lsum[16], part[16];
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 16; ++sp) {
                if (sp < ns) {
                    const float* rml = cluster.map_shared_rank(sCml, sp);
                    ms[sp] = rml[row * 2];
                    lsum[sp] = rml[row * 2 + 1];
                    part[sp] = cluster.map_shared_rank(sC, sp)[idx];
                    mm = fmaxf(mm, ms[sp]);
                }
            }
            float acc = 0.f, ls = 0.f;
#pragma unroll
            for (int sp = 0; sp < 16; ++sp) {
                if (sp < ns) {
                    const float f = (ms[sp] == -INFINITY) ? 0.f : exp2f(ms[sp] - mm);
                    ls += f * lsum[sp];
                    acc += f * part[sp];
                }
            }
            p.out[th0 * d + idx] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
        }
        cluster.sync();
        PB_TL(PB_TL_ATTN_DECODE, PB_TL_EXIT);
        return;
    }
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
    const int ns = p.n_splits;
    const size_t th0 = (size_t)tok * p.n_heads + kvh * G;
    if (ns <= 64) {
        // Every load below is issued before its value is needed, so the merge costs a few trips to the L2 cache and
        // not one per split.  Maximum and sum of every split into shared memory; one warp per row turns them into
        // the weight of each split; then every output element adds its splits up in ascending order.
        float* sMs = sL + 64;                               // [G][64] maxima, then [G][64] sums, then [G] 1 / total
        float* sLs = sMs + 16 * 64;
        float* sInv = sLs + 16 * 64;
        for (int idx = threadIdx.x; idx < G * ns; idx += DEC_THREADS) {
            const int row = idx / ns, sp = idx - row * ns;
            const float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((th0 + row) * ns + sp) * 2));
            sMs[row * 64 + sp] = v.x;
            sLs[row * 64 + sp] = v.y;
        }
        __syncthreads();
        for (int row = warp; row < G; row += DEC_THREADS / 32) {
            float mm = -INFINITY;
            for (int sp = lane; sp < ns; sp += 32) mm = fmaxf(mm, sMs[row * 64 + sp]);
            mm = pb_warp_max(mm);
            // the sum over the splits in ascending order, by one lane: the splits are few
            float ls = 0.f;
            for (int sp = lane; sp < ns; sp += 32) {
                const float ms = sMs[row * 64 + sp];
                sMs[row * 64 + sp] = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);   // the split's weight
            }
            __syncwarp();
            if (lane == 0) {
                for (int sp = 0; sp < ns; ++sp) ls += sMs[row * 64 + sp] * sLs[row * 64 + sp];
                sInv[row] = ls > 0.f ? 1.0f / ls : 0.f;
            }
        }
        __syncthreads();
        // two output elements per thread and pass, their loads (up to 8 splits each) issued together
        for (int idx0 = threadIdx.x; idx0 < G * d; idx0 += 2 * DEC_THREADS) {
            float acc[2] = {0.f, 0.f};
            for (int s0 = 0; s0 < ns; s0 += 8) {
                float v[2][8];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int idx = idx0 + e * DEC_THREADS;
                    const int row = idx / d, col = idx - row * d;
                    const float* po = p.part_o + (th0 + row) * ns * d + col;
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[e][u] = (idx < G * d && s0 + u < ns) ? __ldcg(po + (size_t)(s0 + u) * d) : 0.f;
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int idx = idx0 + e * DEC_THREADS;
                    if (idx < G * d) {
                        const int row = idx / d;
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (s0 + u < ns) acc[e] += sMs[row * 64 + s0 + u] * v[e][u];
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int idx = idx0 + e * DEC_THREADS;
                if (idx < G * d) {
                    const int row = idx / d, col = idx - row * d;
                    p.out[(th0 + row) * d + col] = __float2bfloat16_rn(acc[e] * sInv[row]);
                }
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < G * d; idx += DEC_THREADS) {
        const int row = idx / d, col = idx - row * d;
        const size_t th = th0 + row;
        const float* ml = p.part_ml + th * ns * 2;
        float mm = -INFINITY;
        for (int s = 0; s < ns; ++s) mm = fmaxf(mm, __ldcg(ml + 2 * s));
        float acc = 0.f, ls = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = __ldcg(ml + 2 * s);
            const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
            ls += f * __ldcg(ml + 2 * s + 1);
            acc += f * __ldcg(p.part_o + (th * ns + s) * d + col);
        }
        p.out[th * d + col] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
    }
}

template <int DMAX, bool BULK, bool PAIR> static size_t decode_smem() {
    using T = DecodeTiling<DMAX, BULK, PAIR>;
    size_t tiles = (size_t)T::STAGES * T::STAGE_ELEMS * 2 + (size_t)16 * (DMAX + 8) * 2 + DEC_MAX_PAGES * 4;
    // the warps' partial results, the splits' maxima and sums, this block's part for its cluster
    size_t merge = (size_t)(4 * 16 * DMAX + 128 + 2 * 16 * 64 + 16 + 16 * DMAX + 32) * 4;
    return tiles > merge ? tiles : merge;
}

template <int DMAX, bool BULK, bool PAIR> static int decode_configure() {
    static bool configured = false;
    size_t smem = decode_smem<DMAX, BULK, PAIR>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<DMAX, BULK, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("attention_decode: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    return 0;
}

// How many clusters of `ns` blocks of this kernel the device holds at a time (0: it cannot place one); asked once per size.
template <int DMAX, bool BULK, bool PAIR> static int decode_clusters_resident(int ns) {
    using T = DecodeTiling<DMAX, BULK, PAIR>;
    static int known[DEC_MAX_CLUSTER + 1];
    static bool asked[DEC_MAX_CLUSTER + 1] = {false};
    if (ns < 2 || ns > DEC_MAX_CLUSTER) return 0;
    if (!asked[ns]) {
        asked[ns] = true;
        known[ns] = 0;
        if (decode_configure<DMAX, BULK, PAIR>() != 0) return 0;
        cudaError_t e = cudaSuccess;
        if (ns > 8) e = cudaFuncSetAttribute(attn_decode_kernel<DMAX, BULK, PAIR>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(ns * 4096, 1, 1);
            cfg.blockDim = dim3(T::THREADS);
            cfg.dynamicSmemBytes = decode_smem<DMAX, BULK, PAIR>();
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = ns; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            e = cudaOccupancyMaxActiveClusters(&n, attn_decode_kernel<DMAX, BULK, PAIR>, &cfg);
            if (e == cudaSuccess && n > 0) known[ns] = n;
        }
        (void)cudaGetLastError();
    }
    return known[ns];
}

template <int DMAX, bool BULK, bool PAIR>
static int launch_decode(const DecodeParams& dp, cudaStream_t stream) {
    using T = DecodeTiling<DMAX, BULK, PAIR>;
    size_t smem = decode_smem<DMAX, BULK, PAIR>();
    if (int e = decode_configure<DMAX, BULK, PAIR>()) return e;
    const dim3 grid(dp.a.n_splits, dp.a.n_kv_heads, dp.a.n_tokens);
    DecodeParams q = dp;
    const int ns = dp.a.n_splits;
    q.cluster = (dp.cluster && decode_clusters_resident<DMAX, BULK, PAIR>(ns) > 0) ? 1 : 0;
    if (q.cluster) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(T::THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = ns; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pb_pdl_enabled() ? 2 : 1;
        cudaLaunchKernelEx(&cfg, attn_decode_kernel<DMAX, BULK, PAIR>, q);
    } else {
        pb_launch(attn_decode_kernel<DMAX, BULK, PAIR>, grid, dim3(T::THREADS), smem, stream, q);
    }
    return 0;
}

static int g_dec_sms = 0;
static int dec_sms() {
    if (g_dec_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_dec_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_dec_sms <= 0) g_dec_sms = 148;
    }
    return g_dec_sms;
}

// Blocks of this kernel that one multiprocessor holds at a time when every (token, head) pair can have a
// multiprocessor of its own (for choosing the number of splits).
PB_API int pb_attention_decode_blocks_per_sm(int head_dim) {
    size_t smem = head_dim <= 64 ? decode_smem<64, false, false>() : head_dim <= 128 ? decode_smem<128, false, false>() : decode_smem<256, false, false>();
    int n = (int)((227 * 1024) / (smem + 1024));
    return n < 1 ? 1 : n;
}

// Whether the splits of a (token, key/value head) are launched as a thread-block cluster: yes unless
// PRELUDE_DECODE_CLUSTER=0 or pb_attention_decode_set_cluster(0) says otherwise.
static int g_dec_clusters = -1;
static int dec_use_clusters() {
    if (g_dec_clusters < 0) {
        const char* off = getenv("PRELUDE_DECODE_CLUSTER");
        g_dec_clusters = (off && off[0] == '0') ? 0 : 1;
    }
    return g_dec_clusters;
}
PB_API void pb_attention_decode_set_cluster(int on) { g_dec_clusters = on ? 1 : 0; }

// The most splits whose blocks can add their parts up as one thread-block cluster (more go through scratch memory).
PB_API int pb_attention_decode_cluster_max() { return dec_use_clusters() ? DEC_MAX_CLUSTER : 0; }

// Scratch floats a call needs for its splits: (head_dim + 2) per token, head and split.
PB_API long long pb_attention_decode_scratch_floats(int n_tokens, int n_heads, int head_dim, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_tokens * n_heads * n_splits * (head_dim + 2);
}

static bool dec_bulk(int head_dim, int page_size, int swizzle) {
    // bulk copies bring whole runs of a page: a run must tile the 64-key tile evenly and start at a multiple
    // of 8 tokens (the rows then sit at the row numbers their permutation was made for)
    return swizzle && page_size % 8 == 0 && (BNW % page_size == 0 || page_size % BNW == 0) &&
           (head_dim == 64 || head_dim == 128 || head_dim == 256);    // the dense layout has no room for a narrower head
}

// Into how many parts a decode step cuts the keys of every (token, key/value head), for contexts of up to
// max_context keys, and whether the parts are added up inside a thread-block cluster (the return value is the
// count, plus 256 when they are).  Every candidate is rated by what its busiest multiprocessor has to stream, in
// 64-key tiles, plus what adding the parts up costs (measured on B200: about three tiles' time inside a cluster,
// about seven through scratch memory, a tile taking 0.6 us).  Candidates: no cut; 2 to 8 parts as a cluster, but
// only where the device holds the clusters of all pairs at one time (a cluster needs its blocks on one processor
// group, and a second round of clusters would wait for the first; the driver says how many fit); and, through
// scratch memory, as many parts as the device holds blocks at a time (never more than there are tiles, or 64).
PB_API int pb_attention_decode_plan(int n_tokens, int n_kv_heads, int head_dim, int page_size, int swizzle, int max_context) {
    const int sms = dec_sms();
    const long long pairs = (long long)(n_tokens < 1 ? 1 : n_tokens) * (n_kv_heads < 1 ? 1 : n_kv_heads);
    const int tiles = max_context < 1 ? 1 : (max_context + 63) / 64;
    const bool bulk = dec_bulk(head_dim, page_size, swizzle);
    const int dmax = head_dim <= 64 ? 64 : head_dim <= 128 ? 128 : 256;
    long long most = (long long)sms * pb_attention_decode_blocks_per_sm(head_dim) / pairs;
    if (most > tiles) most = tiles;
    if (most > 64) most = 64;
    if (most < 1) most = 1;
    if (pairs > 65536) return 1;
    auto load = [&](long long s) { return (double)((pairs * s + sms - 1) / sms) * ((double)tiles / (double)s); };
    int best = 1;
    double best_cost = load(1);
    if (most > 1 && load(most) + 7.0 < best_cost) { best = (int)most; best_cost = load(most) + 7.0; }
    if (dec_use_clusters()) {
        for (int s = 2; s <= 8 && s <= tiles; ++s) {
            const bool pair = bulk && head_dim <= 128 && pairs * s > sms;
            int held = 0;
            if (dmax == 64) held = bulk ? (pair ? decode_clusters_resident<64, true, true>(s) : decode_clusters_resident<64, true, false>(s))
                                        : decode_clusters_resident<64, false, false>(s);
            else if (dmax == 128) held = bulk ? (pair ? decode_clusters_resident<128, true, true>(s) : decode_clusters_resident<128, true, false>(s))
                                              : decode_clusters_resident<128, false, false>(s);
            else held = bulk ? decode_clusters_resident<256, true, false>(s) : decode_clusters_resident<256, false, false>(s);
            if (held < pairs) continue;
            const double cost = load(s) + 3.0;
            if (cost <= best_cost) { best = s | 256; best_cost = cost; }
        }
    }
    return best;
}

// cluster: add the splits' parts up inside a thread-block cluster where the device can place one of n_splits blocks
// (up to 16), else through scratch memory.
// scratch: pb_attention_decode_scratch_floats(...) floats, or null when n_splits == 1.
// counters: n_tokens * n_kv_heads ints, zero before the first call; every call leaves them
// zero, so calls that follow one another on a stream may share them.  Null when n_splits == 1.
PB_API int pb_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                    const int32_t* block_table, int table_stride, const int32_t* positions,
                                    const int32_t* token_seq, int page_size, int num_pages, int n_tokens,
                                    int n_heads, int n_kv_heads, int head_dim, float scale, int window, int swizzle,
                                    int n_splits, int cluster, float* scratch, int* counters, int* status, cudaStream_t stream) {
    DecodeParams dp{};
    AttnParams& p = dp.a;
    p.q = (const __nv_bfloat16*)q; p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions; p.token_seq = token_seq;
    p.n_splits = n_splits; p.table_stride = table_stride; p.page_size = page_size; p.num_pages = num_pages;
    p.n_tokens = n_tokens; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.swizzle = swizzle;
    if (int e = attn_check_common("attention_decode", p)) return e;
    PB_REQUIRE(!swizzle || head_dim % 64 == 0, "attention_decode: permuted pages need head_dim %% 64 == 0");
    p.group = n_heads / n_kv_heads;
    PB_REQUIRE(p.group <= 16, "attention_decode: %d query heads per key/value head; at most 16 fit a tile", p.group);
    PB_REQUIRE(n_splits >= 1 && n_splits <= 1024, "attention_decode: n_splits=%d", n_splits);
    PB_REQUIRE(n_tokens < 65536 && n_kv_heads < 65536, "attention_decode: bad grid");
    dp.cluster = (cluster && dec_use_clusters() && n_splits > 1 && n_splits <= DEC_MAX_CLUSTER) ? 1 : 0;
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
    const bool bulk = dec_bulk(head_dim, page_size, swizzle);
    // more blocks than multiprocessors: two per multiprocessor with half the ring each
    const bool pair = bulk && head_dim <= 128 && (long long)n_tokens * n_kv_heads * n_splits > dec_sms();
    int e = pair ? (head_dim == 64 ? launch_decode<64, true, true>(dp, stream) : launch_decode<128, true, true>(dp, stream))
          : bulk ? (head_dim == 64 ? launch_decode<64, true, false>(dp, stream)
                    : head_dim == 128 ? launch_decode<128, true, false>(dp, stream) : launch_decode<256, true, false>(dp, stream))
                 : (head_dim <= 64 ? launch_decode<64, false, false>(dp, stream)
                    : head_dim <= 128 ? launch_decode<128, false, false>(dp, stream) : launch_decode<256, false, false>(dp, stream));
    if (e) return e;
    PB_CHECK_LAUNCH("attention_decode");
    return 0;
}

