// A chain of products for the few rows of a decode step, in ONE launch:
//     y1 = f1(x W1^T),  y2 = f2(y1 W2^T),  ...        (M <= 16 rows, bfloat16, float32 accumulation)
// as a feed-forward needs them: silu(gate) * up of the merged gate/up projection, then the down projection.
//
// Each of these products alone is a stream over its weight matrix (gemm_stream.cu).  Launched one after the other,
// every product pays for the memory system standing still twice: while its last stages are being worked on and
// its blocks leave, and while the next kernel's blocks arrive and fill their rings.  Here the blocks stay, and the
// loader warps never stop: the weights of the next product follow the last rows of this one through the same ring
// of shared-memory stages, while the compute warps finish the product, meet the other blocks at a barrier in
// global memory (the next product reads what all blocks have written) and fetch their rows of the new input.
//
//  * One block per multiprocessor, every block resident (the launch asks for no more blocks than the device has
//    multiprocessors, one fits on each; a block that still waits at the barrier after about a second raises the
//    status word and all go on to their end, so a device that does not hold them all shows as an error).
//  * A product ("phase") gives every block a run of output features and, where K is cut into parts, one part of
//    K: phase q uses blocks_x * splits blocks, block b -> (b % blocks_x, b / blocks_x); the others only join the
//    barriers.
//  * The ring's stages have one size for all phases (8 rows of the longest chunk of K); a phase cuts its rows into
//    chunks that fit.  Stage numbers, barrier phases and the count of issued stages run on across the phases, so
//    loaders and compute warps need no agreement beyond walking the same loops.
//  * x of a phase after the first has been written by other blocks of this launch: it is fetched, like the first
//    phase's, with one bulk copy per row, after the barrier and a fence between the two ways to memory.
//
// The reference has no counterpart (its decode step launches one library product per projection,
// crates/prelude-cuda/src/ops/gemm.rs:35-137).
#include "attention_common.cuh"

#define GC_WARPS 8                              // compute warps
#define GC_LOADERS 4                            // loader warps; each issues GC_ROWS / GC_LOADERS copies per stage
#define GC_THREADS ((GC_WARPS + GC_LOADERS) * 32)
#define GC_ROWS 8                               // features per stage; a tile of the product is two stages
#define GC_MAX_STAGES 8
#define GC_CHAINS 4                             // independent accumulators per warp
#define GC_SMEM_LIMIT (227 * 1024 - 2048)
#define GC_MAX_PHASES 4
#define GC_MAX_GROUPS 16                        // groups of blocks at one barrier
#define GC_COUNTERS (GC_MAX_PHASES * GC_MAX_GROUPS + 1)

struct GcPhase {
    const __nv_bfloat16* W;     // [N, ldw] (gated: N gate rows, then N up rows)
    const __nv_bfloat16* X;     // [M, ldx], K * splits columns
    void* out;                  // kind 0: bfloat16 [M, ldo]; kind 1: float32 [splits][M, ldo], split_stride apart
    long long ldw, ldx, ldo, split_stride;
    int N;                      // output features
    int K;                      // columns of one part of K
    int splits;                 // parts of K
    int blocks_x;               // blocks along the features
    int ks, n_chunks;           // elements of K per stage, chunks per row of a part
    int gated;                  // the output is silu(gate) * up
    int kind;                   // 0: bfloat16 result; 1: float32 partial sums, one set per part of K
    int groups;                 // the barrier before this phase: groups of blocks that wait for one another only
};

struct GcParams {
    GcPhase ph[GC_MAX_PHASES];
    int n_phases;
    int M;
    int stages;                 // stages of the ring
    int slot_bytes;             // bytes of one stage
    int x_bytes;                // bytes kept for x (the largest phase's)
    unsigned* gbar;             // [GC_COUNTERS] zero on entry and on exit: arrivals per (barrier, group), blocks that have left
    int* status;
};

__device__ __forceinline__ void gc_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void gc_bar_compute() { asm volatile("bar.sync 1, %0;\n" ::"n"(GC_WARPS * 32) : "memory"); }
__device__ __forceinline__ void gc_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void gc_ldmatrix_x2(unsigned& r0, unsigned& r1, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ unsigned gc_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The run of features and the part of K that this block has in a phase.
struct GcShare {
    int r0, r1, by;
    bool active;
};
__device__ __forceinline__ GcShare gc_share(const GcPhase& f) {
    GcShare s;
    const int b = blockIdx.x;
    s.active = b < f.blocks_x * f.splits;
    const int bx = s.active ? b % f.blocks_x : 0;
    s.by = s.active ? b / f.blocks_x : 0;
    s.r0 = (int)((long long)bx * f.N / f.blocks_x);
    s.r1 = (int)((long long)(bx + 1) * f.N / f.blocks_x);
    return s;
}

// MT: 8-row tiles of x (M <= 8 * MT)
template <int MT>
__global__ void __launch_bounds__(GC_THREADS, 1) gemm_chain_kernel(const __grid_constant__ GcParams p) {
    pb_grid_dep_launch();
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full_bar[GC_MAX_STAGES], empty_bar[GC_MAX_STAGES], x_bar;
    __shared__ int s_issued, s_dead;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* sX = smem;                                  // [M] rows of the current phase's x
    unsigned char* ring = sX + p.x_bytes;
    float* red = reinterpret_cast<float*>(ring + (size_t)p.stages * p.slot_bytes);   // [GC_WARPS][8 MT batch rows][16 features]

    if (threadIdx.x == 0) {
        s_issued = 0;
        s_dead = 0;
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], GC_LOADERS); mbar_init(&empty_bar[s], GC_WARPS); }
        mbar_init(&x_bar, GC_LOADERS);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp >= GC_WARPS) {
        // ---------------- loaders: warp j copies rows 2 j and 2 j + 1 of every stage (lanes 0 and 1) ----------------
        // Weights are written by no kernel: the loaders wait for nobody but the ring, through all phases.
        const int lw = warp - GC_WARPS;
        constexpr int PER = GC_ROWS / GC_LOADERS;
        bool ok = true;
        int stage = 0, phase = 0, i = 0;
#pragma unroll 1
        for (int q = 0; q < p.n_phases && ok; ++q) {
            const GcPhase& f = p.ph[q];
            const GcShare sh = gc_share(f);
            if (!sh.active) continue;
            const int span = f.gated ? GC_ROWS : 16;           // features per tile
            const int n_tiles = (sh.r1 - sh.r0 + span - 1) / span;
            const int w_stride = f.ks * 2 + 16;                // bytes between rows of a stage
            const __nv_bfloat16* W = f.W + (size_t)sh.by * f.K;
#pragma unroll 1
            for (int tile = 0; tile < n_tiles && ok; ++tile) {
                const int halves = (f.gated || sh.r1 - (sh.r0 + tile * span) > GC_ROWS) ? 2 : 1;
#pragma unroll 1
                for (int kc = 0; kc < f.n_chunks && ok; ++kc) {
                    for (int h = 0; h < halves; ++h, ++i) {
                        if (i >= p.stages) {                   // the first ring-full finds every stage free
                            ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1);
                            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                        }
                        if (lw == 0 && lane == 0) *(volatile int*)&s_issued = i + 1;   // the stage's previous tenant has been consumed
                        const int feat0 = sh.r0 + tile * span + (f.gated ? 0 : h * GC_ROWS);   // first feature of the stage
                        const int row0 = feat0 + (f.gated ? h * f.N : 0);                    // its row of W: up rows follow the gate rows
                        const int k0 = kc * f.ks, len = min(f.ks, f.K - k0);
                        const int n_rows = min(GC_ROWS, sh.r1 - feat0);
                        const int mine = min(PER, max(0, n_rows - lw * PER));             // rows of this stage that this warp brings
                        // the copies may land before the expected bytes are posted: the phase cannot end before this arrival
                        if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], (unsigned)mine * len * 2);
                        const int rr = lw * PER + lane;
                        if (lane < mine)
                            bulk_copy_g2s(ring + (size_t)stage * p.slot_bytes + (size_t)rr * w_stride,
                                          W + (size_t)(row0 + rr) * f.ldw + k0, (unsigned)len * 2, &full_bar[stage]);
                        if (++stage == p.stages) { stage = 0; phase ^= 1; }
                    }
                }
            }
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 11);
        return;
    }

    // ---------------- compute warps ----------------
    const int g = lane >> 2, t4 = lane & 3;
    const unsigned sX_a = smem_u32(sX), ring_a = smem_u32(ring);
    int stage = 0, phase = 0, item = 0;
    unsigned x_phase = 0;
#pragma unroll 1
    for (int q = 0; q < p.n_phases; ++q) {
        const GcPhase& f = p.ph[q];
        const GcShare sh = gc_share(f);
        if (q == 0) {
            pb_grid_dep_wait();                                // x of the first phase comes from the kernel before
        } else {
            // every block has written its share of the phase before.  The block's threads meet; one of them makes
            // their stores visible to the device (a fence after the meeting covers them all), counts the block in
            // and waits for the others.  Where the blocks that produce a part of x are the ones that consume it
            // (f.groups > 1), a block waits for its own group only.
            gc_bar_compute();
            if (threadIdx.x == 0) {
                const unsigned per_group = gridDim.x / (unsigned)f.groups;
                unsigned* counter = p.gbar + (q - 1) * GC_MAX_GROUPS + blockIdx.x / per_group;
                __threadfence();
                atomicAdd(counter, 1u);
                const long long t0 = clock64();
                while (gc_ld_acquire(counter) < per_group) {
                    if (clock64() - t0 > (1ll << 31)) {        // about a second: some block is not running
                        *(volatile int*)&s_dead = 1;
                        if (p.status) atomicExch(p.status, 13);
                        break;
                    }
                }
                __threadfence();
            }
            gc_bar_compute();
        }
        if (!sh.active || *(volatile int*)&s_dead) continue;

        // this block's rows of x, its part of K: one bulk copy per row, issued by the first four compute warps
        // (warp j brings rows j, j + 4, ...).  After the first phase other blocks of this launch have written x with
        // ordinary stores, which the barrier has made visible; the copy engine reads through another path, hence
        // the fence before the copies.
        const int x_stride = f.K * 2 + 16;                     // bytes between rows of x in shared memory
        if (warp < GC_LOADERS) {
            const int mine = (p.M - warp + GC_LOADERS - 1) / GC_LOADERS;
            if (lane == 0) mbar_arrive_expect_tx(&x_bar, (unsigned)max(mine, 0) * f.K * 2);
            const int m = warp + lane * GC_LOADERS;
            if (m < p.M) {
                if (q > 0) asm volatile("fence.proxy.async.global;\n" ::: "memory");
                bulk_copy_g2s(sX + (size_t)m * x_stride, f.X + (size_t)m * f.ldx + (size_t)sh.by * f.K, (unsigned)f.K * 2, &x_bar);
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&x_bar, x_phase))) {
            if (lane == 0) { *(volatile int*)&s_dead = 1; if (p.status) atomicExch(p.status, 12); }
        }
        x_phase ^= 1;
        gc_bar_compute();
        if (*(volatile int*)&s_dead) continue;

        const int span = f.gated ? GC_ROWS : 16;
        const int n_tiles = (sh.r1 - sh.r0 + span - 1) / span;
        const int w_stride = f.ks * 2 + 16;
        // ldmatrix lanes.  W (row operand, 16 features x 16 k): lane -> feature lane & 15 (the first eight in one
        // stage, the others in the next), k half lane >> 4.  x (column operand): 8 batch rows x 16 k (x2), or
        // 16 batch rows (x4); rows that do not exist read the last row that does, and their sums are never stored.
        const unsigned a_off = (lane & 7) * w_stride + (lane >> 4) * 16;
        const bool upper = (lane & 8) != 0;                    // this lane addresses a row of the second stage
        const int x_row = (MT == 1) ? (lane & 7) : ((lane & 7) + (lane >> 4) * 8);
        const unsigned b_off = min(x_row, p.M - 1) * x_stride + ((lane >> 3) & 1) * 16;
        bool dead = false;
#pragma unroll 1
        for (int tile = 0; tile < n_tiles && !dead; ++tile) {
            const int halves = (f.gated || sh.r1 - (sh.r0 + tile * span) > GC_ROWS) ? 2 : 1;
            float acc[GC_CHAINS][MT][4];
#pragma unroll
            for (int c = 0; c < GC_CHAINS; ++c)
#pragma unroll
                for (int j = 0; j < MT; ++j) acc[c][j][0] = acc[c][j][1] = acc[c][j][2] = acc[c][j][3] = 0.f;
#pragma unroll 1
            for (int kc = 0; kc < f.n_chunks; ++kc) {
                const int stage2 = (stage + 1 == p.stages) ? 0 : stage + 1, phase2 = (stage + 1 == p.stages) ? phase ^ 1 : phase;
                const int last = item + halves - 1;
                bool landed = true;
                if (*(volatile int*)&s_issued <= last) {       // not announced yet: the barrier may still be in an older phase
                    const long long t0 = clock64();
                    while (*(volatile int*)&s_issued <= last)
                        if (clock64() - t0 > (1ll << 31)) { landed = false; break; }
                }
                landed = landed && mbar_wait_bounded(&full_bar[stage], phase);
                if (halves == 2) landed = landed && mbar_wait_bounded(&full_bar[stage2], phase2);
                if (!__all_sync(0xffffffffu, landed)) {
                    if (lane == 0) { *(volatile int*)&s_dead = 1; if (p.status) atomicExch(p.status, 12); }
                    dead = true;
                    break;
                }
                const int k0 = kc * f.ks, steps = min(f.ks, f.K - k0) >> 4;
                // with one stage only, the upper eight rows read the lower ones again (their sums are not stored)
                const unsigned a_base = ring_a + ((upper && halves == 2) ? stage2 : stage) * p.slot_bytes + a_off;
                const unsigned b_base = sX_a + b_off + k0 * 2;
#pragma unroll 1
                for (int s0 = warp; s0 < steps; s0 += GC_WARPS * GC_CHAINS) {
                    unsigned a[GC_CHAINS][4], b[GC_CHAINS][4];
#pragma unroll
                    for (int c = 0; c < GC_CHAINS; ++c) {
                        const int s = s0 + c * GC_WARPS;
                        if (s < steps) {
                            gc_ldmatrix_x4(a[c], a_base + s * 32);
                            if (MT == 1) gc_ldmatrix_x2(b[c][0], b[c][1], b_base + s * 32);
                            else gc_ldmatrix_x4(b[c], b_base + s * 32);
                        }
                    }
#pragma unroll
                    for (int c = 0; c < GC_CHAINS; ++c) {
                        if (s0 + c * GC_WARPS < steps) {
                            mma_bf16_free(acc[c][0], a[c], b[c][0], b[c][1]);
                            if (MT == 2) mma_bf16_free(acc[c][MT - 1], a[c], b[c][2], b[c][3]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {                               // this warp is done with the stages
                    gc_mbar_arrive(&empty_bar[stage]);
                    if (halves == 2) gc_mbar_arrive(&empty_bar[stage2]);
                }
                item += halves;
                for (int h = 0; h < halves; ++h)
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
            // add the eight warps' sums: acc[.][j][e] is feature g (+8 for e >= 2), batch row 8 j + 2 t4 + (e & 1)
            float* mine = red + (size_t)warp * 16 * 8 * MT;
#pragma unroll
            for (int j = 0; j < MT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = acc[0][j][e];
#pragma unroll
                    for (int c = 1; c < GC_CHAINS; ++c) v += acc[c][j][e];
                    mine[(8 * j + 2 * t4 + (e & 1)) * 16 + g + 8 * (e >> 1)] = v;
                }
            gc_bar_compute();
            if (*(volatile int*)&s_dead) { dead = true; break; }
            if (f.gated) {
                // rows 0..7 of the tile are the gate sums of 8 features, rows 8..15 the up sums of the same features
                for (int idx = threadIdx.x; idx < p.M * GC_ROWS; idx += GC_WARPS * 32) {
                    const int m = idx >> 3, rr = idx & 7;
                    const int n = sh.r0 + tile * GC_ROWS + rr;
                    if (n < sh.r1) {
                        float gsum = 0.f, usum = 0.f;
#pragma unroll
                        for (int w = 0; w < GC_WARPS; ++w) {
                            gsum += red[(size_t)w * 16 * 8 * MT + m * 16 + rr];
                            usum += red[(size_t)w * 16 * 8 * MT + m * 16 + rr + 8];
                        }
                        const float v = gsum / (1.0f + expf(-gsum)) * usum;
                        reinterpret_cast<__nv_bfloat16*>(f.out)[(size_t)m * f.ldo + n] = __float2bfloat16_rn(v);
                    }
                }
            } else {
                for (int idx = threadIdx.x; idx < p.M * 16; idx += GC_WARPS * 32) {
                    const int m = idx >> 4, rr = idx & 15;
                    const int n = sh.r0 + tile * 16 + rr;
                    if (n < sh.r1) {
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < GC_WARPS; ++w) v += red[(size_t)w * 16 * 8 * MT + idx];
                        if (f.kind == 1)
                            reinterpret_cast<float*>(f.out)[(size_t)sh.by * f.split_stride + (size_t)m * f.ldo + n] = v;
                        else
                            reinterpret_cast<__nv_bfloat16*>(f.out)[(size_t)m * f.ldo + n] = __float2bfloat16_rn(v);
                    }
                }
            }
            gc_bar_compute();                                  // the sums are read before the next tile overwrites them
        }
    }
    // the block that leaves last puts the counters back to zero for the next launch
    if (p.n_phases > 1 && threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.gbar + GC_COUNTERS - 1, 1u) == gridDim.x - 1) {
            for (int i = 0; i < GC_COUNTERS; ++i) p.gbar[i] = 0;
        }
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static int g_gc_sms = 0;
static int gc_sms() {
    if (g_gc_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_gc_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_gc_sms <= 0) g_gc_sms = 148;
    }
    return g_gc_sms;
}

static int gc_round16(int v) { return (v + 15) / 16 * 16; }

// One stage size for all phases: the longest chunks of K (the fewest copies) that leave room for three stages
// beside the largest x, or for two if three never fit.  Fills ks and n_chunks of every phase, the ring's shape
// and the shared memory needed; false when no shape fits.
static bool gc_plan(GcParams& p, size_t* smem) {
    size_t x_bytes = 0;
    for (int q = 0; q < p.n_phases; ++q) {
        const size_t b = (size_t)p.M * ((size_t)p.ph[q].K * 2 + 16);
        if (b > x_bytes) x_bytes = b;
    }
    const size_t red_bytes = (size_t)GC_WARPS * 16 * 16 * 4;
    if (x_bytes + red_bytes >= GC_SMEM_LIMIT) return false;
    const size_t room = GC_SMEM_LIMIT - x_bytes - red_bytes;
    for (int want = 3; want >= 2; --want) {
        // candidates for the longest chunk, longest first: a phase's K cut into n equal chunks
        int best = 0;
        for (int q = 0; q < p.n_phases; ++q)
            for (int n = 1; n <= 32; ++n) {
                const int cap = gc_round16((p.ph[q].K + n - 1) / n);
                if (cap < 512 && n > 1) break;                  // copies under 1 KB are not worth having
                if ((size_t)GC_ROWS * ((size_t)cap * 2 + 16) * want <= room && cap > best) best = cap;
            }
        if (best == 0) continue;
        int longest = 0;
        for (int q = 0; q < p.n_phases; ++q) {
            GcPhase& f = p.ph[q];
            const int n = (f.K + best - 1) / best;
            f.ks = gc_round16((f.K + n - 1) / n);
            f.n_chunks = (f.K + f.ks - 1) / f.ks;
            if (f.ks > longest) longest = f.ks;
        }
        p.slot_bytes = GC_ROWS * (longest * 2 + 16);
        size_t s = room / (size_t)p.slot_bytes;
        if (s > GC_MAX_STAGES) s = GC_MAX_STAGES;
        p.stages = (int)s;
        p.x_bytes = (int)x_bytes;
        *smem = x_bytes + red_bytes + s * (size_t)p.slot_bytes;
        return true;
    }
    return false;
}

static int gc_launch(GcParams& p, cudaStream_t stream) {
    PB_REQUIRE(p.n_phases >= 1 && p.n_phases <= GC_MAX_PHASES && p.M >= 1 && p.M <= 16, "gemm_chain: %d phases of %d rows", p.n_phases, p.M);
    const int grid = gc_sms();
    for (int q = 0; q < p.n_phases; ++q) {
        GcPhase& f = p.ph[q];
        PB_REQUIRE(f.W && f.X && f.out && pb_aligned(f.W, 16) && pb_aligned(f.X, 16), "gemm_chain: null or unaligned pointer in phase %d", q);
        PB_REQUIRE(f.N >= 1 && f.K >= 16 && f.K % 16 == 0 && f.ldw % 8 == 0 && f.ldx % 8 == 0 && f.splits >= 1 && f.splits <= grid,
                   "gemm_chain: phase %d: N=%d K=%d in %d parts (K %% 16 == 0 and 16-byte aligned rows are needed)", q, f.N, f.K, f.splits);
        PB_REQUIRE(!f.gated || (f.splits == 1 && f.kind == 0), "gemm_chain: the gated form has no cut of K and a bfloat16 result");
        PB_REQUIRE(f.splits == 1 || f.kind == 1, "gemm_chain: parts of K are float32 partial sums");
        int bx = grid / f.splits;
        if (bx > (f.N + 7) / 8) bx = (f.N + 7) / 8;           // at least 8 features per block
        f.blocks_x = bx < 1 ? 1 : bx;
        // The barrier before this phase.  When the phase before gave every block of the grid a run of its features,
        // this one cuts K into parts that are whole runs of those blocks, and every block works in both, then part g
        // of x is written by blocks [g * grid / splits, (g + 1) * grid / splits) and read by the same blocks
        // (block b works on part b / blocks_x): they wait for one another only.
        f.groups = 1;
        if (q > 0) {
            const GcPhase& a = p.ph[q - 1];
            // (the first block of group g starts at feature g * (grid / splits) * N / grid = g * K exactly)
            if (a.splits == 1 && a.blocks_x == grid && f.blocks_x * f.splits == grid && f.splits <= GC_MAX_GROUPS &&
                a.N == f.K * f.splits)
                f.groups = f.splits;
        }
    }
    PB_REQUIRE(p.n_phases == 1 || p.gbar != nullptr, "gemm_chain: more than one phase needs the barrier's counters");
    size_t smem = 0;
    PB_REQUIRE(gc_plan(p, &smem), "gemm_chain: x and two stages of the ring do not fit in shared memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, GC_SMEM_LIMIT);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_chain_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, GC_SMEM_LIMIT);
        if (e != cudaSuccess) return pb_fail("gemm_chain: cannot get %d bytes of shared memory: %s", GC_SMEM_LIMIT, cudaGetErrorString(e));
        configured = true;
    }
    if (p.M <= 8) pb_launch(gemm_chain_kernel<1>, dim3(grid), dim3(GC_THREADS), smem, stream, p);
    else pb_launch(gemm_chain_kernel<2>, dim3(grid), dim3(GC_THREADS), smem, stream, p);
    PB_CHECK_LAUNCH("gemm_chain");
    return 0;
}

static void gc_mlp_phases(GcParams& p, const void* X, long long ldx, const void* W_gate_up, long long ldw1, const void* W_down,
                          long long ldw2, void* act, void* parts, int M, int H, int I, int splits) {
    p = GcParams{};
    p.n_phases = 2;
    p.M = M;
    GcPhase& a = p.ph[0];
    a.W = (const __nv_bfloat16*)W_gate_up; a.ldw = ldw1; a.X = (const __nv_bfloat16*)X; a.ldx = ldx;
    a.out = act; a.ldo = I; a.N = I; a.K = H; a.splits = 1; a.gated = 1; a.kind = 0;
    GcPhase& b = p.ph[1];
    b.W = (const __nv_bfloat16*)W_down; b.ldw = ldw2; b.X = (const __nv_bfloat16*)act; b.ldx = I;
    b.out = parts; b.ldo = H; b.split_stride = (long long)M * H; b.N = H; b.K = I / splits; b.splits = splits; b.gated = 0; b.kind = 1;
}

// 32-bit counters that a chain's barriers need: zero before the first launch, left zero by every launch.
PB_API int pb_mlp_chain_counters() { return GC_COUNTERS; }

// Whether the chain takes a gated feed-forward of these sizes (else the caller launches the products one by one).
PB_API int pb_mlp_chain_supported(int M, int H, int I, int splits, long long ldx, long long ldw1, long long ldw2) {
    if (M < 1 || M > 16 || H < 16 || H % 16 || I < 16 || splits < 1 || I % (16 * splits) || ldx % 8 || ldw1 % 8 || ldw2 % 8) return 0;
    GcParams p;
    gc_mlp_phases(p, nullptr, ldx, nullptr, ldw1, nullptr, ldw2, nullptr, nullptr, M, H, I, splits);
    size_t smem;
    return gc_plan(p, &smem) ? 1 : 0;
}

// A gated feed-forward for the few rows of a decode step in one launch:
//   act   [M, I] bfloat16 = silu(x Wg^T) * (x Wu^T)   with W_gate_up [2 I, ldw1] (I gate rows, then I up rows)
//   parts [splits][M, H] float32: part s = act[:, s-th part of I] W_down[:, s-th part of I]^T; their sum is the result.
// act is scratch that the caller provides.  gbar: zeroed 32-bit counters, left zeroed; calls that overlap on
// the device need counters of their own.  (pb_mlp_chain_counters() of them.)
PB_API int pb_mlp_chain_bf16(const void* X, long long ldx, const void* W_gate_up, long long ldw1, const void* W_down,
                             long long ldw2, void* act, float* parts, int M, int H, int I, int splits, unsigned* gbar,
                             int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_mlp_chain_supported(M, H, I, splits, ldx, ldw1, ldw2), "mlp_chain: M=%d H=%d I=%d in %d parts not taken", M, H, I, splits);
    PB_REQUIRE(act && parts && gbar && pb_aligned(act, 16), "mlp_chain: null or unaligned scratch");
    GcParams p;
    gc_mlp_phases(p, X, ldx, W_gate_up, ldw1, W_down, ldw2, act, parts, M, H, I, splits);
    p.gbar = gbar;
    p.status = status;
    return gc_launch(p, stream);
}
