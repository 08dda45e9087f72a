// y[M, N] = x[M, K] * W[N, K]^T (+ bias) for the few rows of a decode step
// (M <= 16), bfloat16 in, float32 accumulation, bfloat16 or float32 out.
//
// With so few rows the product is a stream over the weight matrix: every byte
// of W is read once and the time is W's bytes over the memory bandwidth, plus
// whatever the kernel adds before the first byte and after the last.  The
// kernel is built to add little:
//  * Every block owns a contiguous run of output features (N / blocks of them,
//    give or take one) and the whole of K for them: no block waits for another,
//    and nothing is summed across blocks afterwards.
//  * Four loader warps stream the block's rows of W through a ring of
//    shared-memory stages (8 rows x one chunk of K per stage, one bulk copy per
//    row, full and empty barriers); the compute warps take the stages two at a
//    time.  Issuing a bulk copy costs a warp about 60 cycles whatever its size,
//    and warps issue side by side (measured), so every loader warp issues two of
//    a stage's eight copies, and the chunks are as long as shared memory allows:
//    a whole row where it fits.  Weights are written by no kernel, so the
//    loaders fill the ring before they wait for the kernel before this one on
//    the stream: the stream is already flowing when x becomes available.
//  * x (a few KB per row) is copied whole into shared memory by the compute warps
//    the moment that kernel is done.
//  * Eight compute warps share the 16-element steps of every pair of stages; W is
//    the row operand of mma.m16n8k16 (16 features: ldmatrix takes its 16 row
//    addresses from the two stages), x the column operand (8 batch rows per
//    instruction), both fetched from rows padded by 16 bytes; every warp keeps
//    four independent chains of sums.  When a 16-feature tile has seen all of K
//    the warps' sums are added through shared memory and stored.
//  * Where K is long and the output narrow (the down projection), x would crowd
//    the ring out of shared memory and every block would fetch all of it.  K can
//    then be cut into a few parts: the grid gets a second dimension, every part
//    works on its columns of W and x only and writes float32 partial sums of
//    its own, and whoever reads the output adds the parts (the residual add
//    does).  Nothing waits for anything.
//  * The gated form serves a feed-forward's merged gate and up projection: W
//    holds the N gate rows, then the N up rows; a tile is 8 features, its first
//    stage their gate rows and its second their up rows, so the two halves of
//    the tensor-core tile are gate and up of the same features and the
//    epilogue writes silu(gate) * up (float32 sums, one rounding) - the
//    activation costs no kernel and the 2N-wide intermediate never exists.
//  * Waits on barriers are bounded in time; a warp that gives up raises the
//    status word and the block goes on to its end.
// The reference leaves these shapes to its GEMM libraries
// (crates/prelude-cuda/src/ops/gemm.rs:35-137; DeepGEMM's small-M path).
// Needs K % 16 == 0, 16-byte aligned rows of W and x, and x to fit in shared
// memory beside the ring (pb_gemm_stream_supported says whether a shape is taken).
#include "attention_common.cuh"

PB_TIMELINE_UNIT(gemm_stream)

#define GS_WARPS 8                              // compute warps
#define GS_LOADERS 4                            // loader warps; each issues GS_ROWS / GS_LOADERS copies per stage
#define GS_THREADS ((GS_WARPS + GS_LOADERS) * 32)
#define GS_ROWS 8                               // features per stage; a tile of the product is two stages
#define GS_MAX_STAGES 8
#define GS_CHAINS 4                             // independent accumulators per warp
#define GS_SMEM_LIMIT (227 * 1024 - 2048)

struct GsParams {
    const __nv_bfloat16* W;
    const __nv_bfloat16* X;
    void* out;
    const float* bias;
    long long ldw, ldx, ldo;
    int M, N, K;
    int ks;                 // elements of K per stage
    int n_chunks;           // chunks of K per row
    int stages;
    int out_f32;
    long long split_stride; // elements between the partial outputs of the splits of K (gridDim.y of them)
    int gated;              // W holds N gate rows, then N up rows; the output is silu(gate) * up, N wide
    int* status;
};

__device__ __forceinline__ void gs_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void gs_bar_compute() { asm volatile("bar.sync 1, %0;\n" ::"n"(GS_WARPS * 32) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4_a(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x2(unsigned& r0, unsigned& r1, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// MT: 8-row tiles of x (M <= 8 * MT)
template <int MT>
__global__ void __launch_bounds__(GS_THREADS, 1) gemm_stream_kernel(GsParams p) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_GEMM_STREAM, PB_TL_ENTRY);
    if (gridDim.y > 1) {
        // K is cut into gridDim.y equal parts (p.K is the length of one); part s multiplies its columns of W with
        // its columns of x and writes a partial output of its own, which the reader adds up
        const int s = blockIdx.y;
        p.W += (size_t)s * p.K;
        p.X += (size_t)s * p.K;
        p.out = reinterpret_cast<float*>(p.out) + (size_t)s * p.split_stride;
        if (s > 0) p.bias = nullptr;
    }
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) uint64_t full_bar[GS_MAX_STAGES], empty_bar[GS_MAX_STAGES], x_bar;
    __shared__ int s_issued, s_dead;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int x_stride = p.K * 2 + 16;                         // bytes between rows of x in shared memory
    const int w_stride = p.ks * 2 + 16;                        // bytes between rows of a stage
    const int stage_bytes = GS_ROWS * w_stride;
    unsigned char* sX = smem;                                  // [M] rows
    unsigned char* ring = sX + (size_t)p.M * x_stride;
    float* red = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);   // [GS_WARPS][8 MT batch rows][16 features]

    // This block's features, in tiles of 16 = two stages of 8 (the last tile may have one).  Loader and compute
    // warps walk the stages in the same order: tile, chunk of K, half.
    const int r0 = (int)((long long)blockIdx.x * p.N / gridDim.x), r1 = (int)((long long)(blockIdx.x + 1) * p.N / gridDim.x);
    const int span = p.gated ? GS_ROWS : 16;                   // features per tile
    const int n_tiles = (r1 - r0 + span - 1) / span;

    if (threadIdx.x == 0) {
        s_issued = 0;
        s_dead = 0;
        for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], GS_LOADERS); mbar_init(&empty_bar[s], GS_WARPS); }
        mbar_init(&x_bar, GS_LOADERS);
        mbar_fence_init();
    }
    __syncthreads();

    if (warp >= GS_WARPS) {
        // ---------------- loaders: warp j copies rows 2 j and 2 j + 1 of every stage (lanes 0 and 1) ----------------
        const int lw = warp - GS_WARPS;
        constexpr int PER = GS_ROWS / GS_LOADERS;
        bool ok = true;
        int stage = 0, phase = 0, i = 0;
#pragma unroll 1
        for (int tile = 0; tile < n_tiles && ok; ++tile) {
            const int halves = (p.gated || r1 - (r0 + tile * span) > GS_ROWS) ? 2 : 1;
#pragma unroll 1
            for (int kc = 0; kc < p.n_chunks && ok; ++kc) {
                for (int h = 0; h < halves; ++h, ++i) {
                    if (i >= p.stages) {                       // the first ring-full finds every stage free
                        ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1);
                        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                    }
                    if (lw == 0 && lane == 0) *(volatile int*)&s_issued = i + 1;   // the stage's previous tenant has been consumed
                    const int feat0 = r0 + tile * span + (p.gated ? 0 : h * GS_ROWS);   // first feature of the stage
                    const int row0 = feat0 + (p.gated ? h * p.N : 0);                 // its row of W: up rows follow the gate rows
                    const int k0 = kc * p.ks, len = min(p.ks, p.K - k0);
                    const int n_rows = min(GS_ROWS, r1 - feat0);
                    const int mine = min(PER, max(0, n_rows - lw * PER));        // rows of this stage that this warp brings
                    // the copies may land before the expected bytes are posted: the phase cannot end before this arrival
                    if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], (unsigned)mine * len * 2);
                    const int rr = lw * PER + lane;
                    if (lane < mine)
                        bulk_copy_g2s(ring + (size_t)stage * stage_bytes + (size_t)rr * w_stride,
                                      p.W + (size_t)(row0 + rr) * p.ldw + k0, (unsigned)len * 2, &full_bar[stage]);
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 11);
        return;
    }

    // ---------------- compute warps ----------------
    pb_grid_dep_wait();                                        // the output may still be in use by the kernel before
    PB_TL(PB_TL_GEMM_STREAM, PB_TL_AFTER_WAIT);
    const int g = lane >> 2, t4 = lane & 3;
    if (warp < GS_LOADERS) {
        // x is this kernel's only input that another kernel writes: the first four compute warps fetch it the
        // moment that kernel is done (warp j brings rows j, j + 4, ...), whatever the loaders are busy with
        const int mine = (p.M - warp + GS_LOADERS - 1) / GS_LOADERS;
        if (lane == 0) mbar_arrive_expect_tx(&x_bar, (unsigned)max(mine, 0) * p.K * 2);
        const int m = warp + lane * GS_LOADERS;
        if (m < p.M) bulk_copy_g2s(sX + (size_t)m * x_stride, p.X + (size_t)m * p.ldx, (unsigned)p.K * 2, &x_bar);
    }
    // A warp that gives up waiting says so in s_dead; the compute warps meet at their barrier all the same
    // and leave together, so none is left waiting for one that has gone.
    if (!__all_sync(0xffffffffu, mbar_wait_bounded(&x_bar, 0))) {
        if (lane == 0) { *(volatile int*)&s_dead = 1; if (p.status) atomicExch(p.status, 12); }
    }
    gs_bar_compute();
    if (*(volatile int*)&s_dead) return;
    PB_TL(PB_TL_GEMM_STREAM, PB_TL_INPUT);
    const unsigned sX_a = smem_u32(sX), ring_a = smem_u32(ring);
    // ldmatrix lanes.  W (row operand, 16 features x 16 k): lane -> feature lane & 15 (the first eight in one
    // stage, the others in the next), k half lane >> 4.  x (column operand): 8 batch rows x 16 k (x2), or
    // 16 batch rows (x4); rows that do not exist read the last row that does, and their sums are never stored.
    const unsigned a_off = (lane & 7) * w_stride + (lane >> 4) * 16;
    const bool upper = (lane & 8) != 0;                        // this lane addresses a row of the second stage
    const int x_row = (MT == 1) ? (lane & 7) : ((lane & 7) + (lane >> 4) * 8);
    const unsigned b_off = min(x_row, p.M - 1) * x_stride + ((lane >> 3) & 1) * 16;
    int stage = 0, phase = 0, item = 0;
#pragma unroll 1
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int halves = (p.gated || r1 - (r0 + tile * span) > GS_ROWS) ? 2 : 1;
        // GS_CHAINS independent chains of sums, so that a product does not wait for the one before it
        float acc[GS_CHAINS][MT][4];
#pragma unroll
        for (int c = 0; c < GS_CHAINS; ++c)
#pragma unroll
            for (int j = 0; j < MT; ++j) acc[c][j][0] = acc[c][j][1] = acc[c][j][2] = acc[c][j][3] = 0.f;
#pragma unroll 1
        for (int kc = 0; kc < p.n_chunks; ++kc) {
            const int stage2 = (stage + 1 == p.stages) ? 0 : stage + 1, phase2 = (stage + 1 == p.stages) ? phase ^ 1 : phase;
            const int last = item + halves - 1;
            bool landed = true;
            if (*(volatile int*)&s_issued <= last) {           // not announced yet: the barrier may still be in an older phase
                const long long t0 = clock64();
                while (*(volatile int*)&s_issued <= last)
                    if (clock64() - t0 > (1ll << 31)) { landed = false; break; }
            }
            landed = landed && mbar_wait_bounded(&full_bar[stage], phase);
            if (halves == 2) landed = landed && mbar_wait_bounded(&full_bar[stage2], phase2);
            if (!__all_sync(0xffffffffu, landed)) {
                if (lane == 0) { *(volatile int*)&s_dead = 1; if (p.status) atomicExch(p.status, 12); }
                break;
            }
            const int k0 = kc * p.ks, steps = min(p.ks, p.K - k0) >> 4;
            // with one stage only, the upper eight rows read the lower ones again (their sums are not stored)
            const unsigned a_base = ring_a + ((upper && halves == 2) ? stage2 : stage) * stage_bytes + a_off;
            const unsigned b_base = sX_a + b_off + k0 * 2;
#pragma unroll 1
            for (int s0 = warp; s0 < steps; s0 += GS_WARPS * GS_CHAINS) {
                unsigned a[GS_CHAINS][4], b[GS_CHAINS][4];
#pragma unroll
                for (int c = 0; c < GS_CHAINS; ++c) {
                    const int s = s0 + c * GS_WARPS;
                    if (s < steps) {
                        ldmatrix_x4_a(a[c], a_base + s * 32);
                        if (MT == 1) ldmatrix_x2(b[c][0], b[c][1], b_base + s * 32);
                        else ldmatrix_x4_a(b[c], b_base + s * 32);
                    }
                }
#pragma unroll
                for (int c = 0; c < GS_CHAINS; ++c) {
                    if (s0 + c * GS_WARPS < steps) {
                        mma_bf16_free(acc[c][0], a[c], b[c][0], b[c][1]);
                        if (MT == 2) mma_bf16_free(acc[c][MT - 1], a[c], b[c][2], b[c][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {                                   // this warp is done with the stages
                gs_mbar_arrive(&empty_bar[stage]);
                if (halves == 2) gs_mbar_arrive(&empty_bar[stage2]);
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
                for (int c = 1; c < GS_CHAINS; ++c) v += acc[c][j][e];
                mine[(8 * j + 2 * t4 + (e & 1)) * 16 + g + 8 * (e >> 1)] = v;
            }
        gs_bar_compute();
        if (*(volatile int*)&s_dead) return;
        if (p.gated) {
            // rows 0..7 of the tile are the gate sums of 8 features, rows 8..15 the up sums of the same features
            for (int idx = threadIdx.x; idx < p.M * GS_ROWS; idx += GS_WARPS * 32) {
                const int m = idx >> 3, rr = idx & 7;
                const int n = r0 + tile * GS_ROWS + rr;
                if (n < r1) {
                    float gsum = 0.f, usum = 0.f;
#pragma unroll
                    for (int w = 0; w < GS_WARPS; ++w) {
                        gsum += red[(size_t)w * 16 * 8 * MT + m * 16 + rr];
                        usum += red[(size_t)w * 16 * 8 * MT + m * 16 + rr + 8];
                    }
                    const float v = gsum / (1.0f + expf(-gsum)) * usum;
                    if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
                    else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
                }
            }
        } else {
            for (int idx = threadIdx.x; idx < p.M * 16; idx += GS_WARPS * 32) {
                const int m = idx >> 4, rr = idx & 15;
                const int n = r0 + tile * 16 + rr;
                if (n < r1) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < GS_WARPS; ++w) v += red[(size_t)w * 16 * 8 * MT + idx];
                    if (p.bias) v += p.bias[n];
                    if (p.out_f32) reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
                    else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
                }
            }
        }
        gs_bar_compute();                                      // the sums are read before the next tile overwrites them
    }
    PB_TL(PB_TL_GEMM_STREAM, PB_TL_DONE);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static int g_gs_sms = 0;
static int gs_sms() {
    if (g_gs_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_gs_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_gs_sms <= 0) g_gs_sms = 148;
    }
    return g_gs_sms;
}

// Chunk of K per stage and number of stages for a shape: the fewest chunks per row (the longest copies) that
// leave room for three stages, or for two if three never fit; false when x and two stages do not fit.
static bool gs_plan(int M, int K, int* ks, int* n_chunks, int* stages, size_t* smem) {
    const size_t x_bytes = (size_t)M * ((size_t)K * 2 + 16);
    const size_t red_bytes = (size_t)GS_WARPS * 16 * 16 * 4;
    if (x_bytes + red_bytes >= GS_SMEM_LIMIT) return false;
    const size_t room = GS_SMEM_LIMIT - x_bytes - red_bytes;
    for (int want = 3; want >= 2; --want) {
        for (int n = 1; n <= K / 16; ++n) {
            const int k_per = ((K + n - 1) / n + 15) / 16 * 16;
            const size_t stage = (size_t)GS_ROWS * ((size_t)k_per * 2 + 16);
            if (k_per * 2 < 1024 && n > 1) break;                 // copies this short are not worth having
            if (stage * want <= room) {
                size_t s = room / stage;
                if (s > GS_MAX_STAGES) s = GS_MAX_STAGES;
                *ks = k_per; *n_chunks = (K + k_per - 1) / k_per; *stages = (int)s;
                *smem = x_bytes + red_bytes + s * stage;
                return true;
            }
        }
    }
    return false;
}

// Whether the kernel takes the shape (else the caller uses another product).
PB_API int pb_gemm_stream_supported(int M, int N, int K, long long ldw, long long ldx) {
    if (M < 1 || M > 16 || N < 1 || K < 16 || K % 16 || ldw % 8 || ldx % 8) return 0;
    int ks, nc, st;
    size_t smem;
    return gs_plan(M, K, &ks, &nc, &st, &smem) ? 1 : 0;
}

// gated: W is [2 N, K], N gate rows then N up rows, and out [M, N] = silu(x Wg^T) * (x Wu^T); no bias, no splits.
// splits > 1 cuts K into that many equal parts (K %% (16 * splits) == 0): out is then float32
// [splits][M][ldo-strided N] with split_stride elements between the parts, and the caller adds them.
PB_API int pb_gemm_stream_bf16(const void* X, const void* W, const float* bias, void* out, int M, int N, int K,
                               long long ldx, long long ldw, long long ldo, int out_f32, int splits, long long split_stride,
                               int gated, int* status, cudaStream_t stream) {
    PB_REQUIRE(!gated || (splits == 1 && bias == nullptr), "gemm_stream: the gated form takes no bias and no cut of K");
    PB_REQUIRE(splits >= 1 && splits <= 16 && (splits == 1 || K % (16 * splits) == 0), "gemm_stream: K=%d cannot be cut into %d parts of whole 16-element steps", K, splits);
    PB_REQUIRE(splits == 1 || (out_f32 && split_stride >= (long long)(M - 1) * ldo + N), "gemm_stream: partial sums are float32, %d apart at least", M * N);
    const int k_part = K / splits;
    PB_REQUIRE(pb_gemm_stream_supported(M, N, k_part, ldw, ldx),
               "gemm_stream: M=%d N=%d K=%d not taken (M <= 16, K %% 16 == 0, 16-byte aligned rows, x must fit in shared memory)", M, N, k_part);
    PB_REQUIRE(X && W && out && pb_aligned(X, 16) && pb_aligned(W, 16), "gemm_stream: null or unaligned pointer");
    GsParams p{};
    p.W = (const __nv_bfloat16*)W; p.X = (const __nv_bfloat16*)X; p.out = out; p.bias = bias;
    p.ldw = ldw; p.ldx = ldx; p.ldo = ldo; p.M = M; p.N = N; p.K = k_part; p.out_f32 = out_f32; p.status = status;
    p.split_stride = split_stride;
    p.gated = gated ? 1 : 0;
    size_t smem;
    gs_plan(M, k_part, &p.ks, &p.n_chunks, &p.stages, &smem);
    int blocks = gs_sms() / splits;
    if (blocks < 1) blocks = 1;
    if (blocks > (N + 7) / 8) blocks = (N + 7) / 8;           // at least 8 features per block
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM_LIMIT);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM_LIMIT);
        if (e != cudaSuccess) return pb_fail("gemm_stream: cannot get %d bytes of shared memory: %s", GS_SMEM_LIMIT, cudaGetErrorString(e));
        configured = true;
    }
    if (M <= 8) pb_launch(gemm_stream_kernel<1>, dim3(blocks, splits), dim3(GS_THREADS), smem, stream, p);
    else pb_launch(gemm_stream_kernel<2>, dim3(blocks, splits), dim3(GS_THREADS), smem, stream, p);
    PB_CHECK_LAUNCH("gemm_stream");
    return 0;
}
