// C = A * B^T on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands brought to shared memory by TMA.
//
//   A: [rows_a, K] bfloat16, K contiguous     B: [rows_b, K] bfloat16, K contiguous
//   C[i, j] = sum_k A[i, k] * B[j, k]          float32 accumulation
//
// A linear layer y = x W^T is A = x (128 tokens per tile), B = W (up to 256
// features per tile), for prompt portions and for decode steps alike.  A decode
// step has a handful of tokens: TMA fills the rows of the A tile that do not
// exist with zeros, and the step is a stream over W.
// (The reference sends these products to DeepGEMM / CUTLASS / cuBLAS,
// crates/prelude-cuda/src/ops/gemm.rs:35-137; its sm_100 path is
// crates/prelude-cuda/deepgemm/src/sm100_bf16.cuh:10-205.)
//
// Structure.  A persistent grid, one block per multiprocessor.  The work is the
// list of (output tile, 64-wide k block) items in tile-major order; every block
// takes one contiguous run of items, so all blocks move the same number of bytes
// whatever the shape.  A run of items inside one tile is a segment: its products
// are accumulated in tensor memory.  A segment that covers its tile's whole K is
// written straight to the output; otherwise the block writes a float32 partial
// tile to scratch memory and counts itself in, and the block that arrives last
// for the tile adds the partial tiles up in block order and writes the output
// (the counters are left at zero for the next call).
//
// Warps: 0..3 read accumulators out of tensor memory and store (tcgen05.ld; warp w
// owns lanes 32w..32w+31), warp 4 issues the TMA loads (one lane), warp 5 owns the
// tensor memory allocation and issues the MMAs (one lane).  Shared memory is a
// ring of stages (A tile 128 x 64, B tile BN x 64, 128-byte swizzle) with a full
// and an empty barrier each; tensor memory holds two accumulators so that a
// segment's stores overlap the next segment's products.  Every wait on a barrier
// is bounded in time; a block that gives up raises the status word, frees its
// tensor memory and returns.  No load uses cluster multicast.
#include "tcgen05.cuh"

#include <stdlib.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_A_BYTES (TC_BM * TC_BK * 2)

struct TcParams {
    void* out;                  // [rows_a, rows_b] bfloat16 or float32
    const float* bias;          // per column of out, or null
    float* scratch;             // [grid][2][128][BN] partial tiles
    int* counters;              // [tiles], zero on entry and on exit
    int* status;
    long long ldo;
    int rows_a, rows_b, K;
    int tiles_a, tiles_b, kblocks, items_per_block;
    int b_is_constant;          // B is written by no kernel (weights): its loads need not wait for the previous kernel
    int out_f32;
};

// N consecutive columns of one output row, from float32 sums
template <int N>
__device__ __forceinline__ void tc_store_n(const TcParams& p, int gi, int gj0, const float* v) {
    if (p.out_f32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)gi * p.ldo + gj0;
        if (gj0 + N <= p.rows_b && !p.bias && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < N; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j)
                if (gj0 + j < p.rows_b) o[j] = v[j] + (p.bias ? p.bias[gj0 + j] : 0.f);
        }
    } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)gi * p.ldo + gj0;
        if (gj0 + N <= p.rows_b && !p.bias && ((reinterpret_cast<uintptr_t>(o) & (2 * N - 1)) == 0)) {
            unsigned w[N / 2];
#pragma unroll
            for (int j = 0; j < N / 2; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<unsigned*>(&h);
            }
            if constexpr (N == 4) {
                *reinterpret_cast<uint2*>(o) = make_uint2(w[0], w[1]);
            } else {
#pragma unroll
                for (int j = 0; j < N / 2; j += 4) *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j)
                if (gj0 + j < p.rows_b) o[j] = __float2bfloat16_rn(v[j] + (p.bias ? p.bias[gj0 + j] : 0.f));
        }
    }
}
__device__ __forceinline__ void tc_store16(const TcParams& p, int gi, int gj0, const float* v) { tc_store_n<16>(p, gi, gj0, v); }

template <int BN>
struct TcShared {
    static constexpr int STAGE_BYTES = TC_A_BYTES + BN * TC_BK * 2;
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > 10 ? 10 : (200 * 1024 / STAGE_BYTES);
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
};

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
    pb_grid_dep_launch();
    using S = TcShared<BN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[S::STAGES], empty_bar[S::STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_holder;
    __shared__ int s_flag, s_ok;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items_total = p.tiles_a * p.tiles_b * p.kblocks;
    const int my_begin = blockIdx.x * p.items_per_block;
    const int my_end = min(items_total, my_begin + p.items_per_block);

    if (threadIdx.x == 0) {
        s_ok = 1;
        for (int s = 0; s < S::STAGES; ++s) { tc_mbar_init(&full_bar[s], 1); tc_mbar_init(&empty_bar[s], 1); }
        for (int a = 0; a < 2; ++a) { tc_mbar_init(&acc_full[a], 1); tc_mbar_init(&acc_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 5) tc_tmem_alloc(&tmem_holder, S::TMEM_COLS);
    if (warp == 4 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_holder;
    // Barriers, tensor memory and descriptors are set up.  Every thread waits for the kernel before this one
    // before it first touches memory that a kernel writes; weights are written by no kernel, so when B holds
    // them the producer starts their stream before that wait and fills the whole ring while the previous
    // kernel is still finishing.
    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int fill = 0;
            bool ok = true;
            const int ahead = p.b_is_constant ? min(S::STAGES, my_end - my_begin) : 0;
            for (int j = 0; j < ahead; ++j) {
                const int it = my_begin + j;
                const int tile = it / p.kblocks, kb = it - tile * p.kblocks;
                tc_mbar_expect_tx(&full_bar[j], S::STAGE_BYTES);
                tc_tma_load_2d(smem + j * S::STAGE_BYTES + TC_A_BYTES, &map_b, kb * TC_BK, (tile / p.tiles_a) * BN, &full_bar[j]);
            }
            pb_grid_dep_wait();
            for (int j = 0; j < ahead; ++j) {
                const int it = my_begin + j;
                const int tile = it / p.kblocks, kb = it - tile * p.kblocks;
                tc_tma_load_2d(smem + j * S::STAGE_BYTES, &map_a, kb * TC_BK, (tile % p.tiles_a) * TC_BM, &full_bar[j]);
            }
            fill = ahead;
            for (int it = my_begin + ahead; it < my_end && ok; ++it, ++fill) {
                const int tile = it / p.kblocks, kb = it - tile * p.kblocks;
                const int ta = tile % p.tiles_a, tb = tile / p.tiles_a;      // A tiles vary fastest: neighbours share the B panel
                const int stage = fill % S::STAGES;
                ok = tc_mbar_wait(&empty_bar[stage], ((fill / S::STAGES) & 1) ^ 1);
                if (!ok) break;
                unsigned char* sa = smem + stage * S::STAGE_BYTES;
                tc_mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
                tc_tma_load_2d(sa, &map_a, kb * TC_BK, ta * TC_BM, &full_bar[stage]);
                tc_tma_load_2d(sa + TC_A_BYTES, &map_b, kb * TC_BK, tb * BN, &full_bar[stage]);
            }
            if (!ok && p.status) atomicExch(p.status, 8);
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer: reads shared and tensor memory only ----------------
        // The whole warp walks the loop and waits; an elected lane issues (under elect.sync the descriptors stay in
        // uniform registers; from a branch on the lane number every tcgen05.mma cost the thread about 100 cycles).
        const uint32_t idesc = tc_instr_desc(BN);
        int fill = 0, seg = 0;
        bool ok = true;
        for (int it = my_begin; it < my_end && ok; ++seg) {
            const int tile = it / p.kblocks;
            const int seg_end = min(my_end, (tile + 1) * p.kblocks);
            const int acc = seg & 1;
            ok = __all_sync(0xffffffffu, tc_mbar_wait(&acc_empty[acc], ((seg >> 1) & 1) ^ 1));
            if (!ok) break;
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (int i = it; i < seg_end; ++i, ++fill) {
                const int stage = fill % S::STAGES;
                ok = __all_sync(0xffffffffu, tc_mbar_wait(&full_bar[stage], (fill / S::STAGES) & 1));
                if (!ok) break;
                tc_fence_after();
                if (tc_elect_one()) {
                    const unsigned char* sa = smem + stage * S::STAGE_BYTES;
                    const uint64_t da = tc_smem_desc(sa), db = tc_smem_desc(sa + TC_A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)                         // 32 bytes along K per instruction
                        tc_mma(d_tmem, da + 2 * k, db + 2 * k, idesc, (i > it || k > 0) ? 1u : 0u);
                    tc_commit(&empty_bar[stage]);                                // the stage is free when these finish
                    if (i + 1 == seg_end) tc_commit(&acc_full[acc]);
                }
                __syncwarp();
            }
            if (!ok) break;
            it = seg_end;
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 9);
    } else {
        // ---------------- epilogue: 4 warps, 128 accumulator rows ----------------
        pb_grid_dep_wait();                                                      // the output and the scratch may still be in use
        const int row = warp * 32 + lane;                                        // row of the tile = tensor-memory lane
        int seg = 0;
        bool ok = true;
        for (int it = my_begin; it < my_end; ++seg) {
            const int tile = it / p.kblocks;
            const int tile_begin = tile * p.kblocks, tile_end = tile_begin + p.kblocks;
            const int seg_end = min(my_end, tile_end);
            const int ta = tile % p.tiles_a, tb = tile / p.tiles_a;
            const int acc = seg & 1;
            if (ok) ok = tc_mbar_wait(&acc_full[acc], (seg >> 1) & 1);
            if (!ok) s_ok = 0;
            tc_bar_epilogue();                                                   // the four warps go on, or give up, together
            if (!s_ok) { ok = false; break; }
            tc_fence_after();
            const bool whole = (it == tile_begin) && (seg_end == tile_end);
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(warp * 32) << 16);
            const int rows_here = min(TC_BM, p.rows_a - ta * TC_BM);             // rows of the tile that exist
            const int gi = ta * TC_BM + row;                                     // row of A
            float* part = p.scratch + ((size_t)blockIdx.x * 2 + (it == my_begin ? 0 : 1)) * TC_BM * BN;
            // a decode step has a handful of rows: warps whose 32 rows are all padding skip the loads
            if (warp * 32 < rows_here) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float v[16];
                    tc_tmem_ld16(taddr + c0, v);
                    if (gi < p.rows_a) {
                        if (!whole) {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                *reinterpret_cast<float4*>(part + (size_t)row * BN + c0 + 4 * q) =
                                    make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
                            tc_store16(p, gi, tb * BN + c0, v);
                        }
                    }
                    __syncwarp();                                                // the next tensor-memory load needs the whole warp
                }
            }
            // the accumulator may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&acc_empty[acc]);
            if (!whole) {
                // count this block in; the last one for the tile adds the partial tiles up, in block order
                const int c_first = tile_begin / p.items_per_block, c_last = (tile_end - 1) / p.items_per_block;
                __threadfence();
                tc_bar_epilogue();
                if (threadIdx.x == 0) {
                    const int old = atomicAdd(p.counters + tile, 1);
                    s_flag = (old == c_last - c_first);
                    if (s_flag) p.counters[tile] = 0;
                }
                tc_bar_epilogue();
                if (s_flag) {
                    __threadfence();
                    // all 128 threads share the rows that exist: four columns each, the partial tiles of
                    // the blocks c_first..c_last added in that order (independent loads, four in flight)
                    const int quads = BN / 4;
                    for (int idx = threadIdx.x; idx < rows_here * quads; idx += 128) {
                        const int r = idx / quads, c4 = (idx - r * quads) * 4;
                        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int c = c_first; c <= c_last; c += 4) {
                            float4 x[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int cc = min(c + u, c_last);
                                const int slot = (cc * p.items_per_block >= tile_begin) ? 0 : 1;
                                x[u] = __ldcg(reinterpret_cast<const float4*>(
                                    p.scratch + ((size_t)cc * 2 + slot) * TC_BM * BN + (size_t)r * BN + c4));
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (c + u <= c_last) { sum.x += x[u].x; sum.y += x[u].y; sum.z += x[u].z; sum.w += x[u].w; }
                        }
                        const float vv[4] = {sum.x, sum.y, sum.z, sum.w};
                        tc_store_n<4>(p, ta * TC_BM + r, tb * BN + c4, vv);
                    }
                }
                tc_bar_epilogue();
            }
            it = seg_end;
        }
        if (!ok && lane == 0 && p.status) atomicExch(p.status, 10);
    }
    // everybody is done with tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        tc_fence_after();
        tc_tmem_dealloc(tmem_base, S::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
// a [rows, K] bfloat16 matrix with row stride ld (elements), boxes of {64 k, box_rows}
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, long long ld, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pb_fail("gemm_tc: cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d ld=%lld)", (int)r, rows, K, ld);
    return 0;
}

static int g_tc_sms = 0;
static int tc_sms() {
    if (g_tc_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_tc_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_tc_sms <= 0) g_tc_sms = 148;
    }
    return g_tc_sms;
}

static int pick_bn(int rows_b) { return rows_b <= 16 ? 16 : rows_b <= 32 ? 32 : rows_b <= 64 ? 64 : rows_b <= 128 ? 128 : 256; }

#define TC_MAX_TILES 65536    // arrival counters sit at the start of the scratch, partial tiles after them

static void tc_plan(int rows_a, int rows_b, int K, int* bn, int* tiles_a, int* tiles_b, int* kblocks, int* ipb, int* blocks) {
    *bn = pick_bn(rows_b);
    *tiles_a = (rows_a + TC_BM - 1) / TC_BM;
    *tiles_b = (rows_b + *bn - 1) / *bn;
    *kblocks = (K + TC_BK - 1) / TC_BK;
    const long long items = (long long)*tiles_a * *tiles_b * *kblocks;
    long long b = tc_sms();
    if (b > items) b = items;
    *ipb = (int)((items + b - 1) / b);
    *blocks = (int)((items + *ipb - 1) / *ipb);
}

// Whether the kernel takes the shape: 16-byte aligned rows (K and both row strides multiples of 8).
PB_API int pb_gemm_tc_supported(int rows_a, int rows_b, int K, long long lda, long long ldb) {
    if (rows_a < 1 || rows_b < 1 || K < 8 || K % 8 || lda % 8 || ldb % 8) return 0;
    long long tiles = (long long)((rows_a + TC_BM - 1) / TC_BM) * ((rows_b + pick_bn(rows_b) - 1) / pick_bn(rows_b));
    return tiles <= TC_MAX_TILES;
}

// Bytes of scratch a call needs: TC_MAX_TILES counters, then two partial tiles per block.
PB_API long long pb_gemm_tc_scratch_bytes(int rows_a, int rows_b, int K) {
    int bn, ta, tb, kb, ipb, blocks;
    tc_plan(rows_a, rows_b, K, &bn, &ta, &tb, &kb, &ipb, &blocks);
    return (long long)TC_MAX_TILES * 4 + (long long)blocks * 2 * TC_BM * bn * 4;
}

template <int BN>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int blocks, cudaStream_t stream) {
    using S = TcShared<BN>;
    static bool configured = false;
    const size_t smem = (size_t)S::STAGES * S::STAGE_BYTES + 1024;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return pb_fail("gemm_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    pb_launch(gemm_tc_kernel<BN>, dim3(blocks), dim3(TC_THREADS), smem, stream, ma, mb, p);
    return 0;
}

// out[i * ldo + j] = sum_k A[i, k] B[j, k] (+ bias[j]).
// bias: per column of out, float32 or null.  out_f32: 1 for float32 output, 0 for bfloat16.
// b_is_constant: 1 when no kernel writes B (a weight matrix): its stream then starts before the
// previous kernel on the stream has finished.
// scratch: pb_gemm_tc_scratch_bytes(...) bytes whose first 4 * TC_MAX_TILES bytes (the counters) are zero
// before the first call; every call leaves them zero, so calls on one stream may share the buffer.
PB_API int pb_gemm_tc_bf16(const void* A, const void* B, const float* bias, void* out, int rows_a, int rows_b, int K,
                           long long lda, long long ldb, long long ldo, int b_is_constant, int out_f32, void* scratch,
                           int* status, cudaStream_t stream) {
    PB_REQUIRE(pb_gemm_tc_supported(rows_a, rows_b, K, lda, ldb),
               "gemm_tc: rows_a=%d rows_b=%d K=%d lda=%lld ldb=%lld not taken (rows must be 16-byte aligned)", rows_a, rows_b, K, lda, ldb);
    PB_REQUIRE(A && B && out && scratch && pb_aligned(A, 16) && pb_aligned(B, 16), "gemm_tc: null or unaligned pointer");
    if (int e = get_encode()) return e;
    TcParams p{};
    int bn, blocks;
    tc_plan(rows_a, rows_b, K, &bn, &p.tiles_a, &p.tiles_b, &p.kblocks, &p.items_per_block, &blocks);
    p.out = out; p.bias = bias; p.status = status; p.ldo = ldo; p.rows_a = rows_a; p.rows_b = rows_b; p.K = K;
    p.b_is_constant = b_is_constant; p.out_f32 = out_f32;
    p.counters = (int*)scratch;
    p.scratch = (float*)((char*)scratch + (size_t)TC_MAX_TILES * 4);
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, A, rows_a, K, lda, TC_BM)) return e;
    if (int e = make_map(&mb, B, rows_b, K, ldb, bn)) return e;
    int e = bn == 16 ? tc_launch<16>(ma, mb, p, blocks, stream)
          : bn == 32 ? tc_launch<32>(ma, mb, p, blocks, stream)
          : bn == 64 ? tc_launch<64>(ma, mb, p, blocks, stream)
          : bn == 128 ? tc_launch<128>(ma, mb, p, blocks, stream) : tc_launch<256>(ma, mb, p, blocks, stream);
    if (e) return e;
    PB_CHECK_LAUNCH("gemm_tc");
    return 0;
}
