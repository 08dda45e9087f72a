// y[M, N] = x[M, K] * W[N, K]^T for few rows (decode steps: M = requests in
// the batch), bfloat16 in, float32 accumulation, bfloat16 out.
//
// With so few rows the product is a stream over the weight matrix: every byte
// of W is read once and the time is W's bytes over the memory bandwidth.  The
// kernel is built around that stream.
//
//  * W is the row operand of the tensor-core instruction (16 output features x
//    16 k per mma.m16n8k16), x the column operand (8 batch rows per tile).  Each
//    lane loads 16 contiguous bytes of a weight row straight from global memory
//    into registers; the eight k values of such a load are dealt to two
//    instructions, and x is loaded with the same dealing, so the sum over k is
//    the same set of products in a permuted order and no shuffle or shared
//    memory is needed for W.
//  * The work is cut into items of 32 output features x 512 k (32 KB of W),
//    numbered feature-group-major, and every block takes one contiguous run of
//    items, so all blocks stream the same number of bytes whatever the shape
//    (2560 outputs or 19456).  A block keeps accumulating while its items stay
//    in one feature group.  A group whose items are spread over several blocks
//    gets partial sums in scratch memory; the block that arrives last adds them
//    in block order (fixed, so the result does not depend on timing) and writes
//    the output.  The arrival counters are left at zero for the next call.
//  * Inside a block, 2 x 4 warps: two 16-feature tiles, four warps taking every
//    fourth 32-k step of the item, added up through shared memory.
//
// The reference leaves these shapes to its GEMM libraries
// (crates/prelude-cuda/src/ops/gemm.rs:35-137; DeepGEMM's small-M path).
// Needs K % 32 == 0, N % 16 == 0, M <= 64, 16-byte aligned rows.
#include "common.cuh"

#define SK_THREADS 256
#define SK_ROWS 32            // output features per item
#define SK_KC 512             // k per item
#define SK_KW 4               // warps along k

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16816(float* c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyParams {
    const __nv_bfloat16* W;
    const __nv_bfloat16* X;
    __nv_bfloat16* Y;
    const float* bias;
    float* scratch;         // [gridDim.x][2][SK_ROWS][8 * MT] partial sums
    int* counters;          // [n_groups], zero on entry, zero on exit
    long long ldw, ldx, ldy;
    int M, N, K;
    int n_groups, k_chunks, items_per_block;
};

// MT: number of 8-row tiles of x (M <= 8 * MT)
template <int MT>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(SkinnyParams p) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    constexpr int MP = 8 * MT;
    __shared__ float red[SK_KW][SK_ROWS][MP + 1];
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int wn = warp & 1, wk = warp >> 1;        // which 16-feature tile, which k phase
    const int items_total = p.n_groups * p.k_chunks;
    const int my_begin = blockIdx.x * p.items_per_block;
    const int my_end = min(items_total, my_begin + p.items_per_block);

    for (int it = my_begin; it < my_end;) {
        const int grp = it / p.k_chunks;
        const int grp_begin = grp * p.k_chunks, grp_end = grp_begin + p.k_chunks;
        const int seg_end = min(my_end, grp_end);
        const int k_begin = (it - grp_begin) * SK_KC, k_end = min(p.K, (seg_end - grp_begin) * SK_KC);
        const int n0 = grp * SK_ROWS + wn * 16;

        float acc[MT][4];
#pragma unroll
        for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

        if (n0 < p.N) {
            const __nv_bfloat16* w0 = p.W + (size_t)(n0 + g) * p.ldw + 8 * t4;
            const __nv_bfloat16* w1 = w0 + 8 * p.ldw;
            const int steps = (k_end - k_begin) / 32;
            // this warp's steps: wk, wk + 4, ...; four of them in flight
            for (int s = wk; s < steps; s += 4 * SK_KW) {
                uint4 a_lo[4], a_hi[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int k = k_begin + (s + u * SK_KW) * 32;
                    if (s + u * SK_KW < steps) {
                        a_lo[u] = ld_stream16(w0 + k);
                        a_hi[u] = ld_stream16(w1 + k);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (s + u * SK_KW < steps) {
                        const int k = k_begin + (s + u * SK_KW) * 32 + 8 * t4;
#pragma unroll
                        for (int j = 0; j < MT; ++j) {
                            const int m = 8 * j + g;
                            uint4 b = make_uint4(0, 0, 0, 0);
                            if (m < p.M) b = *reinterpret_cast<const uint4*>(p.X + (size_t)m * p.ldx + k);
                            mma16816(acc[j], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, b.x, b.y);
                            mma16816(acc[j], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, b.z, b.w);
                        }
                    }
                }
            }
        }
        // add the four k phases of the block: acc[j][e] is feature n0 + g (+8 for e >= 2), row 8j + 2 t4 + (e & 1)
#pragma unroll
        for (int j = 0; j < MT; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) red[wk][wn * 16 + g + 8 * (e >> 1)][8 * j + 2 * t4 + (e & 1)] = acc[j][e];
        }
        __syncthreads();
        const bool whole = (it == grp_begin) && (seg_end == grp_end);
        float* part = p.scratch + ((size_t)blockIdx.x * 2 + (it == my_begin ? 0 : 1)) * SK_ROWS * MP;
        for (int idx = threadIdx.x; idx < SK_ROWS * MP; idx += SK_THREADS) {
            const int r = idx / MP, m = idx - r * MP;
            float v = red[0][r][m];
#pragma unroll
            for (int q = 1; q < SK_KW; ++q) v += red[q][r][m];
            if (whole) {
                const int n = grp * SK_ROWS + r;
                if (m < p.M && n < p.N) {
                    if (p.bias) v += p.bias[n];
                    p.Y[(size_t)m * p.ldy + n] = __float2bfloat16_rn(v);
                }
            } else {
                part[idx] = v;
            }
        }
        if (!whole) {
            // the group is shared with other blocks: the last to arrive adds all partial sums up
            const int c_first = grp_begin / p.items_per_block, c_last = (grp_end - 1) / p.items_per_block;
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const int old = atomicAdd(p.counters + grp, 1);
                s_last = (old == c_last - c_first);
                if (s_last) p.counters[grp] = 0;
            }
            __syncthreads();
            if (s_last) {
                __threadfence();
                for (int idx = threadIdx.x; idx < SK_ROWS * MP; idx += SK_THREADS) {
                    const int r = idx / MP, m = idx - r * MP;
                    const int n = grp * SK_ROWS + r;
                    if (m >= p.M || n >= p.N) continue;
                    float v = 0.f;
                    for (int c = c_first; c <= c_last; ++c) {
                        const int slot = (max(c * p.items_per_block, grp_begin) == c * p.items_per_block) ? 0 : 1;
                        v += __ldcg(p.scratch + ((size_t)c * 2 + slot) * SK_ROWS * MP + idx);
                    }
                    if (p.bias) v += p.bias[n];
                    p.Y[(size_t)m * p.ldy + n] = __float2bfloat16_rn(v);
                }
            }
        }
        __syncthreads();
        it = seg_end;
    }
}

// Blocks a call uses, and the scratch it needs, for a device with `sms` multiprocessors.
static int skinny_grid(int N, int K, int sms, int* items_per_block, int* n_groups, int* k_chunks) {
    *n_groups = (N + SK_ROWS - 1) / SK_ROWS;
    *k_chunks = (K + SK_KC - 1) / SK_KC;
    const int items = *n_groups * *k_chunks;
    int blocks = sms * 2;
    if (blocks > items) blocks = items;
    *items_per_block = (items + blocks - 1) / blocks;
    return (items + *items_per_block - 1) / *items_per_block;
}

static int g_sms = 0;
static int device_sms() {
    if (g_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_sms <= 0) g_sms = 148;
    }
    return g_sms;
}

#define SK_MAX_GROUPS 8192     // arrival counters sit at the start of the scratch, partial sums after them

// Bytes of scratch a call needs: SK_MAX_GROUPS int counters, then the partial sums.
PB_API long long pb_gemm_skinny_scratch_bytes(int M, int N, int K) {
    int ipb, ng, kc;
    const int blocks = skinny_grid(N, K, device_sms(), &ipb, &ng, &kc);
    const int mp = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    return (long long)SK_MAX_GROUPS * 4 + (long long)blocks * 2 * SK_ROWS * mp * 4;
}

// Whether the kernel takes the shape (else the caller uses the library product).
PB_API int pb_gemm_skinny_supported(int M, int N, int K, long long ldw, long long ldx) {
    return M >= 1 && M <= 64 && N % 16 == 0 && K % 32 == 0 && ldw % 8 == 0 && ldx % 8 == 0 &&
           (N + SK_ROWS - 1) / SK_ROWS <= SK_MAX_GROUPS;
}

// scratch: pb_gemm_skinny_scratch_bytes(...) bytes; its first 4 * SK_MAX_GROUPS bytes (the
// arrival counters) must be zero before the first call and are left zero by every call, so
// calls that run one after the other on a stream may share one scratch buffer.
PB_API int pb_gemm_skinny_bf16(const void* X, const void* W, const float* bias, void* Y, int M, int N, int K,
                               long long ldx, long long ldw, long long ldy, void* scratch, cudaStream_t stream) {
    PB_REQUIRE(pb_gemm_skinny_supported(M, N, K, ldw, ldx),
               "gemm_skinny: M=%d N=%d K=%d not taken (M <= 64, N %% 16 == 0, K %% 32 == 0, rows 16-byte aligned)", M, N, K);
    PB_REQUIRE(pb_aligned(X, 16) && pb_aligned(W, 16) && X && W && Y && scratch, "gemm_skinny: null or unaligned pointer");
    SkinnyParams p{};
    p.W = (const __nv_bfloat16*)W; p.X = (const __nv_bfloat16*)X; p.Y = (__nv_bfloat16*)Y; p.bias = bias;
    p.ldw = ldw; p.ldx = ldx; p.ldy = ldy; p.M = M; p.N = N; p.K = K;
    const int blocks = skinny_grid(N, K, device_sms(), &p.items_per_block, &p.n_groups, &p.k_chunks);
    const int mp = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
    p.counters = (int*)scratch;
    p.scratch = (float*)((char*)scratch + (size_t)SK_MAX_GROUPS * 4);
    if (mp == 8) pb_launch(gemm_skinny_kernel<1>, dim3(blocks), dim3(SK_THREADS), 0, stream, p);
    else if (mp == 16) pb_launch(gemm_skinny_kernel<2>, dim3(blocks), dim3(SK_THREADS), 0, stream, p);
    else if (mp == 32) pb_launch(gemm_skinny_kernel<4>, dim3(blocks), dim3(SK_THREADS), 0, stream, p);
    else pb_launch(gemm_skinny_kernel<8>, dim3(blocks), dim3(SK_THREADS), 0, stream, p);
    PB_CHECK_LAUNCH("gemm_skinny");
    return 0;
}
