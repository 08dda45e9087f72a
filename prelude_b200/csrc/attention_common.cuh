// Helpers shared by the tensor-core attention kernels (and the weight-streaming product): asynchronous
// copies and their barriers, the bfloat16 mma, the parameter block, and the computation of one
// 64-key attention tile.
#pragma once
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

// --- bulk asynchronous copies that complete on a shared-memory barrier -------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// one arrival that also announces `bytes` of copies to come
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Wait for the barrier's phase with the given parity for about a second at most: false on giving up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (clock64() - start < (1ll << 31)) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// `bytes` (a multiple of 16) from global to shared memory, both 16-byte aligned; completion is counted on `bar`
__device__ __forceinline__ void bulk_copy_g2s(void* smem, const void* gmem, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// orders earlier ordinary shared-memory accesses of this thread before later asynchronous copies
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// m16n8k16 bfloat16 product with float32 accumulation; not `volatile`: the compiler may move it among the loads around it
__device__ __forceinline__ void mma_bf16_free(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q;        // [T, nH, D]
    const __nv_bfloat16* k_pages;  // [pages, nKV, page_size, D]
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
    int swizzle;                   // pages store the 16-byte chunks of a token row permuted (see pb_kv_elem_offset)
    float scale_log2;              // scale * log2(e)
    int* status;
};

// ---------------------------------------------------------------------------------------
// the tile computation shared by the prefill and the decode kernel
// ---------------------------------------------------------------------------------------
#include <type_traits>

#define ATT_RESCALE_STEP 8.0f   // log2 of the growth of a row maximum that forces a rescale

template <int I, int N, typename F> __device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// ldmatrix from a shared-memory byte address plus a compile-time offset
template <int IMM> __device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(IMM));
}
template <int IMM> __device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr), "n"(IMM));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Geometry of a key (or value) tile in shared memory, as the tile computation sees it.
template <int DMAX, bool BULK> struct AttnTileGeom {
    static constexpr int STRIDE = BULK ? DMAX : DMAX + 8;     // elements per row in shared memory
    static constexpr int ROW_BYTES = STRIDE * 2;
    static constexpr int TILE_BYTES = BN * ROW_BYTES;          // one tile of keys (or of values)
    // ldmatrix row addresses: with permuted chunks, chunk c of row r sits at c ^ (r & 7).  The chunk
    // index of step kk is 2 kk + b with a per-lane bit b, and r & 7 = lane & 7, so the position is
    // (2 kk) ^ x with the per-lane constant x = b ^ (lane & 7): four distinct values of the low bits
    // (kk & 3), kept in registers, and bit 3 of the chunk (kk >> 2), an immediate.
    static constexpr int NOFF = BULK ? 4 : 1;
};

// What a compute thread keeps about its place in the fragments.
template <int DMAX, bool BULK> struct FragOffsets {
    unsigned q[AttnTileGeom<DMAX, BULK>::NOFF], k[AttnTileGeom<DMAX, BULK>::NOFF], v[AttnTileGeom<DMAX, BULK>::NOFF];
};

// The fragment offsets of a lane whose warp owns rows row0 .. row0 + 15 of the q tile.
template <int DMAX, bool BULK>
__device__ __forceinline__ void attn_frag_offsets(FragOffsets<DMAX, BULK>& f, int row0, int lane) {
    using T = AttnTileGeom<DMAX, BULK>;
    const int x = lane & 7;
    const int q_row = row0 + (lane & 15), q_b = lane >> 4;
    const int k_row = (lane >> 4) * 8 + x, k_b = (lane >> 3) & 1;
    const int v_row = ((lane >> 3) & 1) * 8 + x, v_b = lane >> 4;
#pragma unroll
    for (int j = 0; j < T::NOFF; ++j) {
        f.q[j] = q_row * T::ROW_BYTES + (BULK ? (((2 * j) ^ (q_b ^ x)) << 4) : q_b * 16);
        f.k[j] = k_row * T::ROW_BYTES + (BULK ? (((2 * j) ^ (k_b ^ x)) << 4) : k_b * 16);
        f.v[j] = v_row * T::ROW_BYTES + (BULK ? (((2 * j) ^ (v_b ^ x)) << 4) : v_b * 16);
    }
}

template <int DMAX, bool BULK, int KK> __device__ __forceinline__ constexpr int step_imm() {
    // byte offset of 16-element step KK beyond the per-lane offset that serves it
    return BULK ? (KK >> 2) * 128 : KK * 32;
}

// One 64-key tile against a warp's 16 rows: scores, running maximum and sum, O += P V.  Written for few
// instructions per tensor-core product: the byte offsets of every ldmatrix are per-thread constants plus
// immediates, masking runs only when `edge` says the tile holds an invisible key, the scale is folded into
// the exponent's multiply-add, and the accumulator is rescaled only when a row's maximum grew by more than
// 2^ATT_RESCALE_STEP (sum and accumulator then stay relative to a slightly stale maximum, which the final
// division cancels).
template <int DMAX, bool BULK>
__device__ __forceinline__ void attn_tile(float (&o)[DMAX / 8][4], float (&m)[2], float (&l)[2],
                                             const FragOffsets<DMAX, BULK>& f, unsigned sQ, unsigned sK, unsigned sV,
                                             int d, int key0, const int (&row_pos)[2], bool edge, int window,
                                             float scale_log2, int t4) {
    using T = AttnTileGeom<DMAX, BULK>;
    constexpr int KSTEPS = DMAX / 16;
    constexpr bool PIPE = DMAX <= 128;        // larger heads leave no registers for fragments fetched ahead

    // ---- S = Q K^T: 16 rows x 64 keys; the fragments of the next 16-element step are fetched ahead ----
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
        unsigned qa[PIPE ? 2 : 1][4], kb[PIPE ? 2 : 1][4][4];
        unsigned kaddr[T::NOFF], qaddr[T::NOFF];
#pragma unroll
        for (int j = 0; j < T::NOFF; ++j) { kaddr[j] = sK + f.k[j]; qaddr[j] = sQ + f.q[j]; }
        auto fetch = [&](auto kk_c, int buf) {
            constexpr int kk = decltype(kk_c)::value;
            constexpr int imm = step_imm<DMAX, BULK, kk>();
            ldsm_x4<imm>(qa[buf], qaddr[BULK ? (kk & 3) : 0]);
            static_for<0, 4>([&](auto n2_c) {
                constexpr int n2 = decltype(n2_c)::value;
                ldsm_x4<imm + n2 * 16 * T::ROW_BYTES>(kb[buf][n2], kaddr[BULK ? (kk & 3) : 0]);
            });
        };
        if (PIPE) fetch(std::integral_constant<int, 0>{}, 0);
        static_for<0, KSTEPS>([&](auto kk_c) {
            constexpr int kk = decltype(kk_c)::value;
            constexpr int buf = PIPE ? (kk & 1) : 0;
            if (BULK || kk * 16 < d) {
                if constexpr (!PIPE) fetch(kk_c, 0);
                else if constexpr (kk + 1 < KSTEPS) {
                    if (BULK || (kk + 1) * 16 < d) fetch(std::integral_constant<int, kk + 1>{}, buf ^ 1);
                }
#pragma unroll
                for (int n2 = 0; n2 < 4; ++n2) {
                    mma_bf16_free(s[2 * n2], qa[buf], kb[buf][n2][0], kb[buf][n2][1]);
                    mma_bf16_free(s[2 * n2 + 1], qa[buf], kb[buf][n2][2], kb[buf][n2][3]);
                }
            }
        });
    }

    // ---- mask (only in tiles with an invisible key), running maximum ----
    if (edge) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = key0 + nt * 8 + 2 * t4 + (e & 1);
                const int pr = row_pos[e >> 1];
                const bool vis = j <= pr && (window <= 0 || j > pr - window);
                s[nt][e] = vis ? s[nt][e] : -INFINITY;
            }
        }
    }
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        rmax[0] = fmaxf(rmax[0], fmaxf(s[nt][0], s[nt][1]));
        rmax[1] = fmaxf(rmax[1], fmaxf(s[nt][2], s[nt][3]));
    }
    bool grow = false;
    float cand[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
        rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
        cand[h] = fmaxf(m[h], rmax[h] * scale_log2);          // scale > 0: the maximum commutes with it
        grow = grow || cand[h] > m[h] + ATT_RESCALE_STEP;      // also true for -inf -> finite
    }
    if (__any_sync(0xffffffffu, grow)) {
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            corr[h] = (m[h] == -INFINITY) ? 0.f : ex2_approx(m[h] - cand[h]);   // cand >= m; both -inf: nothing summed yet
            m[h] = cand[h];
            l[h] *= corr[h];
        }
#pragma unroll
        for (int i = 0; i < DMAX / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
    }
    // exp2(s * scale - m); a row that has seen nothing yet has m = -inf and only -inf scores: exp2(-inf - 0) = 0
    const float mref[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float pv = ex2_approx(fmaf(s[nt][e], scale_log2, -mref[e >> 1]));
            s[nt][e] = pv;
            l[e >> 1] += pv;
        }
    }

    // ---- O += P V: 4 key steps x KSTEPS dim steps, one ldmatrix and two products each, fetched two steps ahead ----
    {
        unsigned pa[4][4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            pa[ks][0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pa[ks][1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pa[ks][2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[ks][3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
        }
        unsigned vaddr[T::NOFF];
#pragma unroll
        for (int j = 0; j < T::NOFF; ++j) vaddr[j] = sV + f.v[j];
        constexpr int TOTAL = 4 * KSTEPS, AHEAD = PIPE ? 2 : 0;
        unsigned vb[PIPE ? 3 : 1][4];
        auto fetch_v = [&](auto t_c) {
            constexpr int t = decltype(t_c)::value;
            constexpr int ks = t / KSTEPS, d2 = t % KSTEPS;
            if (BULK || d2 * 16 < d)
                ldsm_x4_trans<step_imm<DMAX, BULK, d2>() + ks * 16 * T::ROW_BYTES>(vb[PIPE ? t % 3 : 0], vaddr[BULK ? (d2 & 3) : 0]);
        };
        static_for<0, AHEAD>([&](auto t_c) { fetch_v(t_c); });
        static_for<0, TOTAL>([&](auto t_c) {
            constexpr int t = decltype(t_c)::value;
            constexpr int ks = t / KSTEPS, d2 = t % KSTEPS;
            if constexpr (t + AHEAD < TOTAL || AHEAD == 0) fetch_v(std::integral_constant<int, t + AHEAD>{});
            if (BULK || d2 * 16 < d) {
                constexpr int b = PIPE ? t % 3 : 0;
                mma_bf16_free(o[2 * d2], pa[ks], vb[b][0], vb[b][1]);
                mma_bf16_free(o[2 * d2 + 1], pa[ks], vb[b][2], vb[b][3]);
            }
        });
    }
}


static inline int attn_check_common(const char* name, const AttnParams& p) {
    PB_REQUIRE(p.n_heads > 0 && p.n_kv_heads > 0 && p.n_heads % p.n_kv_heads == 0,
               "%s: %d query heads over %d key/value heads", name, p.n_heads, p.n_kv_heads);
    PB_REQUIRE(p.head_dim >= 16 && p.head_dim <= 256 && p.head_dim % 16 == 0,
               "%s: head_dim=%d; the tensor-core kernels take multiples of 16 up to 256", name, p.head_dim);
    PB_REQUIRE(p.page_size > 0 && p.num_pages > 0 && p.table_stride > 0, "%s: bad cache geometry", name);
    PB_REQUIRE(pb_aligned(p.q, 16) && pb_aligned(p.k_pages, 16) && pb_aligned(p.v_pages, 16) && pb_aligned(p.out, 4),
               "%s: q and the pages must be 16-byte aligned", name);
    return 0;
}

