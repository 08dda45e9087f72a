// Helpers shared by the tensor-core attention kernels: asynchronous 16-byte copies,
// ldmatrix, the bfloat16 mma, the parameter block and the page-gathering tile load.
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

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// the same product without `volatile`: the compiler may move it among the loads around it
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

// One tile of BN keys and values of one key/value head into shared memory;
// rows outside [kv_begin, kv_end) (and rows whose page id is bad) are zero-filled.
// Pages below kv_begin may have been given back already and are never looked up.
template <int DMAX>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV, const AttnParams& p,
                                             const int32_t* table, int kvh, int key0, int kv_begin, int kv_end) {
    constexpr int STRIDE = DMAX + 8;
    const int chunks = p.head_dim >> 3;                    // 16-byte chunks in a row
    const int total = BN * chunks;
    for (int c = threadIdx.x; c < total; c += ATT_THREADS) {
        const int row = c / chunks, ch = c - row * chunks;
        const int j = key0 + row;
        bool ok = j >= kv_begin && j < kv_end;
        size_t src = 0;
        if (ok) {
            const int page = table[j / p.page_size];
            if (page < 0 || page >= p.num_pages) {
                ok = false;
                if (p.status) atomicExch(p.status, 6);
            } else {
                const int in_page = j % p.page_size;
                src = (((size_t)page * p.n_kv_heads + kvh) * p.page_size + in_page) * p.head_dim + (p.swizzle ? ((ch ^ (in_page & 7)) * 8) : ch * 8);
            }
        }
        cp_async16(sK + row * STRIDE + ch * 8, p.k_pages + src, ok);
        cp_async16(sV + row * STRIDE + ch * 8, p.v_pages + src, ok);
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

// Prompt portions (and any mix of portions and single tokens).  Tiles are listed by the host:
