// Token selection from float32 logits: argmax and temperature sampling.
//
// Greedy: the largest logit, ties to the smaller index
// (crates/prelude-cuda/src/kernels/kernels_src/sample/fast_argmax_vocab.cu:15-16,43).
// Temperature: p = softmax(logits / T) in float32, then one multinomial draw
// (crates/prelude-core/src/engine/sampling/logits_processor.rs:100-110); a
// temperature below 1e-7 means greedy (same file, line 31).  The reference
// draws on the host from a seeded generator; here the draw is made on the
// device from Philox4x32-10 keyed by the request's seed with the request's
// step as counter, and the token is the first index whose cumulative
// probability, summed in index order, exceeds u * total.
//
// One block per row.
#include "common.cuh"

#include <math.h>

#define SAMP_THREADS 1024

struct ArgPair {
    float v;
    int i;
};
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgPair block_argmax(const float* __restrict__ row, int vocab, ArgPair* smem) {
    ArgPair best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = row[i];
        if (v > best.v || (v == best.v && i < best.i)) best = ArgPair{v, i};   // NaN never wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) smem[warp] = best;
    __syncthreads();
    ArgPair r = smem[0];
    for (int w = 1; w < nwarp; ++w) r = better(r, smem[w]);
    __syncthreads();
    if (r.i == 0x7fffffff) r.i = 0;   // a row of NaN or -inf
    return r;
}

__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* __restrict__ logits, long long row_stride,
                                                               int vocab, int32_t* __restrict__ out) {
    __shared__ ArgPair smem[32];
    ArgPair r = block_argmax(logits + (size_t)blockIdx.x * row_stride, vocab, smem);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

PB_API int pb_argmax(const float* logits, long long row_stride, int rows, int vocab, int32_t* out,
                     cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
    if (rows == 0) return 0;
    argmax_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, row_stride, vocab, out);
    PB_CHECK_LAUNCH("argmax");
    return 0;
}

// ---------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")
// ---------------------------------------------------------------------------
__host__ __device__ inline void philox4x32_10(uint32_t key0, uint32_t key1, uint32_t c[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)M0 * c[0], p1 = (uint64_t)M1 * c[2];
        uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
        uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
        uint32_t n0 = hi1 ^ c[1] ^ key0, n1 = lo1, n2 = hi0 ^ c[3] ^ key1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        key0 += W0; key1 += W1;
    }
}

// uniform in [0, 1) with 24 bits
__host__ __device__ inline float philox_uniform(uint64_t seed, uint64_t counter) {
    uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u};
    philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), c);
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

// For tests: the uniform number the sampler uses for (seed, counter).
PB_API float pb_philox_uniform(uint64_t seed, uint64_t counter) { return philox_uniform(seed, counter); }

__global__ void __launch_bounds__(SAMP_THREADS) sample_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ counters, int32_t* __restrict__ out) {
    __shared__ ArgPair smem[32];
    __shared__ float sums[SAMP_THREADS];
    __shared__ int winner;
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    const float temp = temperature[blockIdx.x];
    ArgPair top = block_argmax(row, vocab, smem);
    if (!(temp >= 1e-7f)) {
        if (threadIdx.x == 0) out[blockIdx.x] = top.i;
        return;
    }
    const float inv_t = 1.0f / temp;
    // contiguous chunk per thread, so that the cumulative sum runs in index order
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
    float local = 0.f;
    for (int i = begin; i < end; ++i) local += expf((row[i] - top.v) * inv_t);
    sums[threadIdx.x] = local;
    if (threadIdx.x == 0) winner = -1;
    __syncthreads();
    // inclusive scan over the per-thread sums (Hillis-Steele)
    for (int off = 1; off < blockDim.x; off <<= 1) {
        float add = threadIdx.x >= off ? sums[threadIdx.x - off] : 0.f;
        __syncthreads();
        sums[threadIdx.x] += add;
        __syncthreads();
    }
    const float total = sums[blockDim.x - 1];
    const float u = philox_uniform(seeds[blockIdx.x], counters[blockIdx.x]);
    const float target = u * total;
    const float incl = sums[threadIdx.x];
    const float excl = threadIdx.x == 0 ? 0.f : sums[threadIdx.x - 1];
    if (begin < end && excl <= target && target < incl) {
        // this thread's chunk holds the draw: walk it
        float run = excl;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((row[i] - top.v) * inv_t);
            if (target < run) { pick = i; break; }
        }
        atomicMax(&winner, pick);   // exactly one thread satisfies the test
    }
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = winner >= 0 ? winner : top.i;   // rounding at the far end: most likely token
}

PB_API int pb_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                     const uint64_t* seeds, const uint64_t* counters, int32_t* out, cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    PB_REQUIRE(logits && temperature && seeds && counters && out, "sample: null pointer");
    if (rows == 0) return 0;
    sample_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, row_stride, vocab, temperature, seeds, counters, out);
    PB_CHECK_LAUNCH("sample");
    return 0;
}

// probs[r, :] = softmax(logits[r, :] / T_r), for the host-side top-k / top-p draw.
__global__ void __launch_bounds__(SAMP_THREADS) softmax_temperature_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    float* __restrict__ probs) {
    __shared__ ArgPair smem[32];
    __shared__ float red[32];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    float* prow = probs + (size_t)blockIdx.x * vocab;
    ArgPair top = block_argmax(row, vocab, smem);
    const float inv_t = 1.0f / fmaxf(temperature[blockIdx.x], 1e-7f);
    float local = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float e = expf((row[i] - top.v) * inv_t);
        prow[i] = e;
        local += e;
    }
    local = pb_warp_sum(local);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += red[w];
    const float inv = 1.0f / total;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) prow[i] *= inv;
}

PB_API int pb_softmax_temperature(const float* logits, long long row_stride, int rows, int vocab,
                                  const float* temperature, float* probs, cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "softmax_temperature: bad sizes");
    if (rows == 0) return 0;
    softmax_temperature_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, row_stride, vocab, temperature, probs);
    PB_CHECK_LAUNCH("softmax_temperature");
    return 0;
}
