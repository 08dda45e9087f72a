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
// Two passes.  The first cuts every row into chunks of a few thousand logits, one
// block each: the chunk's maximum, its first index, and (when the row samples)
// the chunk's sum of exp((x - chunk max) / T).  The second, one block per row,
// combines the chunks in index order, and for a sampling row finds the chunk the
// draw falls into and walks that chunk alone.
#include "common.cuh"

#include <math.h>
#include <mutex>

#define SAMP_THREADS 1024
#define PART_THREADS 256
#define PART_CHUNK 4096
#define PART_MAX_BLOCKS 64

struct ArgPair {
    float v;
    int i;
};
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// Largest value and its first index over row[begin, end); every thread gets the result.
__device__ ArgPair block_argmax(const float* __restrict__ row, int begin, int end, ArgPair* smem) {
    ArgPair best{-INFINITY, 0x7fffffff};
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
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
    return r;
}

__device__ float block_sum_ordered(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += smem[w];
    __syncthreads();
    return total;
}

static int part_blocks(int vocab) {
    int n = (vocab + PART_CHUNK - 1) / PART_CHUNK;
    return n < 1 ? 1 : (n > PART_MAX_BLOCKS ? PART_MAX_BLOCKS : n);
}

// Floats of scratch that argmax and sample need for `rows` rows of `vocab` logits.
PB_API long long pb_sample_scratch_floats(int rows, int vocab) { return (long long)rows * part_blocks(vocab) * 4; }

// pass 1: grid (chunks, rows).  part[row][chunk] = {max, first index (int bits), sum of exp((x - max) / T), unused}
__global__ void __launch_bounds__(PART_THREADS) sample_partial_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    float* __restrict__ part) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ ArgPair smem[32];
    __shared__ float red[32];
    const int nblk = gridDim.x, b = blockIdx.x, r = blockIdx.y;
    const int chunk = (vocab + nblk - 1) / nblk;
    const int begin = min(vocab, b * chunk), end = min(vocab, begin + chunk);
    const float* row = logits + (size_t)r * row_stride;
    ArgPair top = block_argmax(row, begin, end, smem);
    float sum = 0.f;
    const float temp = temperature ? temperature[r] : 0.f;
    if (temp >= 1e-7f && top.v > -INFINITY) {
        const float inv_t = 1.0f / temp;
        float local = 0.f;
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) local += expf((row[i] - top.v) * inv_t);
        sum = block_sum_ordered(local, red);
    }
    if (threadIdx.x == 0) {
        float* o = part + ((size_t)r * nblk + b) * 4;
        o[0] = top.v;
        o[1] = __int_as_float(top.i);
        o[2] = sum;
    }
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

// pass 2: one block per row
__global__ void __launch_bounds__(PART_THREADS) sample_final_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ counters, const float* __restrict__ part,
    int nblk, int32_t* __restrict__ out) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float sums[PART_THREADS];
    __shared__ float s_top, s_target;
    __shared__ int s_chunk, s_best, s_winner;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float* pr = part + (size_t)r * nblk * 4;
    const float temp = temperature ? temperature[r] : 0.f;
    const bool greedy = !(temp >= 1e-7f);
    const float inv_t = greedy ? 0.f : 1.0f / temp;
    if (threadIdx.x == 0) {
        ArgPair best{-INFINITY, 0x7fffffff};
        for (int b = 0; b < nblk; ++b) best = better(best, ArgPair{pr[4 * b], __float_as_int(pr[4 * b + 1])});
        if (best.i == 0x7fffffff) best.i = 0;               // a row of NaN or -inf
        s_best = best.i;
        s_top = best.v;
        s_chunk = -1;
        s_winner = -1;
        if (!greedy && best.v > -INFINITY) {
            float total = 0.f;
            for (int b = 0; b < nblk; ++b) total += pr[4 * b + 2] * expf((pr[4 * b] - best.v) * inv_t);
            const float target = philox_uniform(seeds[r], counters[r]) * total;
            float run = 0.f;
            for (int b = 0; b < nblk; ++b) {
                const float w = pr[4 * b + 2] * expf((pr[4 * b] - best.v) * inv_t);
                if (target < run + w) { s_chunk = b; s_target = target - run; break; }
                run += w;
            }
        }
    }
    __syncthreads();
    if (s_chunk < 0) {                                      // greedy, or rounding at the far end: the most likely token
        if (threadIdx.x == 0) out[r] = s_best;
        return;
    }
    // walk the chunk that holds the draw: contiguous pieces per thread, cumulative sum in index order
    const int chunk = (vocab + nblk - 1) / nblk;
    const int cb = min(vocab, s_chunk * chunk), ce = min(vocab, cb + chunk);
    const int piece = (ce - cb + blockDim.x - 1) / blockDim.x;
    const int begin = min(ce, cb + (int)threadIdx.x * piece), end = min(ce, begin + piece);
    const float top = s_top, target = s_target;
    float local = 0.f;
    for (int i = begin; i < end; ++i) local += expf((row[i] - top) * inv_t);
    sums[threadIdx.x] = local;
    __syncthreads();
    for (int off = 1; off < blockDim.x; off <<= 1) {        // inclusive scan (Hillis-Steele)
        float add = threadIdx.x >= off ? sums[threadIdx.x - off] : 0.f;
        __syncthreads();
        sums[threadIdx.x] += add;
        __syncthreads();
    }
    const float incl = sums[threadIdx.x], excl = threadIdx.x == 0 ? 0.f : sums[threadIdx.x - 1];
    if (begin < end && excl <= target && target < incl) {
        float run = excl;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((row[i] - top) * inv_t);
            if (target < run) { pick = i; break; }
        }
        atomicMax(&s_winner, pick);                         // at most one thread satisfies the test
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int w = s_winner;
        if (w < 0) {                                        // the chunk total and the walk disagree in the last bit: last token with weight
            w = ce - 1;
        }
        out[r] = w;
    }
}

static int launch_two_pass(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                           const uint64_t* seeds, const uint64_t* counters, float* scratch, int32_t* out,
                           cudaStream_t stream) {
    const int nblk = part_blocks(vocab);
    pb_launch(sample_partial_kernel, dim3(nblk, rows), dim3(PART_THREADS), 0, stream, logits, row_stride, vocab, temperature, scratch);
    pb_launch(sample_final_kernel, dim3(rows), dim3(PART_THREADS), 0, stream, logits, row_stride, vocab, temperature, seeds, counters,
                                                           scratch, nblk, out);
    return 0;
}

// scratch: pb_sample_scratch_floats(rows, vocab) floats.
PB_API int pb_argmax(const float* logits, long long row_stride, int rows, int vocab, int32_t* out, float* scratch,
                     cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && rows < 65536 && vocab > 0 && row_stride >= vocab, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
    PB_REQUIRE(logits && out && scratch, "argmax: null pointer");
    if (rows == 0) return 0;
    launch_two_pass(logits, row_stride, rows, vocab, nullptr, nullptr, nullptr, scratch, out, stream);
    PB_CHECK_LAUNCH("argmax");
    return 0;
}

PB_API int pb_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                     const uint64_t* seeds, const uint64_t* counters, int32_t* out, float* scratch,
                     cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && rows < 65536 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    PB_REQUIRE(logits && temperature && seeds && counters && out && scratch, "sample: null pointer");
    if (rows == 0) return 0;
    launch_two_pass(logits, row_stride, rows, vocab, temperature, seeds, counters, scratch, out, stream);
    PB_CHECK_LAUNCH("sample");
    return 0;
}

// probs[r, :] = softmax(logits[r, :] / T_r), for the host-side top-k / top-p draw.
__global__ void __launch_bounds__(SAMP_THREADS) softmax_temperature_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    float* __restrict__ probs) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ ArgPair smem[32];
    __shared__ float red[32];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    float* prow = probs + (size_t)blockIdx.x * vocab;
    ArgPair top = block_argmax(row, 0, vocab, smem);
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
    pb_launch(softmax_temperature_kernel, dim3(rows), dim3(SAMP_THREADS), 0, stream, logits, row_stride, vocab, temperature, probs);
    PB_CHECK_LAUNCH("softmax_temperature");
    return 0;
}

// ---------------------------------------------------------------------------
// Row-wise argmax that brings its own scratch (declared in no_alloc.h).
//
// pb_argmax needs a few floats of scratch per row for its two passes, and its
// callers get them from an allocator.  Some callers have none to ask: a C or
// C++ host that links this library without torch and runs with a fixed memory
// plan, or code that runs where allocation is forbidden (a stream that is being
// captured, a callback on the launch path).  For them the scratch lives in the
// library image: one array per GPU, 256 KB, present from the moment the library
// is loaded on that GPU until the process ends.
//
// Nothing in the array has to start at zero: the first pass writes every slot
// the second pass reads.  All calls share the one array and it keeps what the
// last call left there, so two calls that run on the GPU at the same time (two
// streams, two threads) overwrite each other's partial results; calls on one
// stream are safe.  The first call on a device looks up the array's device
// address (cudaGetSymbolAddress: no allocation, but it may load the module), so
// make that first call before any stream capture begins.
// ---------------------------------------------------------------------------
#define PB_NOALLOC_MAX_ROWS 256
#define PB_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_noalloc_scratch[PB_NOALLOC_MAX_ROWS * PART_MAX_BLOCKS * 4];
static float* g_noalloc_scratch_addr[PB_NOALLOC_MAX_DEVICES] = {nullptr};

PB_API int pb_argmax_noalloc(const float* logits, long long row_stride, int rows, int vocab, int32_t* out,
                             cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "argmax_noalloc: bad sizes rows=%d vocab=%d", rows, vocab);
    PB_REQUIRE(rows <= PB_NOALLOC_MAX_ROWS,
               "argmax_noalloc: rows=%d is more than the %d rows the built-in scratch holds; split the call or use pb_argmax",
               rows, PB_NOALLOC_MAX_ROWS);
    PB_REQUIRE(logits && out, "argmax_noalloc: null pointer");
    if (rows == 0) return 0;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return pb_fail("argmax_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    PB_REQUIRE(dev >= 0 && dev < PB_NOALLOC_MAX_DEVICES, "argmax_noalloc: device %d", dev);
    // The array that is used is the CURRENT device's.  The logits must live there too (and the stream must be one
    // of that device's, which the runtime checks at the launch): another device's array is not this call's to use.
    cudaPointerAttributes where;
    e = cudaPointerGetAttributes(&where, logits);
    if (e != cudaSuccess) return pb_fail("argmax_noalloc: cannot tell where the logits live: %s", cudaGetErrorString(e));
    PB_REQUIRE(where.type != cudaMemoryTypeDevice || where.device == dev,
               "argmax_noalloc: the logits live on device %d, the current device is %d; make the logits' device current first",
               where.device, dev);
    {
        // the first call on a device resolves the address; a lock keeps two threads' first calls apart
        static std::mutex first_call;
        std::lock_guard<std::mutex> hold(first_call);
        if (g_noalloc_scratch_addr[dev] == nullptr) {
            // the array's name is a host-side handle here, not a device address: ask the runtime for the address
            float* addr = nullptr;
            e = cudaGetSymbolAddress((void**)&addr, g_noalloc_scratch);
            if (e != cudaSuccess || addr == nullptr)
                return pb_fail("argmax_noalloc: cannot find the built-in scratch on device %d: %s", dev, cudaGetErrorString(e));
            g_noalloc_scratch_addr[dev] = addr;
        }
    }
    launch_two_pass(logits, row_stride, rows, vocab, nullptr, nullptr, nullptr, g_noalloc_scratch_addr[dev], out, stream);
    PB_CHECK_LAUNCH("argmax_noalloc");
    return 0;
}
