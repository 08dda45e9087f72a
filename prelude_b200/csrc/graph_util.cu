// Small kernels around a captured decode step.
//
// A CUDA graph replays fixed launches on fixed addresses, so everything that
// changes from step to step lives in device buffers that these kernels (and one
// host-to-device copy) update: entries of the device-resident block tables, and,
// for a step that feeds itself, the next token and position of every request.
// The reference keeps fixed-address input buffers per captured batch size for
// the same purpose (crates/prelude-cuda/src/cuda_graph/buffers.rs:12-185).
#include "common.cuh"

// dst[idx[i]] = val[i]; an index outside [0, dst_len) is skipped and raises *status.
__global__ void scatter_i32_kernel(int32_t* __restrict__ dst, long long dst_len, const int32_t* __restrict__ idx,
                                   const int32_t* __restrict__ val, int n, int* __restrict__ status) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    long long at = idx[i];
    if (at < 0 || at >= dst_len) {
        if (status) atomicExch(status, 5);
        return;
    }
    dst[at] = val[i];
}

PB_API int pb_scatter_i32(int32_t* dst, long long dst_len, const int32_t* idx, const int32_t* val, int n, int* status,
                          cudaStream_t stream) {
    PB_REQUIRE(n >= 0 && dst_len >= 0, "scatter_i32: bad sizes");
    if (n == 0) return 0;
    PB_REQUIRE(dst && idx && val, "scatter_i32: null pointer");
    pb_launch(scatter_i32_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, dst, dst_len, idx, val, n, status);
    PB_CHECK_LAUNCH("scatter_i32");
    return 0;
}

// After a decode step: the sampled token becomes the next input, positions and
// sampling counters move on by one (and with them the count of tokens in the cache).  Lets a captured step run again and again
// without the host in between.
__global__ void decode_advance_kernel(int32_t* __restrict__ tokens, int32_t* __restrict__ positions,
                                      int32_t* __restrict__ kv_len, long long* __restrict__ counters,
                                      const int32_t* __restrict__ sampled, int n, int max_positions) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    tokens[i] = sampled[i];
    if (positions[i] + 1 < max_positions) {
        positions[i] += 1;
        if (kv_len) kv_len[i] = positions[i] + 1;          // tokens in the cache after the next step
    }
    if (counters) counters[i] += 1;
}

PB_API int pb_decode_advance(int32_t* tokens, int32_t* positions, int32_t* kv_len, long long* counters,
                             const int32_t* sampled, int n, int max_positions, cudaStream_t stream) {
    PB_REQUIRE(n >= 0 && tokens && positions && sampled, "decode_advance: bad arguments");
    if (n == 0) return 0;
    pb_launch(decode_advance_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, positions, kv_len, counters, sampled, n, max_positions);
    PB_CHECK_LAUNCH("decode_advance");
    return 0;
}
