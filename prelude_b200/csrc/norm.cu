// RMSNorm and fused residual-add + RMSNorm.
//
//   y = x / sqrt(mean(x^2) + eps) * w          (all arithmetic in float32)
//
// The residual stream `res` is float32 in every mode.  The fused form does
//   res += x ;  y = rmsnorm(res) * w
// in one pass over the row, which is the reference's add+norm protocol
// (crates/prelude-core/src/models/commons/linear.rs:471-488; kernels
// crates/prelude-cuda/src/kernels/kernels_src/normalization/rmsnorm.cu:33-51, 230-355)
// with the sum kept in 32-bit instead of being rounded to the model type.
//
// One block per row.  The block size depends on the row width only, so the
// order of the reduction, and with it every bit of the result, is the same
// whatever else is in the batch.
#include "common.cuh"


PB_TIMELINE_UNIT(norm)

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = pb_warp_sum(v);
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < nwarp; ++i) total += smem[i];   // same order in every thread
    __syncthreads();
    return total;
}

template <typename TX, typename TY>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride, float* __restrict__ res,
                                   const float* __restrict__ w, TY* __restrict__ y, int width, float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    size_t row = blockIdx.x;
    float* r = res + row * width;
    TY* out = y + row * width;
    float ss = 0.f;
    if (x != nullptr) {
        const TX* xr = x + row * width;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = r[i];
            for (int s = 0; s < n_parts; ++s) v += pb_ld(xr + s * part_stride + i);     // the parts in ascending order
            r[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = r[i];
            ss += v * v;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, r[i] * inv * w[i]);
}

// Four elements per thread and access, the row kept in registers between the
// two passes.  width % 4 == 0, width <= 4 * blockDim * ITERS.
template <typename TX, typename TY, int ITERS>
__global__ void add_rmsnorm_vec4_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride, float* __restrict__ res,
                                        const float* __restrict__ w, TY* __restrict__ y, int width, float eps) {
    pb_grid_dep_launch();
    PB_TL(PB_TL_NORM, PB_TL_ENTRY);
    __shared__ float red[32];
    size_t row = blockIdx.x;
    float4* r4 = reinterpret_cast<float4*>(res + row * width);
    const int n4 = width >> 2;
    // the scale is written by no kernel: it is fetched while the kernel before this one is still running
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 scale[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) scale[it] = w4[i];
    }
    pb_grid_dep_wait();
    PB_TL(PB_TL_NORM, PB_TL_AFTER_WAIT);
    float4 keep[ITERS];
    float ss = 0.f;
    // Every load of the row is issued before the first sum (up to four parts): the kernel is one round trip to
    // the L2 cache, a reduction and a store, and with the loads of one iteration behind the store of the one
    // before it was three round trips (4.1 us for 8 rows of 2,560 in a decode step).
    float4 part[ITERS][4];
    uint2 raw[ITERS];
    const bool ahead = x != nullptr && (sizeof(TX) == 2 || n_parts <= 4);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            keep[it] = r4[i];
            if (ahead) {
                const TX* xr = x + row * width + 4 * (size_t)i;
                if constexpr (sizeof(TX) == 2) {
                    raw[it] = *reinterpret_cast<const uint2*>(xr);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        part[it][u] = (u < n_parts) ? *reinterpret_cast<const float4*>(xr + (size_t)u * part_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            float4 v = keep[it];
            if (x != nullptr) {
                const TX* xr = x + row * width + 4 * (size_t)i;
                if constexpr (sizeof(TX) == 2) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[it]);
                    float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
                    v.x += a.x; v.y += a.y; v.z += b.x; v.w += b.y;
                } else if (ahead) {
                    // the parts in ascending order
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (u < n_parts) { v.x += part[it][u].x; v.y += part[it][u].y; v.z += part[it][u].z; v.w += part[it][u].w; }
                } else {
                    // the parts in ascending order, four loads in flight at a time
                    for (int s0 = 0; s0 < n_parts; s0 += 4) {
                        float4 a[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            a[u] = (s0 + u < n_parts) ? *reinterpret_cast<const float4*>(xr + (size_t)(s0 + u) * part_stride)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (s0 + u < n_parts) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
                    }
                }
                r4[i] = v;
            }
            keep[it] = v;
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        int i = threadIdx.x + it * blockDim.x;
        if (i < n4) {
            float4 v = keep[it], g = scale[it];
            float o0 = v.x * inv * g.x, o1 = v.y * inv * g.y, o2 = v.z * inv * g.z, o3 = v.w * inv * g.w;
            TY* out = y + row * width + 4 * (size_t)i;
            if constexpr (sizeof(TY) == 2) {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
                uint2 raw;
                raw.x = *reinterpret_cast<uint32_t*>(&p0);
                raw.y = *reinterpret_cast<uint32_t*>(&p1);
                *reinterpret_cast<uint2*>(out) = raw;
            } else {
                *reinterpret_cast<float4*>(out) = make_float4(o0, o1, o2, o3);
            }
        }
    }
    PB_TL(PB_TL_NORM, PB_TL_DONE);
}

static int norm_threads(int width) {
    if (width <= 64) return 32;
    if (width <= 512) return 64;
    if (width <= 2048) return 128;
    return 256;
}

template <typename TX, typename TY>
static int launch_add_rmsnorm(const void* x, int n_parts, size_t part_stride, float* res, const float* w, void* y, int rows,
                              int width, float eps, cudaStream_t stream) {
    int threads = norm_threads(width);
    bool vec = width % 4 == 0 && pb_aligned(res, 16) && pb_aligned(w, 16) && pb_aligned(y, 8 * sizeof(TY) / 2) &&
               (x == nullptr || (pb_aligned(x, 8 * sizeof(TX) / 2) && part_stride % 4 == 0)) && width <= 4 * threads * 8;
    if (vec) {
        int iters = (width / 4 + threads - 1) / threads;
        if (iters <= 2)
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 2>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps);
        else if (iters <= 4)
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 4>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps);
        else
            pb_launch(add_rmsnorm_vec4_kernel<TX, TY, 8>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps);
    } else {
        pb_launch(add_rmsnorm_kernel<TX, TY>, dim3(rows), dim3(threads), 0, stream, (const TX*)x, n_parts, part_stride, res, w, (TY*)y, width, eps);
    }
    return 0;
}

// res[rows, width] float32 (updated in place when x is given); x may be null
// (no add); w float32 [width]; y [rows, width] of type dtype.  x has type dtype,
// or, with x_parts > 0, it is x_parts float32 arrays [rows, width], part_stride
// elements apart, whose sum is what is added (the partial sums of a product
// whose K was cut into parts).
PB_API int pb_add_rmsnorm(const void* x, int x_parts, long long part_stride, float* res, const float* w, void* y, int dtype,
                          int rows, int width, float eps, cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && width > 0, "add_rmsnorm: bad sizes rows=%d width=%d", rows, width);
    PB_REQUIRE(res && w && y, "add_rmsnorm: null pointer");
    PB_REQUIRE(x_parts >= 0 && x_parts <= 64 && (x_parts == 0 || (x && part_stride >= (long long)rows * width)),
               "add_rmsnorm: %d parts %lld apart", x_parts, part_stride);
    if (rows == 0) return 0;
    if (x_parts > 0) {
        PB_DISPATCH_DTYPE(dtype, T, (launch_add_rmsnorm<float, T>(x, x_parts, (size_t)part_stride, res, w, y, rows, width, eps, stream)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T, (launch_add_rmsnorm<T, T>(x, 1, 0, res, w, y, rows, width, eps, stream)));
    }
    PB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// Final norm on chosen rows only: y[i] = rmsnorm(res[rows[i]] + x[rows[i]]) * w.
// The residual stream is left as it is; only the rows whose logits are wanted
// are normalised (the reference selects the last row of each request after the
// final norm, crates/prelude-core/src/models/commons/mod.rs:227-243; the order
// does not change the values).
template <typename TX, typename TY>
__global__ void gather_add_rmsnorm_kernel(const TX* __restrict__ x, int n_parts, size_t part_stride,
                                          const float* __restrict__ res, const int32_t* __restrict__ rows,
                                          const float* __restrict__ w, TY* __restrict__ y, int width, int n_rows_total,
                                          float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    const int src = rows[blockIdx.x];
    TY* out = y + (size_t)blockIdx.x * width;
    if (src < 0 || src >= n_rows_total) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, 0.f);
        return;
    }
    const float* r = res + (size_t)src * width;
    const TX* xr = x ? x + (size_t)src * width : nullptr;
    auto value = [&](int i) {
        float v = r[i];
        if (xr) for (int s = 0; s < n_parts; ++s) v += pb_ld(xr + s * part_stride + i);   // the parts in ascending order
        return v;
    };
    // a thread's elements stay in registers between the two passes where the row is short enough (16 per thread:
    // rows of up to 4,096 at 256 threads); the loads of the first pass are independent of one another
    constexpr int KEEP = 16;
    float kept[KEEP];
    const bool fits = width <= KEEP * (int)blockDim.x;
    float ss = 0.f;
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            kept[k] = i < width ? value(i) : 0.f;
            ss += kept[k] * kept[k];
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = value(i);
            ss += v * v;
        }
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    if (fits) {
#pragma unroll
        for (int k = 0; k < KEEP; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) pb_st(out + i, kept[k] * inv * w[i]);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(out + i, value(i) * inv * w[i]);
    }
}

// x as for pb_add_rmsnorm: of type dtype, or x_parts float32 arrays to be added up.
PB_API int pb_gather_add_rmsnorm(const void* x, int x_parts, long long part_stride, const float* res, const int32_t* rows,
                                 const float* w, void* y, int dtype, int n_out, int n_rows_total, int width, float eps,
                                 cudaStream_t stream) {
    PB_REQUIRE(n_out >= 0 && width > 0 && n_rows_total >= 0, "gather_add_rmsnorm: bad sizes");
    PB_REQUIRE(res && rows && w && y, "gather_add_rmsnorm: null pointer");
    PB_REQUIRE(x_parts >= 0 && x_parts <= 64 && (x_parts == 0 || (x && part_stride >= (long long)n_rows_total * width)),
               "gather_add_rmsnorm: %d parts %lld apart", x_parts, part_stride);
    if (n_out == 0) return 0;
    if (x_parts > 0) {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(gather_add_rmsnorm_kernel<float, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream,
                (const float*)x, x_parts, (size_t)part_stride, res, rows, w, (T*)y, width, n_rows_total, eps)));
    } else {
        PB_DISPATCH_DTYPE(dtype, T,
            (pb_launch(gather_add_rmsnorm_kernel<T, T>, dim3(n_out), dim3(norm_threads(width)), 0, stream,
                (const T*)x, 1, (size_t)0, res, rows, w, (T*)y, width, n_rows_total, eps)));
    }
    PB_CHECK_LAUNCH("gather_add_rmsnorm");
    return 0;
}

// Plain norm of a tensor of the model's own type (used by parts that are not
// on the residual stream, and by the per-kernel tests).
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y, int width,
                               float eps) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float red[32];
    size_t row = blockIdx.x;
    const T* xr = x + row * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = pb_ld(xr + i);
        ss += v * v;
    }
    float total = block_sum(ss, red);
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) pb_st(y + row * width + i, pb_ld(xr + i) * inv * w[i]);
}

PB_API int pb_rmsnorm(const void* x, const float* w, void* y, int dtype, int rows, int width, float eps,
                      cudaStream_t stream) {
    PB_REQUIRE(rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", rows, width);
    PB_REQUIRE(x && w && y, "rmsnorm: null pointer");
    if (rows == 0) return 0;
    PB_DISPATCH_DTYPE(dtype, T,
        (pb_launch(rmsnorm_kernel<T>, dim3(rows), dim3(norm_threads(width)), 0, stream, (const T*)x, w, (T*)y, width, eps)));
    PB_CHECK_LAUNCH("rmsnorm");
    return 0;
}
