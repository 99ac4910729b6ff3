// RMSNorm over rows: y = (x * scale) * w, scale = 1 / sqrtf(mean(x^2) + eps).
//
// HBM-bound: 8 bytes of traffic per value (4 read, 4 written), about 4 flops.  Layout in HBM: x and y are
// dense F32 [rows][cols]; w is [cols] and lives in L1/L2 after the first row.
//
// Fast path (cols = 128 * V, V <= 32): one warp owns a row and holds all of it in registers - V 128-bit loads
// per lane issued back to back (the whole row is in flight at once: 8 KiB per warp at cols = 2048), one pass
// over HBM, the sum of squares reduced by warp shuffles in double (the CPU definition accumulates F32 squares
// in a double; a double tree sum differs from its sequential sum only below 2^-50 relative, far inside the
// narrowing to F32), then V 128-bit streaming stores.  No shared memory, no block barrier.
// Narrow rows (per-head norm, cols = 256) give a lane only two loads, so a warp takes several rows per trip
// to keep the same number of bytes in flight.
// Generic path (any cols that is a multiple of 4): one CTA per row, two passes, the second served by L2.
#include "common.cuh"
#include "norm_math.cuh"

namespace fnb {
namespace {

// V vectors per lane per row, R rows per warp per trip
template <int V, int R>
__global__ void __launch_bounds__(128) rms_norm_warp_kernel(const float * __restrict__ x, const float * __restrict__ w,
                                                            float eps, float * __restrict__ y, int64_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int cols = 128 * V;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const float4 * w4 = reinterpret_cast<const float4 *>(w);

    for (int64_t r0 = warp * R; r0 < rows; r0 += n_warps * R) {
        float4 v[R][V];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const bool live = r0 + r < rows;
            const float4 * src = reinterpret_cast<const float4 *>(x + (r0 + (live ? r : 0)) * cols);
#pragma unroll
            for (int i = 0; i < V; ++i) v[r][i] = ld_stream(src + i * 32 + lane);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            double acc = 0.0;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                acc = sq_acc(acc, v[r][i].x);
                acc = sq_acc(acc, v[r][i].y);
                acc = sq_acc(acc, v[r][i].z);
                acc = sq_acc(acc, v[r][i].w);
            }
            const float scale = norm_scale(warp_sum_f64(acc), cols, eps);
            if (r0 + r < rows) {
                float4 * dst = reinterpret_cast<float4 *>(y + (r0 + r) * cols);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    float4 o = v[r][i];
                    o.x = __fmul_rn(o.x, scale);
                    o.y = __fmul_rn(o.y, scale);
                    o.z = __fmul_rn(o.z, scale);
                    o.w = __fmul_rn(o.w, scale);
                    if (w != nullptr) {
                        const float4 g = __ldg(w4 + i * 32 + lane);
                        o.x = __fmul_rn(o.x, g.x);
                        o.y = __fmul_rn(o.y, g.y);
                        o.z = __fmul_rn(o.z, g.z);
                        o.w = __fmul_rn(o.w, g.w);
                    }
                    st_stream(dst + i * 32 + lane, o);
                }
            }
        }
    }
}

// any cols % 4 == 0: CTA per row, pass 1 sums, pass 2 (L2-resident) scales
__global__ void __launch_bounds__(256) rms_norm_generic_kernel(const float * __restrict__ x, const float * __restrict__ w,
                                                               float eps, float * __restrict__ y, int64_t rows,
                                                               int cols) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ double part[8];
    __shared__ float s_scale;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int n4 = cols >> 2;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float4 * src = reinterpret_cast<const float4 *>(x + r * cols);
        double acc = 0.0;
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = __ldg(src + i);
            acc = sq_acc(acc, v.x);
            acc = sq_acc(acc, v.y);
            acc = sq_acc(acc, v.z);
            acc = sq_acc(acc, v.w);
        }
        acc = warp_sum_f64(acc);
        if (lane == 0) part[wid] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double s = 0.0;
            for (int i = 0; i < 8; ++i) s = __dadd_rn(s, part[i]);
            s_scale = norm_scale(s, cols, eps);
        }
        __syncthreads();
        const float scale = s_scale;
        float4 * dst = reinterpret_cast<float4 *>(y + r * cols);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            float4 o = __ldg(src + i);
            o.x = __fmul_rn(o.x, scale);
            o.y = __fmul_rn(o.y, scale);
            o.z = __fmul_rn(o.z, scale);
            o.w = __fmul_rn(o.w, scale);
            if (w != nullptr) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + i);
                o.x = __fmul_rn(o.x, g.x);
                o.y = __fmul_rn(o.y, g.y);
                o.z = __fmul_rn(o.z, g.z);
                o.w = __fmul_rn(o.w, g.w);
            }
            st_stream(dst + i, o);
        }
        __syncthreads();
    }
}

template <int V, int R>
void launch_warp(const float * x, const float * w, float eps, float * y, int64_t rows, cudaStream_t s) {
    const int64_t warps_needed = (rows + R - 1) / R;
    const int64_t ctas = (warps_needed + 3) / 4;
    // register-resident rows: occupancy is register-bound, 16 CTAs of 4 warps is an upper bound per SM
    const int grid = grid_for(ctas, 16);
    launch_pdl(rms_norm_warp_kernel<V, R>, grid, 128, 0, s, x, w, eps, y, rows);
}

}  // namespace

int32_t rms_norm_launch(const float * x, const float * w, float eps, float * y, int64_t rows, int32_t cols,
                        cudaStream_t s) {
    if (!ok_ptr(x, 16) || !ok_ptr(y, 16) || !ok_opt(w, 16)) return FNB_REJECTED;
    if (rows < 1 || rows > INT32_MAX || cols < 4 || cols > 65536 || cols % 4 != 0) return FNB_REJECTED;
    if (!(eps >= 0.0f)) return FNB_REJECTED;
    switch (cols) {
        case 128: launch_warp<1, 8>(x, w, eps, y, rows, s); break;
        case 256: launch_warp<2, 4>(x, w, eps, y, rows, s); break;
        case 512: launch_warp<4, 2>(x, w, eps, y, rows, s); break;
        case 1024: launch_warp<8, 2>(x, w, eps, y, rows, s); break;
        case 2048: launch_warp<16, 1>(x, w, eps, y, rows, s); break;
        case 2560: launch_warp<20, 1>(x, w, eps, y, rows, s); break;
        case 4096: launch_warp<32, 1>(x, w, eps, y, rows, s); break;
        default:
            rms_norm_generic_kernel<<<grid_for(rows, 8), 256, 0, s>>>(x, w, eps, y, rows, cols);
            break;
    }
    return launch_status();
}

}  // namespace fnb

extern "C" int32_t fnb_rms_norm_f32(const float * x, const float * w, float eps, float * y, int64_t rows,
                                    int32_t cols, void * stream) {
    return fnb::rms_norm_launch(x, w, eps, y, rows, cols, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_rms_norm_heads_f32(const float * x, const float * w, float eps, float * y, int64_t rows,
                                          int32_t n_heads, int32_t head_dim, void * stream) {
    if (n_heads < 1 || n_heads > 1024 || rows < 1 || rows > INT32_MAX / n_heads) return FNB_REJECTED;
    return fnb::rms_norm_launch(x, w, eps, y, rows * n_heads, head_dim, static_cast<cudaStream_t>(stream));
}
