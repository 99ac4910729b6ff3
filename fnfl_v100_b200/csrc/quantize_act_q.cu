// The reference engine's planar 32-value activation, the input of its Q2_0 down rows: per chunk of 32 values
//     s = amax / 127,  inv = 1 / s (both 0 for an all-zero chunk),  code = trunc(x inv +- 0.5) clamped to +-127
// (round half away from zero), codes as int8 [rows][n], scales as F32 [rows][n / 32].  Replaces
// fn::experts::cpu::quantize_act_q (fn/kernels/experts/cpu_kernels.h:45-62; cpu_q2_avx2.cpp:180-226) for its codes and
// scales, bit for bit on finite inputs (its code sums, hx and bit-plane image are derived data the down kernel builds
// for itself).  HBM-bound: 4 bytes read, 1.125 written a value.
#include "common.cuh"

namespace fnb {
namespace {

#ifndef FNB_ACTQ_GRID
#define FNB_ACTQ_GRID 16
#endif
constexpr int kThreads = 256;
constexpr int kGridPerSm = FNB_ACTQ_GRID;

__global__ void __launch_bounds__(kThreads)
    quantize_act_q_kernel(const float * __restrict__ x, int8_t * __restrict__ codes, float * __restrict__ scales, int64_t rows,
                          int n, int64_t x_stride, int64_t codes_stride, int64_t scales_stride) {
    // TWO lanes a chunk: lane j takes the chunk's float4s j, j + 2, j + 4, j + 6 (every load instruction of the pair
    // covers one 32-byte sector), so the two IEEE divisions of a chunk are paid once per 64 bytes a lane loads; with
    // eight lanes a chunk the kernel was bound by instruction issue at 47 % of the HBM roofline
    const int chunks = n / 32;
    const int64_t total = rows * chunks * 2;
    // a warp stays together (the shuffles name all 32 lanes): lanes past the end redo the last chunk and store nothing
    for (int64_t i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x; i0 - (threadIdx.x & 31) < total;
         i0 += int64_t(gridDim.x) * kThreads) {
        const bool live = i0 < total;
        const int64_t i = live ? i0 : total - 2 + (threadIdx.x & 1);
        const int64_t chunk = i >> 1;
        const int j = int(i & 1);
        const int64_t r = chunk / chunks;
        const int c = int(chunk - r * chunks);
        const float4 * src = reinterpret_cast<const float4 *>(x + r * x_stride + 32 * c) + j;
        float4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = ld_stream(src + 2 * q);
        float amax = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[q].x), fabsf(v[q].y)), fmaxf(fabsf(v[q].z), fabsf(v[q].w))));
        }
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
        const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
        const float inv = s > 0.0f ? __fdiv_rn(1.0f, s) : 0.0f;
        const auto code = [inv](float xv) {
            const float t = __fmul_rn(xv, inv);
            const int q = __float2int_rz(__fadd_rn(t, t >= 0.0f ? 0.5f : -0.5f));
            return uint32_t(max(-127, min(127, q)) & 0xff);
        };
        uint32_t w[4];  // code words j, j + 2, j + 4, j + 6 of the chunk's eight
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = code(v[q].x) | (code(v[q].y) << 8) | (code(v[q].z) << 16) | (code(v[q].w) << 24);
        // lane 0 stores words 0 .. 3, lane 1 words 4 .. 7: each hands the other the two it holds of the other's half
        const uint32_t got0 = __shfl_xor_sync(kFull, j == 0 ? w[2] : w[0], 1);
        const uint32_t got1 = __shfl_xor_sync(kFull, j == 0 ? w[3] : w[1], 1);
        const uint4 o = j == 0 ? make_uint4(w[0], got0, w[1], got1) : make_uint4(got0, w[2], got1, w[3]);
        if (live) {
            st_stream(reinterpret_cast<uint4 *>(codes + r * codes_stride + 32 * c) + j, o);
            if (j == 0) scales[r * scales_stride + c] = s;
        }
    }
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_quantize_act_q(const float * x, int8_t * codes, float * scales, int64_t rows, int32_t n, void * stream) {
    using namespace fnb;
    if (!ok_ptr(x, 16) || !ok_ptr(codes, 16) || !ok_ptr(scales, 4)) return FNB_REJECTED;
    if (rows < 1 || rows > INT32_MAX || n < 32 || n > 65536 || n % 32 != 0) return FNB_REJECTED;
    const int64_t threads = rows * (n / 32) * 2;
    const int grid = grid_for((threads + kThreads - 1) / kThreads, kGridPerSm);
    quantize_act_q_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, codes, scales, rows, n, n, n, n / 32);
    return launch_status();
}
