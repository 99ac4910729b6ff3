// The reference engine's planar 32-value activation, the input of its Q2_0 down rows: per chunk of 32 values
//     s = amax / 127,  inv = 1 / s (both 0 for an all-zero chunk),  code = trunc(x inv +- 0.5) clamped to +-127
// (round half away from zero), codes as int8 [rows][n], scales as F32 [rows][n / 32].  Replaces
// fn::experts::cpu::quantize_act_q (fn/kernels/experts/cpu_kernels.h:45-62; cpu_q2_avx2.cpp:180-226) for its codes and
// scales, bit for bit on finite inputs (its code sums, hx and bit-plane image are derived data the down kernel builds
// for itself).  HBM-bound: 4 bytes read, 1.125 written a value; eight lanes a chunk, a float4 each.
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
    quantize_act_q_kernel(const float * __restrict__ x, int8_t * __restrict__ codes, float * __restrict__ scales, int64_t rows,
                          int n, int64_t x_stride, int64_t codes_stride, int64_t scales_stride) {
    const int chunks = n / 32;
    const int64_t total = rows * chunks * 8;  // a float4 per thread
    // a warp stays together (the shuffles name all 32 lanes): lanes past the end redo the last part and store nothing
    for (int64_t i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x; i0 - (threadIdx.x & 31) < total;
         i0 += int64_t(gridDim.x) * kThreads) {
        const bool live = i0 < total;
        const int64_t i = live ? i0 : total - 8 + (threadIdx.x & 7);
        const int64_t chunk = i >> 3;
        const int part = int(i & 7);
        const int64_t r = chunk / chunks;
        const int c = int(chunk - r * chunks);
        const float4 v = ld_stream(reinterpret_cast<const float4 *>(x + r * x_stride + 32 * c) + part);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 4));
        const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
        const float inv = s > 0.0f ? __fdiv_rn(1.0f, s) : 0.0f;
        const auto code = [inv](float xv) {
            const float t = __fmul_rn(xv, inv);
            const int q = __float2int_rz(__fadd_rn(t, t >= 0.0f ? 0.5f : -0.5f));
            return max(-127, min(127, q));
        };
        const uint32_t w = uint32_t(code(v.x) & 0xff) | (uint32_t(code(v.y) & 0xff) << 8) | (uint32_t(code(v.z) & 0xff) << 16) |
                           (uint32_t(code(v.w) & 0xff) << 24);
        if (live) {
            reinterpret_cast<uint32_t *>(codes + r * codes_stride + 32 * c)[part] = w;
            if (part == 0) scales[r * scales_stride + c] = s;
        }
    }
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_quantize_act_q(const float * x, int8_t * codes, float * scales, int64_t rows, int32_t n, void * stream) {
    using namespace fnb;
    if (!ok_ptr(x, 16) || !ok_ptr(codes, 16) || !ok_ptr(scales, 4)) return FNB_REJECTED;
    if (rows < 1 || rows > INT32_MAX || n < 32 || n > 65536 || n % 32 != 0) return FNB_REJECTED;
    const int64_t threads = rows * (n / 32) * 8;
    const int grid = grid_for((threads + kThreads - 1) / kThreads, 16);
    quantize_act_q_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, codes, scales, rows, n, n, n, n / 32);
    return launch_status();
}
