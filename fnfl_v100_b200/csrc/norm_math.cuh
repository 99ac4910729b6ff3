// The two scalar steps of RMSNorm every kernel that normalises a row shares, so that all of them give the same bits:
// F32 squares accumulated in double, and scale = 1 / sqrtf(float(sum / cols) + eps).
#pragma once

#include "common.cuh"

namespace fnb {

__device__ __forceinline__ float norm_scale(double sum, int cols, float eps) {
    // sum / cols; for a power-of-two cols the product with the exact reciprocal is the same double and much cheaper
    const double m = (cols & (cols - 1)) == 0 ? __dmul_rn(sum, 1.0 / double(cols)) : __ddiv_rn(sum, double(cols));
    const float mean = __double2float_rn(m);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

__device__ __forceinline__ double sq_acc(double acc, float v) { return __dadd_rn(acc, double(__fmul_rn(v, v))); }

// declared here for the launchers that fall back on the stand-alone kernel (rms_norm.cu)
int32_t rms_norm_launch(const float * x, const float * w, float eps, float * y, int64_t rows, int32_t cols, cudaStream_t s);

}  // namespace fnb
