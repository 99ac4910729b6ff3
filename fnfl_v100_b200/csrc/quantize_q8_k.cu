// F32 rows -> ggml Q8_K activation blocks (292 bytes per 256 values: F32 d, 256 int8 codes, 16 int16 sums of 16 codes),
// the format the routed experts' gate / up mat-vec reads on the reference's CPU tier (block_q8_k,
// fn/kernels/experts/cpu_kernels.h; produced there by fn::experts::cpu::quantize_q8_k, experts_cpu.cpp:321).
// Bit-identical to ggml's quantize_row_q8_K_ref (ggml/src/ggml-quants.c:2844-2881) and to the reference's AVX2 form:
// the value of largest magnitude - the FIRST one on ties - maps to -127 (iscale = -127 / max), codes are
// nearest-even(iscale x) by the 1.5 x 2^23 trick capped at 127, d = 1 / iscale.  An all-zero block is written as d = 0,
// zero codes and zero sums (the reference leaves the sums of such a block untouched).
// HBM-bound, 4 bytes read and 1.14 written per value: a warp takes a block, a lane eight consecutive values.
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarps = 8;

__global__ void __launch_bounds__(kWarps * 32) quantize_q8_k_kernel(const float * __restrict__ x, uint32_t * __restrict__ out,
                                                                   int64_t n_blocks) {
    __shared__ __align__(16) uint32_t s_blk[kWarps][76];  // 73 words per block
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp = int64_t(blockIdx.x) * kWarps + wid, n_warps = int64_t(gridDim.x) * kWarps;
    uint32_t * mine = s_blk[wid];
    for (int64_t blk = warp; blk < n_blocks; blk += n_warps) {
        const float4 * src = reinterpret_cast<const float4 *>(x + blk * 256) + 2 * lane;
        const float4 a = ld_stream(src), b = ld_stream(src + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        // largest magnitude and the value that has it, first occurrence: in-lane in index order, then across lanes with
        // the lower lane (lower indices) winning ties
        float amax = 0.0f, mx = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float ax = fabsf(v[j]);
            if (ax > amax) amax = ax, mx = v[j];
        }
        int from = lane;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const float oa = __shfl_xor_sync(kFull, amax, m), om = __shfl_xor_sync(kFull, mx, m);
            const int of = __shfl_xor_sync(kFull, from, m);
            if (oa > amax || (oa == amax && of < from)) amax = oa, mx = om, from = of;
        }
        uint32_t w0 = 0, w1 = 0;
        int sum = 0;
        float d = 0.0f;
        if (amax != 0.0f) {
            const float iscale = __fdiv_rn(-127.0f, mx);
            int q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int bits = __float_as_int(__fadd_rn(__fmul_rn(iscale, v[j]), 12582912.0f));
                const int c = min(127, (bits & 0x007fffff) - 0x00400000);
                q[j] = int(int8_t(c));  // the reference stores the low byte and its sums add the stored bytes
                sum += q[j];
            }
            w0 = pack4(q[0], q[1], q[2], q[3]), w1 = pack4(q[4], q[5], q[6], q[7]);
            d = __fdiv_rn(1.0f, iscale);
        }
        sum += __shfl_xor_sync(kFull, sum, 1);               // 16 codes: lanes 2 k and 2 k + 1
        const int next = __shfl_down_sync(kFull, sum, 2);    // the following group of 16
        mine[1 + 2 * lane] = w0;
        mine[2 + 2 * lane] = w1;
        if ((lane & 3) == 0) mine[65 + (lane >> 2)] = uint32_t(uint16_t(int16_t(sum))) | (uint32_t(uint16_t(int16_t(next))) << 16);
        if (lane == 0) mine[0] = __float_as_uint(d);
        __syncwarp();
        uint32_t * dst = out + blk * 73;
        dst[lane] = mine[lane];
        dst[lane + 32] = mine[lane + 32];
        if (lane < 9) dst[lane + 64] = mine[lane + 64];
        __syncwarp();
    }
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_quantize_q8_k(const float * x, void * out_q8_k, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!ok_ptr(x, 16) || !ok_ptr(out_q8_k, 4)) return FNB_REJECTED;
    if (rows < 1 || rows > INT32_MAX || cols < 256 || cols > (1 << 20) || cols % 256 != 0) return FNB_REJECTED;
    const int64_t n_blocks = rows * (cols / 256);
    const int grid = grid_for((n_blocks + kWarps - 1) / kWarps, 32);
    quantize_q8_k_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint32_t *>(out_q8_k), n_blocks);
    return launch_status();
}
