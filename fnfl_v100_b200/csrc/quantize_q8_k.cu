// F32 rows -> ggml Q8_K activation blocks (292 bytes per 256 values: F32 d, 256 int8 codes, 16 int16 sums of 16 codes),
// the format the routed experts' gate / up mat-vec reads on the reference's CPU tier (block_q8_k,
// fn/kernels/experts/cpu_kernels.h; produced there by fn::experts::cpu::quantize_q8_k, experts_cpu.cpp:321).
// Bit-identical to ggml's quantize_row_q8_K_ref (ggml/src/ggml-quants.c:2844-2881) and to the reference's AVX2 form:
// the value of largest magnitude - the FIRST one on ties - maps to -127 (iscale = -127 / max), codes are
// nearest-even(iscale x) by the 1.5 x 2^23 trick capped at 127, d = 1 / iscale.  An all-zero block is written as d = 0,
// zero codes and zero sums (the reference leaves the sums of such a block untouched).
// HBM-bound, 4 bytes read and 1.14 written per value.  EIGHT lanes take a block (a warp four consecutive blocks): lane j
// the block's float4s j, j + 8 .. j + 56, so every load instruction of the eight covers 128 contiguous bytes, the search
// for the maximum is three shuffle steps and the two IEEE divisions of a block are paid once per 128 bytes a lane loads
// (a warp per block: 80 % of the HBM roofline, bound by instruction issue).
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarps = 8;

__global__ void __launch_bounds__(kWarps * 32) quantize_q8_k_kernel(const float * __restrict__ x, uint32_t * __restrict__ out,
                                                                   int64_t n_blocks) {
    __shared__ __align__(16) uint32_t s_blk[kWarps][4 * 73 + 4];  // four blocks of 73 words, as they lie in global memory
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, j = lane & 7, sub = lane >> 3;
    const int64_t warp = int64_t(blockIdx.x) * kWarps + wid, n_warps = int64_t(gridDim.x) * kWarps;
    uint32_t * mine = s_blk[wid] + 73 * sub;
    for (int64_t blk4 = 4 * warp; blk4 < n_blocks; blk4 += 4 * n_warps) {
        const bool live = blk4 + sub < n_blocks;
        const int64_t blk = live ? blk4 + sub : n_blocks - 1;  // every lane takes part in the shuffles
        const float4 * src = reinterpret_cast<const float4 *>(x + blk * 256) + j;
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = ld_stream(src + 8 * q);
        // largest magnitude, the value that has it and its index, first occurrence: in-lane in index order (float4
        // j + 8 q, components in order), then across the eight lanes with the lower index winning ties
        float amax = 0.0f, mx = 0.0f;
        int at = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float c[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float ax = fabsf(c[e]);
                if (ax > amax) amax = ax, mx = c[e], at = 4 * (j + 8 * q) + e;
            }
        }
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
            const float oa = __shfl_xor_sync(kFull, amax, m), om = __shfl_xor_sync(kFull, mx, m);
            const int oat = __shfl_xor_sync(kFull, at, m);
            if (oa > amax || (oa == amax && oat < at)) amax = oa, mx = om, at = oat;
        }
        float d = 0.0f;
        if (amax != 0.0f) {
            const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float c[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
                int code[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int bits = __float_as_int(__fadd_rn(__fmul_rn(iscale, c[e]), 12582912.0f));
                    code[e] = min(127, (bits & 0x007fffff) - 0x00400000);  // the reference stores the low byte
                }
                mine[1 + j + 8 * q] = pack4_low_bytes(code[0], code[1], code[2], code[3]);
            }
            d = __fdiv_rn(1.0f, iscale);
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) mine[1 + j + 8 * q] = 0u;
        }
        if (j == 0) mine[0] = __float_as_uint(d);
        __syncwarp();
        // sums 2 j and 2 j + 1 of the block's sixteen: code words 8 j .. 8 j + 3 and 8 j + 4 .. 8 j + 7 (the stored bytes)
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s0 = __dp4a(int(mine[1 + 8 * j + e]), 0x01010101, s0);
            s1 = __dp4a(int(mine[5 + 8 * j + e]), 0x01010101, s1);
        }
        mine[65 + j] = uint32_t(uint16_t(int16_t(s0))) | (uint32_t(uint16_t(int16_t(s1))) << 16);
        __syncwarp();
        const int n_words = int(n_blocks - blk4 < 4 ? n_blocks - blk4 : 4) * 73;
        uint32_t * dst = out + blk4 * 73;
        for (int i = lane; i < n_words; i += 32) dst[i] = s_blk[wid][i];
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
    const int grid = grid_for((n_blocks + 4 * kWarps - 1) / (4 * kWarps), 32);
    quantize_q8_k_kernel<<<grid, kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<uint32_t *>(out_q8_k), n_blocks);
    return launch_status();
}
