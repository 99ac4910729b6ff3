// The routed experts' gate / up mat-vec for a decode window with the GLU fused,
//     ff[t][r] = silu(g) u,   g = gate row r . act[t],  u = up row r . act[t],   t < nt,  r in [r0, r1)
// with ggml Q4_K weights against Q8_K activations (fnb_quantize_q8_k).  Replaces fn::experts::cpu::kq_gu_rows for fmt
// q4_k (fn/kernels/experts/cpu_kernels.h; cpu_kq_avx2.cpp:166-224, :362-380) and returns the SAME BITS: the AVX2 kernel
// keeps, per (row, t), eight int32 lanes of scale-weighted 4-byte dot products per super-block, adds them as floats by
// one fused multiply-add per super-block and lane with d = y.d x.d, keeps four lanes of mins x block sums with
// -y.d x.dmin, reduces once at the end in a fixed order and applies g / (1 + expf(-g)) * u (expf as the host C
// library evaluates it: exact_math.cuh).  Here EIGHT GPU LANES stand for the eight AVX2 lanes of one weight row: lane l
// reads bytes 4 l .. 4 l + 3 of each of the row's 32-byte nibble groups straight from global memory (eight lanes, one
// 32-byte sector), the horizontal sums are three shuffle steps in the AVX2 order.
//
// HBM-bound on the weights at the window sizes decode uses: 2 x 1440 bytes per output row at 2560 columns, read once
// for all window rows; the window's Q8_K blocks sit in shared memory.
#include "common.cuh"
#include "exact_math.cuh"

namespace fnb {
namespace {

constexpr int kWarps = 8;
constexpr int kMaxT = 8;

// the eight six-bit scales and eight mins from the 12 packed bytes, four to a word, as ggml unpacks them for its
// vector kernels (the utmp shuffle of ggml_vec_dot_q4_K_q8_K; cpu_kq_avx2.cpp:154-166): about ten logic operations
// for all sixteen values, where get_scale_min_k4 per value costs six each
__device__ __forceinline__ void scales_mins(uint32_t u0, uint32_t u1, uint32_t u2, int (&sc)[8], int (&mn)[8]) {
    const uint32_t k1 = 0x3f3f3f3fu, k2 = 0x0f0f0f0fu, k3 = 0x03030303u;
    const uint32_t s_lo = u0 & k1, s_hi = (u2 & k2) | (((u0 >> 6) & k3) << 4);
    const uint32_t m_lo = u1 & k1, m_hi = ((u2 >> 4) & k2) | (((u1 >> 6) & k3) << 4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        sc[j] = int((s_lo >> (8 * j)) & 0xffu), sc[j + 4] = int((s_hi >> (8 * j)) & 0xffu);
        mn[j] = int((m_lo >> (8 * j)) & 0xffu), mn[j + 4] = int((m_hi >> (8 * j)) & 0xffu);
    }
}

// one weight row against the window: the lane's accumulator per window row (acc) and, on lanes 0..3, the mins lane (accm)
template <int NT>
__device__ __forceinline__ void row_dot(const uint8_t * __restrict__ row, int nb, const uint8_t * act_sm, int l, float (&acc)[NT],
                                        float (&accm)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.0f, accm[t] = 0.0f;
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + 144 * i;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(x));  // d, dmin, 12 scale bytes (144 i is 16-byte aligned)
        uint32_t q4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) q4[j] = __ldg(reinterpret_cast<const uint32_t *>(x + 16 + 32 * j) + l);
        const float xd = f16_bits_to_f32(uint16_t(hdr.x & 0xffffu)), xdmin = f16_bits_to_f32(uint16_t(hdr.x >> 16));
        int sc[8], mn[8];
        scales_mins(hdr.y, hdr.z, hdr.w, sc, mn);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const uint8_t * y = act_sm + (size_t(t) * nb + i) * 292;
            const float yd = *reinterpret_cast<const float *>(y);
            int sumi = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = q4[j] & 0x0f0f0f0fu, hi = (q4[j] >> 4) & 0x0f0f0f0fu;
                const int ylo = *reinterpret_cast<const int *>(y + 4 + 64 * j + 4 * l);
                const int yhi = *reinterpret_cast<const int *>(y + 4 + 64 * j + 32 + 4 * l);
                sumi += sc[2 * j] * __dp4a(int(lo), ylo, 0) + sc[2 * j + 1] * __dp4a(int(hi), yhi, 0);
            }
            acc[t] = __fmaf_rn(__fmul_rn(yd, xd), float(sumi), acc[t]);
            if (l < 4) {  // mins lane l: madd of mins (2 l, 2 l + 1) with the 16-bit pair sums of the block sums
                const int bx = *reinterpret_cast<const int *>(y + 260 + 8 * l);      // bsums[4 l], [4 l + 1]
                const int by = *reinterpret_cast<const int *>(y + 260 + 8 * l + 4);  // bsums[4 l + 2], [4 l + 3]
                const int s0 = int(int16_t(int16_t(bx & 0xffff) + int16_t(bx >> 16)));
                const int s1 = int(int16_t(int16_t(by & 0xffff) + int16_t(by >> 16)));
                const int prod = (l == 0 ? mn[0] : l == 1 ? mn[2] : l == 2 ? mn[4] : mn[6]) * s0 +
                                 (l == 0 ? mn[1] : l == 1 ? mn[3] : l == 2 ? mn[5] : mn[7]) * s1;
                accm[t] = __fmaf_rn(__fmul_rn(-yd, xdmin), float(prod), accm[t]);
            }
        }
    }
}

// one super-block's weight-side values for a lane
struct q4k_lane {
    uint32_t q4[4];
    float xd, xdmin;
    int sc[8], mn[8];
    __device__ __forceinline__ void load(const uint8_t * x, int l) {
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(x));  // d, dmin, 12 scale bytes (144 i is 16-byte aligned)
#pragma unroll
        for (int j = 0; j < 4; ++j) q4[j] = __ldg(reinterpret_cast<const uint32_t *>(x + 16 + 32 * j) + l);
        xd = f16_bits_to_f32(uint16_t(hdr.x & 0xffffu)), xdmin = f16_bits_to_f32(uint16_t(hdr.x >> 16));
        scales_mins(hdr.y, hdr.z, hdr.w, sc, mn);
    }
    __device__ __forceinline__ int min_pair(int l, int s0, int s1) const {  // madd of mins (2 l, 2 l + 1) with the pair sums
        return (l == 0 ? mn[0] : l == 1 ? mn[2] : l == 2 ? mn[4] : mn[6]) * s0 +
               (l == 0 ? mn[1] : l == 1 ? mn[3] : l == 2 ? mn[5] : mn[7]) * s1;
    }
};

// the gate row and the up row of one output against the window, in one pass over the activations (both rows read the
// same Q8_K words): per window row the lane's accumulators (g, u) and, on lanes 0..3, the mins lanes (gm, um)
template <int NT>
__device__ __forceinline__ void rows_dot(const uint8_t * __restrict__ grow, const uint8_t * __restrict__ urow, int nb,
                                         const uint8_t * act_sm, int l, float (&g)[NT], float (&u)[NT], float (&gm)[NT],
                                         float (&um)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) g[t] = 0.0f, u[t] = 0.0f, gm[t] = 0.0f, um[t] = 0.0f;
    for (int i = 0; i < nb; ++i) {
        q4k_lane wg, wu;
        wg.load(grow + 144 * i, l);
        wu.load(urow + 144 * i, l);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const uint8_t * y = act_sm + (size_t(t) * nb + i) * 292;
            const float yd = *reinterpret_cast<const float *>(y);
            int sg = 0, su = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int ylo = *reinterpret_cast<const int *>(y + 4 + 64 * j + 4 * l);
                const int yhi = *reinterpret_cast<const int *>(y + 4 + 64 * j + 32 + 4 * l);
                sg += wg.sc[2 * j] * __dp4a(int(wg.q4[j] & 0x0f0f0f0fu), ylo, 0) +
                      wg.sc[2 * j + 1] * __dp4a(int((wg.q4[j] >> 4) & 0x0f0f0f0fu), yhi, 0);
                su += wu.sc[2 * j] * __dp4a(int(wu.q4[j] & 0x0f0f0f0fu), ylo, 0) +
                      wu.sc[2 * j + 1] * __dp4a(int((wu.q4[j] >> 4) & 0x0f0f0f0fu), yhi, 0);
            }
            g[t] = __fmaf_rn(__fmul_rn(yd, wg.xd), float(sg), g[t]);
            u[t] = __fmaf_rn(__fmul_rn(yd, wu.xd), float(su), u[t]);
            if (l < 4) {  // mins lane l: the 16-bit pair sums of the block sums (hadd_epi16), then madd with the mins
                const int bx = *reinterpret_cast<const int *>(y + 260 + 8 * l);      // bsums[4 l], [4 l + 1]
                const int by = *reinterpret_cast<const int *>(y + 260 + 8 * l + 4);  // bsums[4 l + 2], [4 l + 3]
                const int s0 = int(int16_t(int16_t(bx & 0xffff) + int16_t(bx >> 16)));
                const int s1 = int(int16_t(int16_t(by & 0xffff) + int16_t(by >> 16)));
                gm[t] = __fmaf_rn(__fmul_rn(-yd, wg.xdmin), float(wg.min_pair(l, s0, s1)), gm[t]);
                um[t] = __fmaf_rn(__fmul_rn(-yd, wu.xdmin), float(wu.min_pair(l, s0, s1)), um[t]);
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(kWarps * 32)
    gate_up_q4_k_kernel(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes, int nb,
                        const uint8_t * __restrict__ act, int64_t act_stride, float * __restrict__ ff, int64_t ff_stride,
                        float * __restrict__ gu, int64_t r0, int64_t r1) {
    extern __shared__ __align__(16) uint8_t act_sm[];  // [NT][nb][292]
    load_exp2_table();
    for (int i = threadIdx.x; i < NT * nb * 73; i += blockDim.x) {
        const int t = i / (nb * 73), k = i - t * nb * 73;
        reinterpret_cast<uint32_t *>(act_sm)[i] = __ldg(reinterpret_cast<const uint32_t *>(act + int64_t(t) * act_stride) + k);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, l = lane & 7, sub = lane >> 3;
    const int64_t quad = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5), n_quads = int64_t(gridDim.x) * kWarps;
    for (int64_t r4 = r0 + 4 * quad; r4 < r1; r4 += 4 * n_quads) {
        const int64_t r = r4 + sub;
        const bool live = r < r1;
        const int64_t rr = live ? r : r1 - 1;  // every lane takes part in the shuffles
        float g[NT], u[NT], gm[NT], um[NT];
        // measured at 2 x 131072 rows of 2560 columns: one pass per matrix 0.125 / 0.250 / 0.760 ms at windows of
        // 1 / 3 / 8 rows, both matrices in one pass over the activations 0.144 / 0.300 / 0.580 ms
        if constexpr (NT >= 6) {
            rows_dot<NT>(gate + rr * row_bytes, up + rr * row_bytes, nb, act_sm, l, g, u, gm, um);
        } else {
            row_dot<NT>(gate + rr * row_bytes, nb, act_sm, l, g, gm);
            row_dot<NT>(up + rr * row_bytes, nb, act_sm, l, u, um);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            // hsum_float_8: lane i + 4 onto lane i, lanes 2, 3 onto 0, 1, lane 1 onto lane 0; the mins' four lanes likewise
            float a = g[t], b = u[t], am = gm[t], bm = um[t];
            a = __fadd_rn(__shfl_down_sync(kFull, a, 4, 8), a), b = __fadd_rn(__shfl_down_sync(kFull, b, 4, 8), b);
            a = __fadd_rn(a, __shfl_down_sync(kFull, a, 2, 8)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 2, 8));
            a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 8)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 8));
            am = __fadd_rn(am, __shfl_down_sync(kFull, am, 2, 8)), bm = __fadd_rn(bm, __shfl_down_sync(kFull, bm, 2, 8));
            am = __fadd_rn(am, __shfl_down_sync(kFull, am, 1, 8)), bm = __fadd_rn(bm, __shfl_down_sync(kFull, bm, 1, 8));
            if (l == 0 && live) {
                const float gs = __fadd_rn(a, am), us = __fadd_rn(b, bm);
                ff[int64_t(t) * ff_stride + r] = __fmul_rn(__fdiv_rn(gs, __fadd_rn(1.0f, exact_expf(-gs))), us);
                if (gu != nullptr) {
                    gu[int64_t(t) * ff_stride + r] = gs;
                    gu[(int64_t(NT) + t) * ff_stride + r] = us;
                }
            }
        }
    }
}

template <int NT>
int32_t launch_nt(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride,
                  float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t smem = size_t(NT) * nb * 292;
    if (smem > 47 * 1024) return FNB_REJECTED;  // the window's activations must fit the default shared-memory limit
    const int64_t quads = (r1 - r0 + 3) / 4;
    const int grid = grid_for((quads + kWarps - 1) / kWarps, 32);
    gate_up_q4_k_kernel<NT><<<grid, kWarps * 32, smem, s>>>(gate, up, row_bytes, nb, act, act_stride, ff, ff_stride, gu, r0, r1);
    return launch_status();
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_expert_gate_up_rows_q4_k(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(gate, 16) || !ok_ptr(up, 16) || !ok_ptr(act, 4) || !ok_ptr(ff, 4) || !ok_opt(gu, 4)) return FNB_REJECTED;
    if (n < 256 || n > 16384 || n % 256 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 256;
    if (row_bytes != int64_t(nb) * 144 || act_stride < int64_t(nb) * 292 || act_stride % 4 != 0 || ff_stride < r1) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * gp = static_cast<const uint8_t *>(gate);
    const uint8_t * upp = static_cast<const uint8_t *>(up);
    const uint8_t * a = static_cast<const uint8_t *>(act);
    for (int t0 = 0; t0 < nt; t0 += kMaxT) {  // windows above eight rows take further passes, as the reference's do
        const int m = nt - t0 < kMaxT ? nt - t0 : kMaxT;
        const uint8_t * at = a + int64_t(t0) * act_stride;
        float * ft = ff + int64_t(t0) * ff_stride;
        // g and u of a later pass would need their own [2][m] planes: the debug output is for windows of one pass
        if (gu != nullptr && nt > kMaxT) return FNB_REJECTED;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 2: st = launch_nt<2>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 3: st = launch_nt<3>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 4: st = launch_nt<4>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 5: st = launch_nt<5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 6: st = launch_nt<6>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 7: st = launch_nt<7>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            default: st = launch_nt<8>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}
