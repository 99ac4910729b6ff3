// The routed experts' gate / up mat-vec for a decode window with the GLU fused,
//     ff[t][r] = silu(g) u,   g = gate row r . act[t],  u = up row r . act[t],   t < nt,  r in [r0, r1)
// with ggml Q4_K weights against Q8_K activations (fnb_quantize_q8_k).  Replaces fn::experts::cpu::kq_gu_rows for fmt
// q4_k (fn/kernels/experts/cpu_kernels.h; cpu_kq_avx2.cpp:166-224, :362-380) and returns the SAME BITS: the AVX2 kernel
// keeps, per (row, t), eight int32 lanes of scale-weighted 4-byte dot products per super-block, adds them as floats by
// one fused multiply-add per super-block and lane with d = y.d x.d, keeps four lanes of mins x block sums with
// -y.d x.dmin, reduces once at the end in a fixed order and applies g / (1 + expf(-g)) * u (expf as the host C
// library evaluates it: exact_math.cuh).  Here FOUR GPU LANES stand for the eight AVX2 lanes of one weight row: lane k
// reads bytes 8 k .. 8 k + 7 of each of the row's 32-byte nibble groups straight from global memory (four lanes, one
// 32-byte sector) and keeps AVX2 lanes 2 k, 2 k + 1 and mins lane k; a warp takes four (gate, up) row pairs, the gate
// rows on lanes 0..15 and the up rows on lanes 16..31; the horizontal sums are shuffle steps in the AVX2 order.
// (With eight lanes a row every lane repeated the scale unpacking and header decode for half the weights: 0.115 /
// 0.244 / 0.578 ms against this form's 0.072 / 0.138 / 0.283 ms at 2 x 131072 rows of 2560 columns and windows of
// 1 / 3 / 8 rows.)
//
// HBM-bound on the weights at the window sizes decode uses: 2 x 1440 bytes per output row at 2560 columns, read once
// for all window rows; the window's Q8_K blocks sit in shared memory.
#include "common.cuh"
#include "exact_math.cuh"

namespace fnb {
namespace {

#ifndef FNB_GU_Q4K_WARPS
#define FNB_GU_Q4K_WARPS 8
#endif
#ifndef FNB_GU_Q4K_GRID
#define FNB_GU_Q4K_GRID 8
#endif
#ifndef FNB_GU_Q4K_UNROLL
#define FNB_GU_Q4K_UNROLL 2
#endif

constexpr int kWarps = FNB_GU_Q4K_WARPS;
// Measured at 2 x 131072 rows of 2560 columns, windows of 1 / 3 / 8 rows: 32 CTAs per SM and one super-block per trip
// 0.089 / 0.158 / 0.351 ms; two super-blocks per trip (their loads issued together) 0.080 / 0.154 ms; 8 CTAs per SM
// (each CTA rearranges the window once) 0.082 / 0.144 ms; both 0.072 / 0.138 / 0.283 ms; 4 CTAs per SM 0.070 / 0.152 /
// 0.275 ms; four warps a CTA or five super-blocks per trip were slower.
constexpr int kGridPerSm = FNB_GU_Q4K_GRID;
constexpr int kBlockUnroll = FNB_GU_Q4K_UNROLL;
constexpr int kMaxT = 8;

// the eight six-bit scales and eight mins from the 12 packed bytes, four to a word, as ggml unpacks them for its
// vector kernels (the utmp shuffle of ggml_vec_dot_q4_K_q8_K; cpu_kq_avx2.cpp:154-166): about ten logic operations
// for all sixteen values, where get_scale_min_k4 per value costs six each.  s_lo / m_lo: values 0..3, s_hi / m_hi: 4..7.
struct scales_mins {
    uint32_t s_lo, s_hi, m_lo, m_hi;
    __device__ __forceinline__ scales_mins(uint32_t u0, uint32_t u1, uint32_t u2) {
        const uint32_t k1 = 0x3f3f3f3fu, k2 = 0x0f0f0f0fu, k3 = 0x03030303u;
        s_lo = u0 & k1, s_hi = (u2 & k2) | (((u0 >> 6) & k3) << 4);
        m_lo = u1 & k1, m_hi = ((u2 >> 4) & k2) | (((u1 >> 6) & k3) << 4);
    }
    __device__ __forceinline__ int scale(int j) const { return int(((j < 4 ? s_lo : s_hi) >> (8 * (j & 3))) & 0xffu); }
    // mins 2 k and 2 k + 1 as (low byte, next byte)
    __device__ __forceinline__ uint32_t min_pair(int k) const { return ((k < 2 ? m_lo : m_hi) >> (16 * (k & 1))) & 0xffffu; }
};

// One weight row against the window.  Lane k of the row's four stands for the AVX2 kernel's lanes 2 k and 2 k + 1
// (acc[t][0 / 1]: bytes 8 k .. 8 k + 7 of every 32-byte nibble group, one 64-bit load, four lanes one sector) and for
// its mins lane k (accm[t]).
// Q5: ggml Q5_K rows (176-byte super-blocks: d, dmin, 12 scale bytes, qh[32], qs[128]; value 64 j + b is the low
// nibble of qs[32 j + b] plus 16 x bit 2 j of qh[b], value 64 j + 32 + b the high nibble plus 16 x bit 2 j + 1) through
// the same eight lanes (cpu_kq_avx2.cpp:226-290 q5k_dot); there the mins are ONE scalar per (row, t), accm[t] on every
// lane: summs += dmin x (the eight mins x pair sums, added as integers), a fused multiply-add under the reference's
// flags.
template <int NT, bool Q5>
__device__ __forceinline__ void row_dot(const uint8_t * __restrict__ row, int nb, const uint8_t * codes_sm, const int2 * bs_sm,
                                        const float * d_sm, int k, float (&acc)[NT][2], float (&accm)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = 0.0f, acc[t][1] = 0.0f, accm[t] = 0.0f;
#pragma unroll kBlockUnroll
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + (Q5 ? 176 : 144) * i;
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(x));  // d, dmin, 12 scale bytes (blocks are 16-byte aligned)
        uint2 q4[4], qh = make_uint2(0u, 0u);
        if (Q5) qh = __ldg(reinterpret_cast<const uint2 *>(x + 16) + k);
#pragma unroll
        for (int j = 0; j < 4; ++j) q4[j] = __ldg(reinterpret_cast<const uint2 *>(x + (Q5 ? 48 : 16) + 32 * j) + k);
        // the lane's eight low-nibble and eight high-nibble values of nibble group j, four to a word; formed where they
        // are used (held in arrays across the window rows, Q4_K at a window of one row took 0.103 ms instead of 0.072)
        const auto values = [&](int j, uint2 & vlo, uint2 & vhi) {
            vlo = make_uint2(q4[j].x & 0x0f0f0f0fu, q4[j].y & 0x0f0f0f0fu);
            vhi = make_uint2((q4[j].x >> 4) & 0x0f0f0f0fu, (q4[j].y >> 4) & 0x0f0f0f0fu);
            if (Q5) {
                vlo.x |= ((qh.x >> (2 * j)) & 0x01010101u) << 4, vlo.y |= ((qh.y >> (2 * j)) & 0x01010101u) << 4;
                vhi.x |= ((qh.x >> (2 * j + 1)) & 0x01010101u) << 4, vhi.y |= ((qh.y >> (2 * j + 1)) & 0x01010101u) << 4;
            }
        };
        const float xd = f16_bits_to_f32(uint16_t(hdr.x & 0xffffu)), xdmin = f16_bits_to_f32(uint16_t(hdr.x >> 16));
        const scales_mins sm(hdr.y, hdr.z, hdr.w);
        const uint32_t mp = sm.min_pair(k);
        const int mn0 = int(mp & 0xffu), mn1 = int(mp >> 8);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int b = t * nb + i;
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // the lane's codes of nibble group j: low nibbles' eight, then high nibbles' eight (stored that way)
                const uint4 y = *reinterpret_cast<const uint4 *>(codes_sm + size_t(b) * 256 + 64 * j + 16 * k);
                const int lo = sm.scale(2 * j), hi = sm.scale(2 * j + 1);
                uint2 vlo, vhi;
                values(j, vlo, vhi);
                s0 += lo * __dp4a(int(vlo.x), int(y.x), 0) + hi * __dp4a(int(vhi.x), int(y.z), 0);
                s1 += lo * __dp4a(int(vlo.y), int(y.y), 0) + hi * __dp4a(int(vhi.y), int(y.w), 0);
            }
            const float yd = d_sm[b], d = __fmul_rn(yd, xd);
            acc[t][0] = __fmaf_rn(d, float(s0), acc[t][0]);
            acc[t][1] = __fmaf_rn(d, float(s1), acc[t][1]);
            // mins lane k: madd of mins (2 k, 2 k + 1) with the 16-bit pair sums of the block sums (hadd_epi16)
            const int2 bs = bs_sm[b * 4 + k];
            int prod = mn0 * bs.x + mn1 * bs.y;
            if (Q5) {  // all eight products, on every lane of the row
                prod += __shfl_xor_sync(kFull, prod, 1, 4);
                prod += __shfl_xor_sync(kFull, prod, 2, 4);
            }
            accm[t] = __fmaf_rn(__fmul_rn(-yd, xdmin), float(prod), accm[t]);
        }
    }
}

template <int NT, bool Q5>
__global__ void __launch_bounds__(kWarps * 32)
    gate_up_kq_kernel(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes, int nb,
                        const uint8_t * __restrict__ act, int64_t act_stride, float * __restrict__ ff, int64_t ff_stride,
                        float * __restrict__ gu, int64_t r0, int64_t r1) {
    // the window's Q8_K blocks, rearranged: codes [NT nb][256] (per nibble group and lane: the low nibbles' eight codes,
    // then the high nibbles' eight), pair sums of the block sums [NT nb][4] x 2, scales [NT nb]
    extern __shared__ __align__(16) uint8_t act_sm[];
    uint8_t * codes_sm = act_sm;
    int2 * bs_sm = reinterpret_cast<int2 *>(act_sm + size_t(NT) * nb * 256);
    float * d_sm = reinterpret_cast<float *>(act_sm + size_t(NT) * nb * 288);
    load_exp2_table();
    for (int i = threadIdx.x; i < NT * nb * 73; i += blockDim.x) {
        const int b = i / 73, word = i - b * 73;
        const int t = b / nb, blk = b - t * nb;
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(act + int64_t(t) * act_stride) + blk * 73 + word);
        if (word == 0) {
            d_sm[b] = __uint_as_float(w);
        } else if (word <= 64) {
            // code word c: nibble group c / 16, low / high half (c % 16) / 8, word (c % 8) of the half's 32 bytes = lane
            // (c % 8) / 2, its word (c % 2)
            const int c = word - 1;
            reinterpret_cast<uint32_t *>(codes_sm)[b * 64 + (c >> 4) * 16 + ((c & 7) >> 1) * 4 + ((c >> 3) & 1) * 2 + (c & 1)] = w;
        } else {
            // block sums 2 s, 2 s + 1 -> their 16-bit sum; mins lane k takes sums 2 k (x) and 2 k + 1 (y)
            const int s = word - 65;
            reinterpret_cast<int *>(bs_sm)[b * 8 + s] = int(int16_t(int16_t(w & 0xffffu) + int16_t(w >> 16)));
        }
    }
    __syncthreads();
    // four lanes a row; lanes 0..15 the quad's gate rows, lanes 16..31 its up rows
    const int lane = threadIdx.x & 31, k = lane & 3, sub = (lane >> 2) & 3, mat = lane >> 4;
    const uint8_t * mine = mat == 0 ? gate : up;
    const int64_t quad = int64_t(blockIdx.x) * kWarps + (threadIdx.x >> 5), n_quads = int64_t(gridDim.x) * kWarps;
    for (int64_t r4 = r0 + 4 * quad; r4 < r1; r4 += 4 * n_quads) {
        const int64_t r = r4 + sub;
        const bool live = r < r1;
        const int64_t rr = live ? r : r1 - 1;  // every lane takes part in the shuffles
        float acc[NT][2], accm[NT];
        row_dot<NT, Q5>(mine + rr * row_bytes, nb, codes_sm, bs_sm, d_sm, k, acc, accm);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            // hsum_float_8 with r_l on lane l / 2: r_l + r_(l + 4) (two lanes up), lanes 2, 3 onto 0, 1 (one lane up),
            // lane 1 onto lane 0 (the lane's own pair); the mins' four lanes likewise
            float a = acc[t][0], b = acc[t][1], m = accm[t];
            a = __fadd_rn(__shfl_down_sync(kFull, a, 2, 4), a), b = __fadd_rn(__shfl_down_sync(kFull, b, 2, 4), b);
            a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 4)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 4));
            if (!Q5) {  // Q4_K's four mins lanes: (m0 + m2) + (m1 + m3); Q5_K's mins are one scalar already
                m = __fadd_rn(m, __shfl_down_sync(kFull, m, 2, 4));
                m = __fadd_rn(m, __shfl_down_sync(kFull, m, 1, 4));
            }
            const float dot = __fadd_rn(__fadd_rn(a, b), m);
            const float us = __shfl_down_sync(kFull, dot, 16);  // the up row's sits 16 lanes above the gate row's
            if (mat == 0 && k == 0 && live) {
                ff[int64_t(t) * ff_stride + r] = __fmul_rn(__fdiv_rn(dot, __fadd_rn(1.0f, exact_expf(-dot))), us);
                if (gu != nullptr) {
                    gu[int64_t(t) * ff_stride + r] = dot;
                    gu[(int64_t(NT) + t) * ff_stride + r] = us;
                }
            }
        }
    }
}

template <int NT, bool Q5>
int32_t launch_nt(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride,
                  float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t smem = size_t(NT) * nb * 292;
    if (smem > 47 * 1024) return FNB_REJECTED;  // the window's activations must fit the default shared-memory limit
    const int64_t quads = (r1 - r0 + 3) / 4;
    const int grid = grid_for((quads + kWarps - 1) / kWarps, kGridPerSm);
    gate_up_kq_kernel<NT, Q5><<<grid, kWarps * 32, smem, s>>>(gate, up, row_bytes, nb, act, act_stride, ff, ff_stride, gu, r0, r1);
    return launch_status();
}

}  // namespace
}  // namespace fnb

namespace fnb {
namespace {

template <bool Q5>
int32_t gate_up_rows(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                     int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    if (!ok_ptr(gate, 16) || !ok_ptr(up, 16) || !ok_ptr(act, 4) || !ok_ptr(ff, 4) || !ok_opt(gu, 4)) return FNB_REJECTED;
    if (n < 256 || n > 16384 || n % 256 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 256;
    if (row_bytes != int64_t(nb) * (Q5 ? 176 : 144) || act_stride < int64_t(nb) * 292 || act_stride % 4 != 0 || ff_stride < r1) return FNB_REJECTED;
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
            case 1: st = launch_nt<1, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 2: st = launch_nt<2, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 3: st = launch_nt<3, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 4: st = launch_nt<4, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 5: st = launch_nt<5, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 6: st = launch_nt<6, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 7: st = launch_nt<7, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            default: st = launch_nt<8, Q5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_expert_gate_up_rows_q4_k(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<false>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_q5_k(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<true>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}
