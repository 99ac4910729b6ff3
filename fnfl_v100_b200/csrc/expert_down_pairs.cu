// The routed experts' down mat-vec for a decode window with ggml IQ4_NL weights against Q8_0 activations,
//     out[t][r] = weight row r . act[t],   t < nt,  r in [r0, r1).
// Replaces fn::experts::cpu::iq4nl_down_rows (fn/kernels/experts/cpu_kernels.h:73; cpu_iq_avx2.cpp:481-514, :571-578)
// and returns the SAME BITS: per (row, t) the AVX2 kernel keeps eight F32 lanes; a block (fp16 d, 16 nibble bytes: value
// i is kvalues_iq4nl[low nibble of byte i], value 16 + i the high nibble's) adds to lane l the four products of values
// 4 l .. 4 l + 3 by one fused multiply-add with x.d y.d; the row's result is that file's hsum8: lane l + 4 onto lane l,
// then (s0 + s1) + (s2 + s3).  It multiplies |w| by the code with w's sign applied (_mm256_sign_epi8), which is w x code
// unless the code is -128 (it stays -128): ggml's Q8_0 quantiser cannot emit -128, but a CTA that finds one in its
// window takes the variant that does exactly that.
//
// FOUR GPU lanes a weight row: lane k takes nibble word k of every block, whose low nibbles are AVX2 lane k and whose
// high nibbles are AVX2 lane k + 4; a warp takes eight consecutive rows, which are one contiguous span of the matrix
// (rows back to back), staged one unit ahead by 16-byte cp.async.  The 16-entry table is four registers, looked up by
// byte permutes: low three index bits select within each table half, the fourth chooses the half.
//
// The same kernel takes the reference engine's own Q2_0 down rows (fn::experts::cpu::q2_down_rows,
// fn/kernels/experts/cpu_kernels.h:78-81; cpu_q2_avx2.cpp:62-102): 64-weight blocks of the same 18 bytes (fp16 d, 16
// bytes of 2-bit codes, value 4 i + k at bits 2 k of byte i, weight d (c - 1)) against its planar activation (int8
// codes, one F32 scale per 32 values: fnb_quantize_act_q).  Per pair of blocks eight lanes, lane 4 h + m = block h's
// values 16 m .. 16 m + 15: sum(c q) - sum(q) in integers, converted, times the chunk scale, one fused multiply-add by
// d; an output is ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7)).  Lane k of a row's four takes code word k of both
// blocks of a pair (AVX2 lanes k and 4 + k), exactly the IQ4_NL assignment.
#include <atomic>

#include "common.cuh"
#include "stage_span.cuh"

#ifndef FNB_DOWN_IQ4_GRID
#define FNB_DOWN_IQ4_GRID 4
#endif
#ifndef FNB_DOWN_IQ4_WARPS
#define FNB_DOWN_IQ4_WARPS 8
#endif

namespace fnb {
namespace {

constexpr int kMaxWarps = FNB_DOWN_IQ4_WARPS;
constexpr int kMaxT = 8;
#ifndef FNB_DOWN_PAIRS_PASSES
#define FNB_DOWN_PAIRS_PASSES 2
#endif
// a staged unit is this many groups of eight rows (more bytes per copy, fewer trips).  Windows of 1 / 3 rows, 640 columns:
// Q2_0 0.123 / 0.236 ms with one group, 0.117 / 0.234 with two, 0.123 / 0.234 with four; IQ4_NL 0.138 / 0.197, 0.138 /
// 0.187, 0.152 / 0.216
constexpr int kPasses = FNB_DOWN_PAIRS_PASSES;  // where shared memory allows; else one group
constexpr size_t kSmemLimit = 200 * 1024;
constexpr int kGridPerSm = FNB_DOWN_IQ4_GRID;

// kvalues_iq4nl (ggml-common.h), four entries to a word
constexpr uint32_t kT0 = 0xbfad9881u;  // -127 -104  -83  -65
constexpr uint32_t kT1 = 0xf6eaddcfu;  //  -49  -35  -22  -10
constexpr uint32_t kT2 = 0x26190d01u;  //    1   13   25   38
constexpr uint32_t kT3 = 0x71594535u;  //   53   69   89  113

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t s) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(s));
    return r;
}

// table values of the four nibbles in the low 16 bits of q, in nibble order (byte 0's low, byte 0's high, byte 1's ..)
__device__ __forceinline__ uint32_t lookup4(uint32_t q) {
    const uint32_t sel = q & 0x7777u;                         // three index bits a nibble (bit 3 would mean "replicate sign")
    const uint32_t a = prmt(kT0, kT1, sel), b = prmt(kT2, kT3, sel);
    return prmt(a, b, ((q >> 1) & 0x4444u) | 0x3210u);        // byte i from b where index bit 3 is set
}

// nibble word q (bytes i .. i + 3 of the block's 16) -> its four low-nibble values and its four high-nibble values
__device__ __forceinline__ void decode8(uint32_t q, uint32_t & lo, uint32_t & hi) {
    const uint32_t r0 = lookup4(q), r1 = lookup4(q >> 16);    // (lo0 hi0 lo1 hi1), (lo2 hi2 lo3 hi3)
    lo = prmt(r0, r1, 0x6420u), hi = prmt(r0, r1, 0x7531u);
}

// |w| and the codes with w's sign applied in two's complement, -128 staying -128 (_mm256_sign_epi8)
__device__ __forceinline__ int dot_sign_applied(uint32_t w, uint32_t y) {
    const uint32_t mff = prmt(w, w, 0xba98u);  // 0xFF where w < 0
    const uint32_t one = mff & 0x01010101u;
    const uint32_t absw = (w ^ mff) + one;     // |w| <= 127: no carry out of a byte
    const uint32_t a = y ^ mff;
    const uint32_t ys = ((a & 0x7f7f7f7fu) + one) ^ (a & 0x80808080u);
    return __dp4a(int(absw), int(ys), 0);
}

// two blocks (36 bytes, 4-byte aligned) of the lane's row: words 0 .. 8 = d0 | 16 nibble bytes | d1 | 16 nibble bytes
template <int NT, bool WRAP>
__device__ __forceinline__ void dot_pair(const uint32_t * x, const uint2 * yk, const float * dk, int nb, int k,
                                         float (&acc)[NT][2]) {  // yk, dk: the lane's codes and the scales of this pair, row 0
    const uint32_t w0 = x[0], w4 = x[4];
    const uint32_t qa = __funnelshift_r(x[k], x[k + 1], 16);  // block ib: bytes 2 + 4 k .. 5 + 4 k
    const uint32_t qb = x[5 + k];                             // block ib + 1: bytes 20 + 4 k ..
    const float da = f16_bits_to_f32(uint16_t(w0 & 0xffffu)), db = f16_bits_to_f32(uint16_t(w4 >> 16));
    uint32_t alo, ahi, blo, bhi;
    decode8(qa, alo, ahi);
    decode8(qb, blo, bhi);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const uint2 ya = yk[t * nb * 4], yb = yk[t * nb * 4 + 4];  // codes 4 k .. and 16 + 4 k .. of the two blocks
        const float sa = __fmul_rn(da, dk[t * nb]), sb = __fmul_rn(db, dk[t * nb + 1]);
        int pa0, pa1, pb0, pb1;
        if (WRAP) {
            pa0 = dot_sign_applied(alo, ya.x), pa1 = dot_sign_applied(ahi, ya.y);
            pb0 = dot_sign_applied(blo, yb.x), pb1 = dot_sign_applied(bhi, yb.y);
        } else {
            pa0 = __dp4a(int(alo), int(ya.x), 0), pa1 = __dp4a(int(ahi), int(ya.y), 0);
            pb0 = __dp4a(int(blo), int(yb.x), 0), pb1 = __dp4a(int(bhi), int(yb.y), 0);
        }
        acc[t][0] = __fmaf_rn(sa, float(pa0), acc[t][0]), acc[t][1] = __fmaf_rn(sa, float(pa1), acc[t][1]);
        acc[t][0] = __fmaf_rn(sb, float(pb0), acc[t][0]), acc[t][1] = __fmaf_rn(sb, float(pb1), acc[t][1]);
    }
}

// Q2_0: the lane's activation image of a pair, per window row: its sixteen codes of either block in plane order (plane
// kk = values 4 j + kk, j = 0 .. 3: what the code bits 2 kk select), then {sum of the sixteen, chunk scale} of either block
struct q2_image {
    uint4 planes[2];
    uint4 ps;  // sum0, scale0 bits, sum1, scale1 bits
};

template <int NT>
__device__ __forceinline__ void dot_pair_q2(const uint32_t * x, const q2_image * img, int n_pairs, int k, float (&acc)[NT][2]) {
    const uint32_t w0 = x[0], w4 = x[4];
    const uint32_t qa = __funnelshift_r(x[k], x[k + 1], 16);  // block 0: code bytes 4 k .. 4 k + 3
    const uint32_t qb = x[5 + k];                             // block 1
    const float da = f16_bits_to_f32(uint16_t(w0 & 0xffffu)), db = f16_bits_to_f32(uint16_t(w4 >> 16));
    const uint32_t m3 = 0x03030303u;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const q2_image & im = img[t * n_pairs * 4];
        const uint4 pa = im.planes[0], pb = im.planes[1], ps = im.ps;
        int sa = __dp4a(int(qa & m3), int(pa.x), 0), sb = __dp4a(int(qb & m3), int(pb.x), 0);
        sa = __dp4a(int((qa >> 2) & m3), int(pa.y), sa), sb = __dp4a(int((qb >> 2) & m3), int(pb.y), sb);
        sa = __dp4a(int((qa >> 4) & m3), int(pa.z), sa), sb = __dp4a(int((qb >> 4) & m3), int(pb.z), sb);
        sa = __dp4a(int((qa >> 6) & m3), int(pa.w), sa), sb = __dp4a(int((qb >> 6) & m3), int(pb.w), sb);
        const float va = __fmul_rn(float(sa - int(ps.x)), __uint_as_float(ps.y));
        const float vb = __fmul_rn(float(sb - int(ps.z)), __uint_as_float(ps.w));
        acc[t][0] = __fmaf_rn(da, va, acc[t][0]);
        acc[t][1] = __fmaf_rn(db, vb, acc[t][1]);
    }
}

template <int NT, bool WRAP, bool Q2>
__device__ __forceinline__ void run_warp(const uint8_t * __restrict__ w, int64_t row_bytes, int nb, const uint2 * codes_sm,
                                         const float * d_sm, uint8_t * stage, int unit_bytes, int unit_rows, float * __restrict__ out,
                                         int64_t out_stride, int64_t r0, int64_t r1) {
    const int lane = threadIdx.x & 31, k = lane & 3, sub = lane >> 2;
    const int warps = blockDim.x >> 5;
    const int64_t n_units = (r1 - r0 + unit_rows - 1) / unit_rows, stride = int64_t(gridDim.x) * warps;
    int64_t u = int64_t(blockIdx.x) * warps + (threadIdx.x >> 5);
    if (u >= n_units) return;
    const uint32_t stage_sm = uint32_t(__cvta_generic_to_shared(stage));
    // a unit's rows are one run of the matrix; a ragged last unit copies the rows there are and leaves the others'
    // bytes as they were (their results are not stored)
    const auto issue = [&](int64_t unit, int buf) {
        const int64_t first = r0 + unit * unit_rows;
        const int rows = r1 - first < unit_rows ? int(r1 - first) : unit_rows;
        stage_span(stage_sm + uint32_t(buf) * unit_bytes, w + first * row_bytes, rows * int(row_bytes), lane);
        cp_async_commit();
    };
    issue(u, 0);
    for (int trip = 0;; ++trip) {
        const int64_t un = u + stride;
        const bool more = un < n_units;
        if (more) {
            issue(un, (trip + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const int64_t first = r0 + u * unit_rows;
        const uintptr_t src = reinterpret_cast<uintptr_t>(w + first * row_bytes);
#pragma unroll 1
        for (int pass = 0; pass < unit_rows / 8; ++pass) {
        const int64_t r = first + 8 * pass + sub;
        const uint32_t * x = reinterpret_cast<const uint32_t *>(stage + size_t(trip & 1) * unit_bytes + (src & 15) +
                                                                size_t(8 * pass + sub) * row_bytes);
        float acc[NT][2];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t][0] = 0.0f, acc[t][1] = 0.0f;
        if (Q2) {
            const q2_image * img = reinterpret_cast<const q2_image *>(codes_sm) + k;
            for (int p = 0; p < nb; ++p, x += 9, img += 4) dot_pair_q2<NT>(x, img, nb, k, acc);  // nb: pairs a row
        } else {
            const uint2 * yk = codes_sm + k;
            const float * dk = d_sm;
            for (int ib = 0; ib < nb; ib += 2, x += 9, yk += 8, dk += 2) dot_pair<NT, WRAP>(x, yk, dk, nb, k, acc);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            // hsum8 of the reference's IQ kernels: lane l + 4 onto lane l (this lane's own pair), then s0 + s1 and
            // s2 + s3 (one lane up), then their sum (two lanes up)
            float s;
            if (Q2) {  // reduce1 of the reference's Q2_0 rows: either block's four lanes as a tree, then their sum
                float a = acc[t][0], b = acc[t][1];
                a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 4)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 4));
                a = __fadd_rn(a, __shfl_down_sync(kFull, a, 2, 4)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 2, 4));
                s = __fadd_rn(a, b);
            } else {
                s = __fadd_rn(acc[t][0], acc[t][1]);
                s = __fadd_rn(s, __shfl_down_sync(kFull, s, 1, 4));
                s = __fadd_rn(s, __shfl_down_sync(kFull, s, 2, 4));
            }
            if (k == 0 && r < r1) out[int64_t(t) * out_stride + r] = s;
        }
        }
        __syncwarp();  // every lane is done with the buffer the next trip's copies overwrite
        if (!more) break;
        u = un;
    }
}

// nb: IQ4_NL blocks a row; for Q2_0 the PAIRS of 64-weight blocks a row.  scales / scale_stride: Q2_0's chunk scales.
template <int NT, bool Q2>
__global__ void __launch_bounds__(kMaxWarps * 32)
    down_pairs_kernel(const uint8_t * __restrict__ w, int64_t row_bytes, int nb, const uint8_t * __restrict__ act,
                      int64_t act_stride, const float * __restrict__ scales, int64_t scale_stride, int act_bytes,
                      int unit_bytes, int unit_rows, float * __restrict__ out, int64_t out_stride, int64_t r0, int64_t r1) {
    // the window's Q8_0 blocks rearranged: per block and lane k the code words k and 4 + k as one 8-byte entry
    // [NT nb][4], then the scales widened to F32 [NT nb]; then each warp's two units
    extern __shared__ __align__(16) uint8_t smem[];
    uint2 * codes_sm = reinterpret_cast<uint2 *>(smem);
    float * d_sm = reinterpret_cast<float *>(smem + size_t(NT) * nb * 32);
    int has_m128 = 0;
    // Q2_0: per window row, pair, lane m and block h the sixteen codes 128 p + 64 h + 16 m .. as four plane words (a 4 x 4
    // byte transpose), their sum and their chunk's scale: q2_image [NT][pairs][4]
    for (int i = threadIdx.x; i < (Q2 ? NT * nb * 8 : 0); i += blockDim.x) {
        const int h = i & 1, m = (i >> 1) & 3, tp = i >> 3;
        const int t = tp / nb, p = tp - t * nb;
        const uint4 c = __ldg(reinterpret_cast<const uint4 *>(act + int64_t(t) * act_stride + 128 * p + 64 * h + 16 * m));
        const uint32_t t0 = prmt(c.x, c.y, 0x5140u), t1 = prmt(c.z, c.w, 0x5140u);
        const uint32_t t2 = prmt(c.x, c.y, 0x7362u), t3 = prmt(c.z, c.w, 0x7362u);
        uint32_t * img = reinterpret_cast<uint32_t *>(smem) + size_t(tp * 4 + m) * 12;
        reinterpret_cast<uint4 *>(img)[h] = make_uint4(prmt(t0, t1, 0x5410u), prmt(t0, t1, 0x7632u), prmt(t2, t3, 0x5410u),
                                                       prmt(t2, t3, 0x7632u));
        const int sum = __dp4a(int(c.x), 0x01010101, __dp4a(int(c.y), 0x01010101, __dp4a(int(c.z), 0x01010101, __dp4a(int(c.w), 0x01010101, 0))));
        img[8 + 2 * h] = uint32_t(sum);
        img[9 + 2 * h] = __float_as_uint(__ldg(scales + int64_t(t) * scale_stride + 4 * p + 2 * h + (m >> 1)));
    }
    for (int i = threadIdx.x; i < (Q2 ? 0 : NT * nb * 9); i += blockDim.x) {  // 34-byte blocks, 2-byte aligned: 16-bit loads
        const int b = i / 9, word = i - b * 9;
        const int t = b / nb, blk = b - t * nb;
        const uint16_t * p = reinterpret_cast<const uint16_t *>(act + int64_t(t) * act_stride + size_t(blk) * 34);
        if (word == 0) {
            d_sm[b] = f16_bits_to_f32(__ldg(p));
        } else {
            const int c = word - 1;  // code word c: codes 4 c .. 4 c + 3
            const uint32_t v = uint32_t(__ldg(p + 1 + 2 * c)) | (uint32_t(__ldg(p + 2 + 2 * c)) << 16);
            reinterpret_cast<uint32_t *>(smem)[b * 8 + (c & 3) * 2 + (c >> 2)] = v;
            const uint32_t z = v ^ 0x80808080u;  // a code byte equal to 0x80
            has_m128 |= ((z - 0x01010101u) & ~z & 0x80808080u) != 0u;
        }
    }
    const int wrap = __syncthreads_or(has_m128);
    uint8_t * stage = smem + act_bytes + size_t(threadIdx.x >> 5) * 2 * unit_bytes;
    if (wrap) {
        run_warp<NT, true, Q2>(w, row_bytes, nb, codes_sm, d_sm, stage, unit_bytes, unit_rows, out, out_stride, r0, r1);
    } else {
        run_warp<NT, false, Q2>(w, row_bytes, nb, codes_sm, d_sm, stage, unit_bytes, unit_rows, out, out_stride, r0, r1);
    }
}

template <int NT, bool Q2>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(down_pairs_kernel<NT, Q2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemLimit)) !=
            cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

template <int NT, bool Q2>
int32_t launch_nt(const uint8_t * w, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride, const float * scales,
                  int64_t scale_stride, float * out, int64_t out_stride, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t act_bytes = Q2 ? size_t(NT) * nb * 4 * sizeof(q2_image) : (size_t(NT) * nb * 36 + 15) & ~size_t(15);
    // kPasses groups of eight rows a unit where that still leaves four warps for two CTAs an SM, else one group
    int unit_rows = 8 * kPasses;
    size_t unit_bytes = (size_t(unit_rows) * row_bytes + 16 + 15) & ~size_t(15);
    if (act_bytes + 4 * 2 * unit_bytes > kSmemLimit / 2) {
        unit_rows = 8;
        unit_bytes = (size_t(unit_rows) * row_bytes + 16 + 15) & ~size_t(15);
    }
    if (act_bytes + 2 * unit_bytes > kSmemLimit) return FNB_REJECTED;
    int warps = int((kSmemLimit / 2 - act_bytes) / (2 * unit_bytes));  // two CTAs an SM where that leaves four warps each
    if (warps < 4) warps = int((kSmemLimit - act_bytes) / (2 * unit_bytes));
    warps = warps > kMaxWarps ? kMaxWarps : warps;
    if (!ensure_configured<NT, Q2>()) return FNB_LAUNCH_FAILED;
    const size_t smem = act_bytes + size_t(warps) * 2 * unit_bytes;
    const int64_t units = (r1 - r0 + unit_rows - 1) / unit_rows;
    const int grid = grid_for((units + warps - 1) / warps, kGridPerSm);
    down_pairs_kernel<NT, Q2><<<grid, warps * 32, smem, s>>>(w, row_bytes, nb, act, act_stride, scales, scale_stride,
                                                              int(act_bytes), int(unit_bytes), unit_rows, out, out_stride, r0, r1);
    return launch_status();
}

template <bool Q2>
bool prepare_fmt() {
    return ensure_configured<1, Q2>() && ensure_configured<2, Q2>() && ensure_configured<3, Q2>() && ensure_configured<4, Q2>() &&
           ensure_configured<5, Q2>() && ensure_configured<6, Q2>() && ensure_configured<7, Q2>() && ensure_configured<8, Q2>();
}

// the window in passes of at most eight rows, as the reference's; nb: IQ4_NL blocks or Q2_0 pairs a row
template <bool Q2>
int32_t launch_window(const uint8_t * w, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride, const float * scales,
                      int64_t scale_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1, cudaStream_t s) {
    for (int t0 = 0; t0 < nt; t0 += kMaxT) {
        const int m = nt - t0 < kMaxT ? nt - t0 : kMaxT;
        const uint8_t * at = act + int64_t(t0) * act_stride;
        const float * sc = scales == nullptr ? nullptr : scales + int64_t(t0) * scale_stride;
        float * ot = out + int64_t(t0) * out_stride;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 2: st = launch_nt<2, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 3: st = launch_nt<3, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 4: st = launch_nt<4, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 5: st = launch_nt<5, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 6: st = launch_nt<6, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            case 7: st = launch_nt<7, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
            default: st = launch_nt<8, Q2>(w, row_bytes, nb, at, act_stride, sc, scale_stride, ot, out_stride, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}

}  // namespace

bool expert_down_iq4nl_prepare_device() { return prepare_fmt<false>() && prepare_fmt<true>(); }

}  // namespace fnb

extern "C" int32_t fnb_expert_down_rows_iq4_nl(const void * w, int64_t row_bytes, int32_t n, const void * act,
                                               int64_t act_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0,
                                               int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(w, 16) || !ok_ptr(act, 2) || !ok_ptr(out, 4)) return FNB_REJECTED;
    // an even number of 18-byte blocks a row: rows on 4-byte boundaries, blocks taken in 36-byte pairs
    if (n < 64 || n > 8192 || n % 64 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 32;
    if (row_bytes != int64_t(nb) * 18 || act_stride < int64_t(nb) * 34 || act_stride % 2 != 0 || out_stride < r1) return FNB_REJECTED;
    return launch_window<false>(static_cast<const uint8_t *>(w), row_bytes, nb, static_cast<const uint8_t *>(act), act_stride,
                                nullptr, 0, nt, out, out_stride, r0, r1, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_expert_down_rows_q2_0(const void * w, int64_t row_bytes, int32_t n, const int8_t * codes,
                                             int64_t codes_stride, const float * scales, int64_t scales_stride, int32_t nt,
                                             float * out, int64_t out_stride, int64_t r0, int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(w, 16) || !ok_ptr(codes, 16) || !ok_ptr(scales, 4) || !ok_ptr(out, 4)) return FNB_REJECTED;
    // whole pairs of 64-weight blocks, as the reference's bit-plane image takes them
    if (n < 128 || n > 8192 || n % 128 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int pairs = n / 128;
    if (row_bytes != int64_t(pairs) * 36 || codes_stride < n || codes_stride % 16 != 0 || scales_stride < n / 32 || out_stride < r1) {
        return FNB_REJECTED;
    }
    return launch_window<true>(static_cast<const uint8_t *>(w), row_bytes, pairs, reinterpret_cast<const uint8_t *>(codes),
                               codes_stride, scales, scales_stride, nt, out, out_stride, r0, r1, static_cast<cudaStream_t>(stream));
}
