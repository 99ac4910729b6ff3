// expf, sinf and cosf whose results are bit-identical to the host C library the CPU definition of this path
// calls (GNU libc 2.39, generic non-FMA build): the same double-precision algorithm - 2^(k/32) table with a
// cubic for expf; Cody-Waite / 4-over-pi argument reduction with odd/even minimax polynomials for sinf and
// cosf - evaluated with the same IEEE operations in the same order.  Every double operation is written with
// an explicit round-to-nearest intrinsic so no multiply-add is ever contracted.
//
// Cost: expf is 12 FP64 operations and two conversions per value as defined (expf_steps); the SwiGLU fast path uses
// expf_core, 8 FP64 operations, which rounds to the same float for every input (see there).  sin/cos are needed
// once per token and rotary pair (32 per token), which is noise.
#pragma once

#include "common.cuh"
#include "exact_math_tables.inc"

namespace fnb {

static __constant__ unsigned long long c_exp2_tab[32] = FNB_EXP2_TABLE_INIT;
static __constant__ uint32_t c_inv_pio4[24] = FNB_INV_PIO4_INIT;
// expf's double constants live in constant memory so the FP64 instructions read them as constant-bank
// operands instead of rebuilding 64-bit immediates in registers for every value:
// N / ln2, the 1.5 * 2^52 rounding shift, and the cubic's coefficients scaled by 1 / N^3, 1 / N^2, 1 / N (N = 32)
static __constant__ double c_exp_k[5] = {0x1.71547652b82fep+0 * 32.0, 0x1.8p+52, 0x1.c6af84b912394p-5 / 32768.0,
                                         0x1.ebfce50fac4f3p-3 / 1024.0, 0x1.62e42ff0c52d6p-1 / 32.0};

// The 2^(i/32) table is indexed per lane, so it is staged in shared memory (constant memory would serialise
// divergent indices).  A kernel that calls exact_expf / expf_core runs load_exp2_table and a block barrier first.
static __shared__ unsigned long long s_exp2_tab[32];

__device__ __forceinline__ void load_exp2_table() {
    for (int i = threadIdx.x; i < 32; i += blockDim.x) s_exp2_tab[i] = c_exp2_tab[i];
}

// e^x for |x| < 88 (no overflow, underflow or NaN handling), operation for operation the definition: 12 FP64
// operations, two conversions
__device__ __forceinline__ float expf_steps(float x) {
    const double z = __dmul_rn(c_exp_k[0], double(x));
    double kd = __dadd_rn(z, c_exp_k[1]);
    const unsigned long long ki = (unsigned long long) __double_as_longlong(kd);
    kd = __dsub_rn(kd, c_exp_k[1]);
    const double r = __dsub_rn(z, kd);
    const unsigned long long t = s_exp2_tab[ki & 31] + (ki << 47);
    const double s = __longlong_as_double((long long) t);
    const double p = __dadd_rn(__dmul_rn(c_exp_k[2], r), c_exp_k[3]);
    const double r2 = __dmul_rn(r, r);
    double y = __dadd_rn(__dmul_rn(c_exp_k[4], r), 1.0);
    y = __dadd_rn(__dmul_rn(p, r2), y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

// The same function in 8 FP64 operations: the reduction as above (so k and r are the definition's), the cubic as
// a fused Horner chain.  The two doubles differ by at most 2 units in the last place and the FLOAT they round to is
// the same for EVERY float |x| < 88: checked by enumerating all 2 x 0x42b00000 inputs, on the CPU
// (tests/cpp/expf_fma_exhaustive.c) and on the device (fnb_selftest_expf).  Fusing the reduction too
// (r = fma(x, N/ln2, -k)) is NOT equivalent: two inputs round differently.
// NEG: returns -e^x (the sign rides on the last product: rounding is symmetric, so it is exactly the negated result)
template <bool NEG>
__device__ __forceinline__ float expf_core_signed(float x) {
    const double z = __dmul_rn(c_exp_k[0], double(x));
    double kd = __dadd_rn(z, c_exp_k[1]);
    const unsigned long long ki = (unsigned long long) __double_as_longlong(kd);
    kd = __dsub_rn(kd, c_exp_k[1]);
    const double r = __dsub_rn(z, kd);
    const unsigned long long t = s_exp2_tab[ki & 31] + (ki << 47);
    const double s = __longlong_as_double((long long) t);
    double q = __fma_rn(c_exp_k[2], r, c_exp_k[3]);
    q = __fma_rn(q, r, c_exp_k[4]);
    return __double2float_rn(__dmul_rn(__fma_rn(q, r, 1.0), NEG ? -s : s));
}
__device__ __forceinline__ float expf_core(float x) { return expf_core_signed<false>(x); }

static __device__ __noinline__ float expf_special(float x) {
    const uint32_t bits = __float_as_uint(x);
    if (bits == 0xff800000u) return 0.0f;
    if ((bits & 0x7fffffffu) >= 0x7f800000u) return __fadd_rn(x, x);
    if (x > 0x1.62e42ep6f) return __uint_as_float(0x7f800000u);
    if (x < -0x1.9fe368p6f) return 0.0f;
    if (x < -0x1.9d1d9ep6f) return 0x1p-149f;
    return expf_steps(x);
}

// e^x for every float, special cases included
__device__ __forceinline__ float exact_expf(float x) {
    return (__float_as_uint(x) & 0x7fffffffu) >= 0x42b00000u ? expf_special(x) : expf_steps(x);  // |x| >= 88 or NaN
}

// sine polynomial on the reduced argument
__device__ __forceinline__ float sin_poly(double x, double x2) {
    const double s1 = -0x1.555545995a603p-3, s2 = 0x1.1107605230bc4p-7, s3 = -0x1.994eb3774cf24p-13;
    const double x3 = __dmul_rn(x, x2);
    const double t = __dadd_rn(s2, __dmul_rn(x2, s3));
    const double x7 = __dmul_rn(x3, x2);
    const double s = __dadd_rn(x, __dmul_rn(x3, s1));
    return __double2float_rn(__dadd_rn(s, __dmul_rn(x7, t)));
}
// cosine polynomial; neg flips every coefficient (quadrants where the cosine term is negative)
__device__ __forceinline__ float cos_poly(double x2, bool neg) {
    const double sg = neg ? -1.0 : 1.0;
    const double c0 = sg, c1 = __dmul_rn(sg, -0x1.ffffffd0c621cp-2), c2 = __dmul_rn(sg, 0x1.55553e1068f19p-5);
    const double c3 = __dmul_rn(sg, -0x1.6c087e89a359dp-10), c4 = __dmul_rn(sg, 0x1.99343027bf8c3p-16);
    const double x4 = __dmul_rn(x2, x2);
    const double hi = __dadd_rn(c3, __dmul_rn(x2, c4));
    const double lo = __dadd_rn(c0, __dmul_rn(x2, c1));
    const double x6 = __dmul_rn(x4, x2);
    const double c = __dadd_rn(lo, __dmul_rn(x4, c2));
    return __double2float_rn(__dadd_rn(c, __dmul_rn(x6, hi)));
}

// sin(y) and cos(y) together; the argument reduction is shared, which changes no result bit because both
// functions reduce identically.
__device__ __forceinline__ void exact_sincosf(float y, float * sn, float * cs) {
    const uint32_t iy = __float_as_uint(y);
    const uint32_t top = (iy >> 20) & 0x7ffu;
    double x = double(y);
    if (top < 0x3f4u) {  // |y| < pi/4
        if (top < 0x398u) {  // |y| < 2^-12
            *sn = y;
            *cs = 1.0f;
            return;
        }
        const double x2 = __dmul_rn(x, x);
        *sn = sin_poly(x, x2);
        *cs = cos_poly(x2, false);
        return;
    }
    int n, sign_bit = 0;
    if (top < 0x42fu) {  // |y| < 120: one multiply-subtract against pi/2
        const double r = __dmul_rn(x, 0x1.45F306DC9C883p+23);
        n = (__double2int_rz(r) + 0x800000) >> 24;
        x = __dsub_rn(x, __dmul_rn(double(n), 0x1.921FB54442D18p0));
    } else if (top < 0x7f8u) {  // large: 96 bits of 4/pi against the 24-bit significand
        const uint32_t * arr = &c_inv_pio4[(iy >> 26) & 15u];
        const int sh = int((iy >> 23) & 7u);
        uint32_t m = (iy & 0xffffffu) | 0x800000u;
        m <<= sh;
        unsigned long long res0 = (unsigned long long) (uint32_t) (m * arr[0]);
        const unsigned long long res1 = (unsigned long long) m * arr[4];
        const unsigned long long res2 = (unsigned long long) m * arr[8];
        res0 = (res2 >> 32) | (res0 << 32);
        res0 += res1;
        const unsigned long long q = (res0 + (1ULL << 61)) >> 62;
        res0 -= q << 62;
        x = __dmul_rn(__ll2double_rn((long long) res0), 0x1.921FB54442D18p-62);
        n = int(q);
        sign_bit = int(iy >> 31);
    } else {  // infinity or NaN
        *sn = *cs = __fsub_rn(y, y);
        return;
    }
    const int quad = n + sign_bit;
    const bool flip = ((quad & 3) == 1) || ((quad & 3) == 2);
    const double xs = flip ? -x : x;
    const double x2 = __dmul_rn(x, x);
    const bool neg = (quad & 2) != 0;
    const float ps = sin_poly(xs, x2);
    const float pc = cos_poly(x2, neg);
    // even n: sine takes the sine polynomial; odd n: the two swap
    *sn = (n & 1) ? pc : ps;
    *cs = (n & 1) ? ps : pc;
}

}  // namespace fnb
