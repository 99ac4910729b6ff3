/*
 * TEST INFRASTRUCTURE - part of the CPU oracle, never linked into the product library.
 *
 * Portable restatements of the three libm functions the hot path's CPU definition calls
 * (expf in SwiGLU, sinf/cosf in RoPE).  The reference tree does not vendor a libm: its CPU code calls the
 * platform's (fn/kernels/experts/cpu_iq_avx2.cpp:442 `expf`; the rope definition cited at
 * fn/kernels/qsa/attend.h:12-23 `cosf`/`sinf`).  The dependency is therefore named here: GNU libc 2.39
 * (flt-32 expf / sinf / cosf, which are the Arm Optimized Routines single-precision algorithms: table-driven
 * 2^(k/32) with a cubic in double for expf; double-precision Cody-Waite / 4-over-pi reduction with degree-7/8
 * polynomials for sinf and cosf).  The algorithm is restated below in plain IEEE double arithmetic with no
 * contracted multiply-adds (build with -ffp-contract=off), so the result is a pure function of the input
 * bits on every host - and on the GPU, which evaluates the same operations in the same order.
 *
 * Pinned by tests/test_exact_math.py: bit-for-bit equal to this container's glibc on dense sweeps of the
 * argument ranges the kernels use (glibc's x86-64 ifunc may pick an FMA-contracted build of the same
 * algorithm, which can differ in about one input per 10^8; the test reports that rate).
 */
#ifndef FNB_EXACT_MATH_H
#define FNB_EXACT_MATH_H

#include <stdint.h>
#include <string.h>

#include "../fnfl_v100_b200/csrc/exact_math_tables.inc"

static inline uint32_t fnbo_bits_f32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float fnbo_f32_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint64_t fnbo_bits_f64(double f) { uint64_t u; memcpy(&u, &f, 8); return u; }
static inline double fnbo_f64_bits(uint64_t u) { double f; memcpy(&f, &u, 8); return f; }

static const uint64_t fnbo_exp2_tab[32] = FNB_EXP2_TABLE_INIT;
static const uint32_t fnbo_inv_pio4[24] = FNB_INV_PIO4_INIT;

/* e^x, single precision.  x N/ln2 = k + r, |r| <= 1/2, N = 32; e^x = 2^(k/N) (1 + c2 r + c1 r^2 + c0 r^3). */
static inline float fnbo_expf(float x) {
    const uint32_t ax = fnbo_bits_f32(x) & 0x7fffffffu;
    if (ax >= 0x42b00000u) { /* |x| >= 88 or NaN */
        if (fnbo_bits_f32(x) == 0xff800000u) return 0.0f;
        if (ax >= 0x7f800000u) return x + x;
        if (x > 0x1.62e42ep6f) return fnbo_f32_bits(0x7f800000u);
        if (x < -0x1.9fe368p6f) return 0.0f;
        if (x < -0x1.9d1d9ep6f) return 0x1p-149f; /* the algorithm's may-underflow result */
    }
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double z = inv_ln2_n * (double) x;
    double kd = z + shift;
    const uint64_t ki = fnbo_bits_f64(kd);
    kd -= shift;
    const double r = z - kd;
    const uint64_t t = fnbo_exp2_tab[ki & 31] + (ki << 47);
    const double s = fnbo_f64_bits(t);
    const double p = c0 * r + c1;
    const double r2 = r * r;
    double y = c2 * r + 1.0;
    y = p * r2 + y;
    y = y * s;
    return (float) y;
}

/* polynomial pair on the reduced argument, |x| <= pi/4; neg_cos flips the cosine's sign (quadrants 2, 3) */
static inline float fnbo_sincos_poly(double x, double x2, int use_cos, int neg_cos) {
    if (!use_cos) {
        const double s1 = -0x1.555545995a603p-3, s2 = 0x1.1107605230bc4p-7, s3 = -0x1.994eb3774cf24p-13;
        const double x3 = x * x2;
        const double t = s2 + x2 * s3;
        const double x7 = x3 * x2;
        const double s = x + x3 * s1;
        return (float) (s + x7 * t);
    } else {
        const double sg = neg_cos ? -1.0 : 1.0;
        const double c0 = sg * 0x1p0, c1 = sg * -0x1.ffffffd0c621cp-2, c2 = sg * 0x1.55553e1068f19p-5;
        const double c3 = sg * -0x1.6c087e89a359dp-10, c4 = sg * 0x1.99343027bf8c3p-16;
        const double x4 = x2 * x2;
        const double hi = c3 + x2 * c4;
        const double lo = c0 + x2 * c1;
        const double x6 = x4 * x2;
        const double c = lo + x4 * c2;
        return (float) (c + x6 * hi);
    }
}

/* common body: which = 0 sine, 1 cosine */
static inline float fnbo_sincosf_one(float y, int which) {
    const uint32_t iy = fnbo_bits_f32(y);
    const uint32_t top = (iy >> 20) & 0x7ff;
    double x = (double) y;
    if (top < 0x3f4) { /* |y| < pi/4 (compared on the top 12 bits, as the algorithm does) */
        const double x2 = x * x;
        if (top < 0x398) { /* |y| < 2^-12 */
            return which ? 1.0f : y;
        }
        return fnbo_sincos_poly(x, x2, which, 0);
    }
    int n;
    int sign_bit = 0;
    if (top < 0x42f) { /* |y| < 120 */
        const double r = x * 0x1.45F306DC9C883p+23;
        n = (int) (((int32_t) r + 0x800000) >> 24);
        x = x - (double) n * 0x1.921FB54442D18p0;
    } else if (top < 0x7f8) {
        const uint32_t * arr = &fnbo_inv_pio4[(iy >> 26) & 15];
        const int sh = (int) ((iy >> 23) & 7);
        uint32_t m = (iy & 0xffffffu) | 0x800000u;
        m <<= sh;
        uint64_t res0 = (uint64_t) (uint32_t) (m * arr[0]);
        const uint64_t res1 = (uint64_t) m * arr[4];
        const uint64_t res2 = (uint64_t) m * arr[8];
        res0 = (res2 >> 32) | (res0 << 32);
        res0 += res1;
        const uint64_t q = (res0 + (1ULL << 61)) >> 62;
        res0 -= q << 62;
        x = (double) (int64_t) res0 * 0x1.921FB54442D18p-62;
        n = (int) q;
        sign_bit = (int) (iy >> 31);
    } else {
        return y - y; /* inf or NaN -> NaN */
    }
    const int quad = n + sign_bit;
    const double sgn = ((quad & 3) == 1 || (quad & 3) == 2) ? -1.0 : 1.0;
    return fnbo_sincos_poly(x * sgn, x * x, (n ^ which) & 1, (quad & 2) != 0);
}

static inline float fnbo_sinf(float y) { return fnbo_sincosf_one(y, 0); }
static inline float fnbo_cosf(float y) { return fnbo_sincosf_one(y, 1); }

#endif
