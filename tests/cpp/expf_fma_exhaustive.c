/* Enumerates every float |x| < 88 (both signs) and compares two evaluations of the single-precision e^x algorithm the
 * oracle restates (2^(k/32) table, cubic in double): the definition's order of operations, and the one the CUDA
 * kernels' fast path uses (same reduction, the cubic as a fused Horner chain).  Prints the largest difference of the
 * two doubles in units in the last place and the number of inputs whose FLOAT results differ; exits 0 only when that
 * number is 0.  Also evaluates the variant that fuses the reduction as well, to show that it is NOT equivalent.
 * Build: gcc -O2 -mfma -ffp-contract=off expf_fma_exhaustive.c -lm -lpthread   (threads: argv[1], default 8) */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../oracle/fnb_exact_math.h"

static const double k_inv = 0x1.71547652b82fep+0 * 32.0, k_shift = 0x1.8p+52;
static const double k_c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, k_c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
static const double k_c2 = 0x1.62e42ff0c52d6p-1 / 32.0;

typedef struct {
    uint32_t lo, hi;
    int64_t max_ulp;
    uint64_t differ, differ_fused_reduction;
} job;

static void * run(void * p) {
    job * j = (job *) p;
    for (uint64_t b = j->lo; b < j->hi; ++b) {
        for (int sg = 0; sg < 2; ++sg) {
            const float x = fnbo_f32_bits((uint32_t) b | (sg ? 0x80000000u : 0u));
            const float want = fnbo_expf(x);
            const double z = k_inv * (double) x;
            double kd = z + k_shift;
            const uint64_t ki = fnbo_bits_f64(kd);
            kd -= k_shift;
            const double r = z - kd;
            const double s = fnbo_f64_bits(fnbo_exp2_tab[ki & 31] + (ki << 47));
            double y = k_c2 * r + 1.0;
            y = (k_c0 * r + k_c1) * (r * r) + y;
            y = y * s;
            double q = fma(fma(k_c0, r, k_c1), r, k_c2);
            const double yf = fma(q, r, 1.0) * s;
            int64_t d = (int64_t) fnbo_bits_f64(y) - (int64_t) fnbo_bits_f64(yf);
            if (d < 0) d = -d;
            if (d > j->max_ulp) j->max_ulp = d;
            j->differ += fnbo_bits_f32((float) yf) != fnbo_bits_f32(want);
            /* reduction fused too */
            double kd2 = fma(k_inv, (double) x, k_shift);
            const uint64_t ki2 = fnbo_bits_f64(kd2);
            kd2 -= k_shift;
            const double r2 = fma(k_inv, (double) x, -kd2);
            const double s2 = fnbo_f64_bits(fnbo_exp2_tab[ki2 & 31] + (ki2 << 47));
            q = fma(fma(k_c0, r2, k_c1), r2, k_c2);
            j->differ_fused_reduction += fnbo_bits_f32((float) (fma(q, r2, 1.0) * s2)) != fnbo_bits_f32(want);
        }
    }
    return 0;
}

int main(int argc, char ** argv) {
    int nt = argc > 1 ? atoi(argv[1]) : 8;
    if (nt < 1 || nt > 256) nt = 8;
    pthread_t * th = (pthread_t *) malloc(sizeof(pthread_t) * nt);
    job * jobs = (job *) calloc(nt, sizeof(job));
    const uint64_t end = 0x42b00000u; /* 88.0f */
    for (int i = 0; i < nt; ++i) {
        jobs[i].lo = (uint32_t) (end * i / nt), jobs[i].hi = (uint32_t) (end * (i + 1) / nt);
        pthread_create(&th[i], 0, run, &jobs[i]);
    }
    job t;
    memset(&t, 0, sizeof t);
    for (int i = 0; i < nt; ++i) {
        pthread_join(th[i], 0);
        if (jobs[i].max_ulp > t.max_ulp) t.max_ulp = jobs[i].max_ulp;
        t.differ += jobs[i].differ, t.differ_fused_reduction += jobs[i].differ_fused_reduction;
    }
    printf("inputs %llu max_double_ulp %lld float_differ %llu float_differ_fused_reduction %llu\n",
           (unsigned long long) (2 * end), (long long) t.max_ulp, (unsigned long long) t.differ,
           (unsigned long long) t.differ_fused_reduction);
    return t.differ == 0 ? 0 : 1;
}
