/*
 * TEST INFRASTRUCTURE.  The CPU oracle: a plain-C restatement of the reference's CPU definition of the fused
 * row-wise hot path.  Only tests, the smoke check and the bench's CPU-baseline leg may call it; the product
 * library never does.
 *
 * Each function's comment in fnb_oracle.c names the reference lines it follows.  Block layouts are ggml's
 * (ggml/src/ggml-common.h:258-276 Q8_0 / Q8_1, :334-345 Q4_K, :414-418 IQ3_XXS).
 */
#ifndef FNB_ORACLE_H
#define FNB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNBO_ERR_TOKEN 1u /* a token id outside [0, n_vocab) */
#define FNBO_ERR_SLOT 2u  /* a cache slot outside [0, cache_slots) */

/* 0 = restated exact expf / sinf / cosf (default), 1 = the host libm's */
void fnbo_use_libm(int on);

uint16_t fnbo_f32_to_f16(float f);
float fnbo_f16_to_f32(uint16_t h);
float fnbo_expf_exact(float x);
float fnbo_sinf_exact(float x);
float fnbo_cosf_exact(float x);

void fnbo_quantize_row_q8_0(const float * x, void * y, int64_t k);
void fnbo_quantize_row_q8_1(const float * x, void * y, int64_t k);
void fnbo_dequantize_row_q8_0(const void * x, float * y, int64_t k);
void fnbo_dequantize_row_q4_k(const void * x, float * y, int64_t k);
void fnbo_dequantize_row_iq3_xxs(const void * x, float * y, int64_t k);
void fnbo_dequantize_row_iq3_s(const void * x, float * y, int64_t k);

/* get_rows: out[t] = dequantised row ids[t]; a bad id sets FNBO_ERR_TOKEN in *err and leaves the row unwritten */
void fnbo_get_rows_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                        int64_t rows, int32_t cols);
void fnbo_get_rows_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                           int64_t rows, int32_t cols);

/* y = (x * scale) * w, scale = 1/sqrtf(mean(x^2) + eps); w may be NULL (no weight) */
void fnbo_rms_norm_f32(const float * x, const float * w, float eps, float * y, int64_t rows, int32_t cols);

/* out block b of row r = Q8_1(silu(gate) * up); f32_out (optional) takes the unquantised product */
void fnbo_swiglu_q8_1(const float * gate, const float * up, void * out_q8_1, float * f32_out, int64_t rows,
                      int32_t cols);

typedef struct fnbo_rope_kv_args {
    const float * q;         /* [rows][n_q_heads][head_dim] */
    const float * k;         /* [rows][n_kv_heads][head_dim] */
    const float * v;         /* [rows][n_kv_heads][head_dim] */
    const int32_t * pos;     /* [rows] rotary position */
    const int32_t * slots;   /* [rows] cache slot, or NULL: the slot is the position */
    const float * q_norm_w;  /* [head_dim] or NULL: no per-head norm on q */
    const float * k_norm_w;  /* [head_dim] or NULL */
    float * q_out;           /* [rows][n_q_heads][head_dim] */
    void * k_cache;          /* Q8_0 [cache_slots][n_kv_heads][head_dim / 32] */
    void * v_cache;
    float * k_f32;           /* optional [rows][n_kv_heads][head_dim]: k after norm and rope, before quantising */
    uint32_t * err;
    int64_t rows;
    int64_t cache_slots;
    int32_t n_q_heads, n_kv_heads, head_dim, n_rot;
    float theta_scale;       /* powf(freq_base, -2.0f / n_rot) */
    float eps;
    const int32_t * planes;  /* optional [rows][4]: rotary position planes (fn/kernels/qsa/imrope.cuh:15-24) */
} fnbo_rope_kv_args;

void fnbo_rope_neox_q8_0_append(const fnbo_rope_kv_args * a);
float fnbo_theta_scale(float freq_base, int32_t n_rot);

/* "next" formats of the reference's own GPU path */
/* FNFL activation format: codes int8 [rows][k], scales {d, s} F32 [rows][k/32][2] */
void fnbo_act_quantize(const float * x, int64_t rows, int32_t k, int8_t * codes, float * scales);
void fnbo_swiglu_act(const float * gate, const float * up, int8_t * codes, float * scales, float * f32_out,
                     int64_t rows, int32_t cols);
/* KV8: groups of 64, codes int8 [n], FP16 scale bits [n / 64] */
void fnbo_kv8_quantize(const float * x, int64_t n, int8_t * codes, uint16_t * scales);

/* ggml's Q8_K activation blocks (292 bytes per 256 values: F32 d, 256 codes, 16 sums of 16 codes): the format the
 * routed experts' gate / up mat-vec reads (fn/kernels/experts/cpu_kernels.h block_q8_k; experts_cpu.cpp:321).
 * Follows quantize_row_q8_K_ref (ggml/src/ggml-quants.c:2844-2881): the value of largest magnitude (the FIRST one on
 * ties) maps to -127, codes are nearest-even(iscale x) capped at 127, d = 1 / iscale. */
void fnbo_quantize_row_q8_k(const float * x, void * y, int64_t k);

/* The routed experts' gate / up mat-vec with the GLU fused, ff[t][r] = silu(g) u with g = gate row r . act[t] and
 * u = up row r . act[t]: ggml Q4_K weights (n / 256 super-blocks of 144 bytes a row, row r of either matrix at
 * base + r row_bytes) against Q8_K activations (act + t act_stride).  Follows the reference's AVX2 kernels lane for
 * lane (fn/kernels/experts/cpu_kq_avx2.cpp:166-224 q4k_dot, :362-380 kq_gu_rows): per (row, t) eight int32 lanes of
 * scale-weighted 4-byte dot products per super-block, fused-multiply-added as floats with d = y.d x.d; four lanes of
 * mins x block sums with -y.d x.dmin; hsum_float_8 plus ((m0 + m2) + (m1 + m3)); then g / (1 + expf(-g)) * u.
 * gu: optional [2][nt][rows] receiving g and u themselves. */
void fnbo_expert_gu_rows_q4_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                              int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                              int64_t r1);

/* The same with ggml Q5_K weights (n / 256 super-blocks of 176 bytes a row): fn/kernels/experts/cpu_kq_avx2.cpp:226-290
 * q5k_dot - the Q4_K lane structure over 5-bit values (high bits from qh), the mins as one scalar fused multiply-add a
 * super-block, hsum_float_8(acc) + summs. */
void fnbo_expert_gu_rows_q5_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                              int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                              int64_t r1);

/* The same with ggml IQ3_XXS weights (n / 256 super-blocks of 98 bytes a row): the reference's AVX2 row kernel lane for
 * lane (fn/kernels/experts/cpu_iq_avx2.cpp:256-271, :305-337, :429-445) - eight int32 lanes a super-block of
 * (2 s + 1) x codebook bytes x sign-applied Q8_K codes, one fused multiply-add a super-block with (x.d y.d), ggml's
 * hsum_float_8 order, the format's 1/4 applied to the reduced sum, then g / (1 + expf(-g)) * u. */
void fnbo_expert_gu_rows_iq3_xxs(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                                 int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                 int64_t r1);

/* And with ggml IQ3_S weights (110-byte super-blocks; cpu_iq_avx2.cpp:273-290 through the same row kernel): 9-bit
 * codebook indices, plain sign bits, one 4-bit scale per 32 values, K = 1. */
void fnbo_expert_gu_rows_iq3_s(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                               int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                               int64_t r1);

/* The consumer of the 8-bit activations: the routed experts' down mat-vec, out[t][r] = weight row r . act[t], with
 * ggml's Q5_1 weights against Q8_1 activations (fmt 0) or Q8_0 weights against Q8_0 activations (fmt 1).  Follows the
 * reference's CPU kernels lane for lane (fn/kernels/experts/cpu_kq_avx2.cpp:293-344, :382-394): eight F32 accumulators
 * per (row, t), accumulator j taking bytes 4 j .. 4 j + 3 of every block by one fused multiply-add per block, reduced
 * once at the end in hsum_float_8's order (:103-109).  fmt 2: ggml IQ4_NL weights (18-byte blocks: fp16 d, 16 nibble
 * bytes indexing kvalues_iq4nl) against Q8_0 activations, fn/kernels/experts/cpu_iq_avx2.cpp:481-514: |w| times the
 * code with w's sign applied (a -128 code stays -128), reduced in that file's hsum8 order (:187-193).  w: rows of n / 32 blocks, row r at w + r row_bytes; act: nt rows of
 * n / 32 activation blocks, row t at act + t act_stride; out[t * out_stride + r] for r in [r0, r1). */
void fnbo_expert_down_rows(int32_t fmt, const uint8_t * w, int64_t row_bytes, int32_t n, const uint8_t * act,
                           int64_t act_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1);

/* The reference's planar 32-value activation (fn/kernels/experts/cpu_q2_avx2.cpp:180-226): per chunk of 32 values
 * s = amax / 127, codes trunc(x / s +- 0.5) in +-127 (half away from zero), and the down mat-vec of its Q2_0 weights
 * (64-weight blocks of 18 bytes, weight d (c - 1); :62-102): out[t][r] for r in [r0, r1), n a multiple of 128. */
void fnbo_quantize_act_q(const float * x, int64_t n, int8_t * q, float * scale);
void fnbo_expert_down_rows_q2_0(const uint8_t * w, int64_t row_bytes, int32_t n, const int8_t * q, int64_t q_stride,
                                const float * scale, int64_t scale_stride, int32_t nt, float * out, int64_t out_stride,
                                int64_t r0, int64_t r1);

/* The experts' gate / up rows with the IQ2 formats; fmt is ggml's type number: 16 IQ2_XXS, 17 IQ2_XS, 22 IQ2_S */
void fnbo_expert_gu_rows_iq2(int32_t fmt, const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n,
                             const uint8_t * act, int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu,
                             int64_t r0, int64_t r1);

/* Decode attention in FP64 over already decoded cache rows (the reference's test protocol, fn/kernels/qsa/
 * qa2_test.cpp:469-520, written from the definition in fn/kernels/qsa/attend.h:9-23): for row t and query head h,
 * out = softmax_c(scale q . K[c][g]) . V[c][g] over cells first[t] .. first[t] + count[t] - 1, g = h / (n_q / n_kv),
 * times sigmoid(gate) when gate is given.  k, v: F32 [cells][n_kv][hd] (cell index = absolute cache cell); out: F64. */
void fnbo_attend_f64(const float * q, const float * gate, const float * k, const float * v, const int32_t * first,
                     const int32_t * count, int32_t rows, int32_t n_q, int32_t n_kv, int32_t hd, double scale, double * out);

#ifdef __cplusplus
}
#endif
#endif
