/*
 * TEST INFRASTRUCTURE.  CPU oracle for the fused row-wise hot path: a plain-C restatement of the reference's
 * CPU definition, written to be read next to the reference lines each function cites.  Build with
 * -ffp-contract=off and without -march=native: several results depend on a multiply and an add staying two
 * roundings (fn/quant/decode.h:5-6 makes the same requirement of the reference's own decoders).
 *
 * Pinning.  The quantisers and decoders are checked bit-for-bit against the reference's own C
 * (ggml/src/ggml-quants.c compiled from the reference tree into oracle/_ref, see oracle/Makefile) and against
 * the golden vectors that build produced (tests/golden).  rms_norm, swiglu and rope have no CPU source in the
 * reference tree (its ggml carries no CPU backend): they follow the lines cited on each function and are
 * pinned at tolerance level by FP64 restatements of the reference's own tests, not bit-for-bit.
 */
#include "fnb_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "fnb_exact_math.h"

static int g_use_libm = 0;
void fnbo_use_libm(int on) { g_use_libm = on; }

float fnbo_expf_exact(float x) { return fnbo_expf(x); }
float fnbo_sinf_exact(float x) { return fnbo_sinf(x); }
float fnbo_cosf_exact(float x) { return fnbo_cosf(x); }

static inline float o_expf(float x) { return g_use_libm ? expf(x) : fnbo_expf(x); }
static inline float o_sinf(float x) { return g_use_libm ? sinf(x) : fnbo_sinf(x); }
static inline float o_cosf(float x) { return g_use_libm ? cosf(x) : fnbo_cosf(x); }

/* ---- FP16 <-> FP32: IEEE round-to-nearest-even; NaN -> 0x7E00 with the sign, as
 * ggml/src/ggml-impl.h:412-438 (ggml_compute_fp32_to_fp16) produces; widening is exact (:391-410). ---- */
uint16_t fnbo_f32_to_f16(float f) {
    const uint32_t x = fnbo_bits_f32(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return (uint16_t) (sign | 0x7e00u);
    if (ax >= 0x477ff000u) return (uint16_t) (sign | 0x7c00u); /* rounds to 2^16 or beyond: inf */
    if (ax < 0x33000001u) return (uint16_t) sign;              /* <= 2^-25: ties-to-even gives zero */
    const int32_t e = (int32_t) (ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    uint32_t shift, base;
    if (e < -14) { /* FP16 subnormal: value = man * 2^(e-23), unit 2^-24 */
        shift = (uint32_t) (-e - 1); /* 23 - (e + 24) */
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t) (e + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    h += base;
    if (rem > half || (rem == half && (h & 1u))) ++h;
    return (uint16_t) (sign | h);
}

float fnbo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t) (h & 0x8000u) << 16;
    const uint32_t ex = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (ex == 0) {
        if (man == 0) return fnbo_f32_bits(sign);
        const float v = (float) man * 0x1p-24f; /* exact */
        return fnbo_f32_bits(fnbo_bits_f32(v) | sign);
    }
    if (ex == 31) return fnbo_f32_bits(sign | 0x7f800000u | (man << 13));
    return fnbo_f32_bits(sign | ((ex + 112u) << 23) | (man << 13));
}

/* C's (int8_t) of a rounded float goes through a 32-bit convert on x86-64: out of range or NaN gives
 * INT32_MIN, whose low byte is 0.  Stated explicitly so the rule is the same on every target. */
static inline int8_t o_to_i8(float r) {
    if (!(r > -2147483904.0f && r < 2147483648.0f)) return 0;
    return (int8_t) (uint8_t) ((uint32_t) (int32_t) r & 0xffu);
}

/* ---- Q8_0: ggml/src/ggml-quants.c:274-297 (quantize_row_q8_0_ref) ---- */
void fnbo_quantize_row_q8_0(const float * x, void * yv, int64_t k) {
    uint8_t * y = (uint8_t *) yv;
    for (int64_t b = 0; b < k / 32; ++b) {
        const float * v = x + 32 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) {
            const float a = fabsf(v[j]);
            amax = amax > a ? amax : a;
        }
        const float d = amax / 127.0f;
        const float id = d ? 1.0f / d : 0.0f;
        const uint16_t dh = fnbo_f32_to_f16(d);
        memcpy(y + 34 * b, &dh, 2);
        for (int j = 0; j < 32; ++j) {
            ((int8_t *) y)[34 * b + 2 + j] = o_to_i8(roundf(v[j] * id));
        }
    }
}

/* ---- Q8_1: ggml/src/ggml-quants.c:300-333 (quantize_row_q8_1_ref); s = fp16(sum * d), d unrounded ---- */
void fnbo_quantize_row_q8_1(const float * x, void * yv, int64_t k) {
    uint8_t * y = (uint8_t *) yv;
    for (int64_t b = 0; b < k / 32; ++b) {
        const float * v = x + 32 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) {
            const float a = fabsf(v[j]);
            amax = amax > a ? amax : a;
        }
        const float d = amax / 127.0f;
        const float id = d ? 1.0f / d : 0.0f;
        const uint16_t dh = fnbo_f32_to_f16(d);
        int sum = 0;
        for (int j = 0; j < 32; ++j) {
            const int8_t q = o_to_i8(roundf(v[j] * id));
            ((int8_t *) y)[36 * b + 4 + j] = q;
            sum += q;
        }
        const uint16_t sh = fnbo_f32_to_f16((float) sum * d);
        memcpy(y + 36 * b, &dh, 2);
        memcpy(y + 36 * b + 2, &sh, 2);
    }
}

/* ---- ggml/src/ggml-quants.c:551-565 ---- */
void fnbo_dequantize_row_q8_0(const void * xv, float * y, int64_t k) {
    const uint8_t * x = (const uint8_t *) xv;
    for (int64_t b = 0; b < k / 32; ++b) {
        uint16_t dh;
        memcpy(&dh, x + 34 * b, 2);
        const float d = fnbo_f16_to_f32(dh);
        for (int j = 0; j < 32; ++j) y[32 * b + j] = (float) ((const int8_t *) x)[34 * b + 2 + j] * d;
    }
}

/* ---- Q4_K: ggml/src/ggml-quants.c:1527-1549 with the 6-bit scale/min unpack of :878-886; the same rule is
 * stated independently at fn/quant/decode.cpp:88-106.  y = d*sc*q - dmin*m, product then subtract. ---- */
static inline void o_scale_min_k4(int j, const uint8_t * s, uint8_t * sc, uint8_t * m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t) ((s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t) ((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

void fnbo_dequantize_row_q4_k(const void * xv, float * y, int64_t k) {
    const uint8_t * x = (const uint8_t *) xv;
    for (int64_t b = 0; b < k / 256; ++b, x += 144) {
        uint16_t dh, mh;
        memcpy(&dh, x, 2);
        memcpy(&mh, x + 2, 2);
        const float d = fnbo_f16_to_f32(dh), dmin = fnbo_f16_to_f32(mh);
        const uint8_t * scales = x + 4;
        const uint8_t * q = x + 16;
        for (int g = 0; g < 4; ++g) {
            uint8_t sc, m;
            o_scale_min_k4(2 * g, scales, &sc, &m);
            const float d1 = d * (float) sc, m1 = dmin * (float) m;
            o_scale_min_k4(2 * g + 1, scales, &sc, &m);
            const float d2 = d * (float) sc, m2 = dmin * (float) m;
            for (int l = 0; l < 32; ++l) *y++ = d1 * (float) (q[l] & 0x0f) - m1;
            for (int l = 0; l < 32; ++l) *y++ = d2 * (float) (q[l] >> 4) - m2;
            q += 32;
        }
    }
}

/* ---- IQ3_XXS: ggml/src/ggml-quants.c:2573-2601; codebook ggml/src/ggml-common.h:1062, sign rule :554-567
 * (7 stored sign bits, the eighth is their parity); independently at fn/quant/decode.cpp:224-242. ---- */
static const uint16_t o_grid_packed[256] = {
#include "../fnfl_v100_b200/csrc/iq3xxs_grid_packed.inc"
};

static inline float o_grid_mag(unsigned level) { return level == 7 ? 62.0f : (float) (4 + 8 * level); }

void fnbo_dequantize_row_iq3_xxs(const void * xv, float * y, int64_t k) {
    const uint8_t * x = (const uint8_t *) xv;
    for (int64_t b = 0; b < k / 256; ++b, x += 98) {
        uint16_t dh;
        memcpy(&dh, x, 2);
        const float d = fnbo_f16_to_f32(dh);
        const uint8_t * qs = x + 2;
        const uint8_t * sas = x + 2 + 64;
        for (int ib = 0; ib < 8; ++ib) {
            uint32_t aux;
            memcpy(&aux, sas + 4 * ib, 4);
            const float db = d * (0.5f + (float) (aux >> 28)) * 0.5f;
            for (int l = 0; l < 4; ++l) {
                const unsigned s7 = (aux >> (7 * l)) & 127u;
                const unsigned signs = s7 | ((unsigned) (__builtin_popcount(s7) & 1) << 7);
                for (int h = 0; h < 2; ++h) {
                    const unsigned code = o_grid_packed[qs[8 * ib + 2 * l + h]];
                    for (int j = 0; j < 4; ++j) {
                        const float g = o_grid_mag((code >> (3 * j)) & 7u);
                        const float sg = (signs >> (4 * h + j)) & 1u ? -1.0f : 1.0f;
                        y[4 * h + j] = db * g * sg;
                    }
                }
                y += 8;
            }
        }
    }
}

/* ---- IQ3_S (the reference engine's own embedding format): ggml/src/ggml-quants.c:2605-2644; block
 * ggml/src/ggml-common.h:420-428 {fp16 d, qs[64], qh[8], signs[32], scales[4]}; codebook iq3s_grid (512 entries of
 * four odd magnitudes).  Index n of a block: 9-bit codebook index qs[n] | bit (n % 8) of qh[n / 8] << 8, scale
 * d * (1 + 2 * nibble (n / 8) of scales), sign bits (n % 2) * 4 .. + 3 of signs[n / 2]; independently at
 * fn/quant/decode.cpp (decode_iq3_s) and fn/kernels/dense/iq3s.cuh:53-77. ---- */
static const uint16_t o_grid3s_packed[512] = {
#include "../fnfl_v100_b200/csrc/iq3s_grid_packed.inc"
};

void fnbo_dequantize_row_iq3_s(const void * xv, float * y, int64_t k) {
    const uint8_t * x = (const uint8_t *) xv;
    for (int64_t b = 0; b < k / 256; ++b, x += 110) {
        uint16_t dh;
        memcpy(&dh, x, 2);
        const float d = fnbo_f16_to_f32(dh);
        const uint8_t * qs = x + 2, * qh = x + 66, * signs = x + 74, * scales = x + 106;
        for (int n = 0; n < 64; ++n) {
            const int ib = n / 8, m = n % 8;
            const int nib = (ib & 1) ? scales[ib / 2] >> 4 : scales[ib / 2] & 0x0f;
            const float db = d * (float) (1 + 2 * nib);
            const unsigned code = o_grid3s_packed[qs[n] | (((qh[ib] >> m) & 1u) << 8)];
            const unsigned sg = signs[n / 2] >> (4 * (n & 1));
            for (int j = 0; j < 4; ++j) {
                const float g = (float) (2 * ((code >> (3 * j)) & 7u) + 1);
                y[4 * n + j] = db * g * ((sg >> j) & 1u ? -1.0f : 1.0f);
            }
        }
        y += 256;
    }
}

/* ---- get_rows on a quantised table is the row decoder applied to row ids[t] (the ggml op's definition);
 * the bad-id rule is the reference kernel's: fn/kernels/embed/embed.cu:43-48, embed.h:15-17. ---- */
void fnbo_get_rows_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                        int64_t rows, int32_t cols) {
    const size_t rb = (size_t) (cols / 256) * 144;
    for (int64_t t = 0; t < rows; ++t) {
        if (ids[t] < 0 || ids[t] >= n_vocab) {
            if (err) *err |= FNBO_ERR_TOKEN;
            continue;
        }
        fnbo_dequantize_row_q4_k((const uint8_t *) table + rb * (size_t) ids[t], out + (size_t) t * cols, cols);
    }
}

void fnbo_get_rows_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                           int64_t rows, int32_t cols) {
    const size_t rb = (size_t) (cols / 256) * 98;
    for (int64_t t = 0; t < rows; ++t) {
        if (ids[t] < 0 || ids[t] >= n_vocab) {
            if (err) *err |= FNBO_ERR_TOKEN;
            continue;
        }
        fnbo_dequantize_row_iq3_xxs((const uint8_t *) table + rb * (size_t) ids[t], out + (size_t) t * cols, cols);
    }
}

/* ---- RMSNorm.  The reference mirrors the graph "rms_norm(x) then mul by the weight"
 * (fn/kernels/draft/draft.h:31; fn/kernels/qsa/attend.h:14-15,33): scale = 1/sqrtf(mean + eps),
 * y = (x * scale) * w.  The CPU op it mirrors (ggml's CPU backend, not in the reference tree) sums the F32
 * squares into a double in element order and narrows the mean once; that published rule is restated here.
 * FP64 statements of the same norm: fn/kernels/qsa/qa2_test.cpp:244-252,
 * fn/kernels/draft/draft_prompt_test.cpp:66-75. ---- */
void fnbo_rms_norm_f32(const float * x, const float * w, float eps, float * y, int64_t rows, int32_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float * xr = x + (size_t) r * cols;
        float * yr = y + (size_t) r * cols;
        double sum = 0.0;
        for (int i = 0; i < cols; ++i) sum += (double) (xr[i] * xr[i]);
        const float mean = (float) (sum / cols);
        const float scale = 1.0f / sqrtf(mean + eps);
        if (w) {
            for (int i = 0; i < cols; ++i) yr[i] = (xr[i] * scale) * w[i];
        } else {
            for (int i = 0; i < cols; ++i) yr[i] = xr[i] * scale;
        }
    }
}

/* ---- SwiGLU: silu(g) * u with silu(g) = g / (1 + expf(-g)) in F32, the form every in-tree statement uses
 * (fn/kernels/experts/experts_dev.cuh:197, fn/kernels/dense/dense.cu:148,
 * fn/kernels/experts/cpu_iq_avx2.cpp:442), then the Q8_1 row quantiser over the product. ---- */
static inline float o_swiglu(float g, float u) { return (g / (1.0f + o_expf(-g))) * u; }

void fnbo_swiglu_q8_1(const float * gate, const float * up, void * out, float * f32_out, int64_t rows,
                      int32_t cols) {
    float tmp[32];
    const int64_t nb = rows * (cols / 32);
    for (int64_t b = 0; b < nb; ++b) {
        for (int j = 0; j < 32; ++j) tmp[j] = o_swiglu(gate[32 * b + j], up[32 * b + j]);
        if (f32_out) memcpy(f32_out + 32 * b, tmp, sizeof tmp);
        fnbo_quantize_row_q8_1(tmp, (uint8_t *) out + 36 * b, 32);
    }
}

/* theta_scale = powf(freq_base, -2/n_rot), computed once on the host: fn/kernels/qsa/attend.cu:830-832 */
float fnbo_theta_scale(float freq_base, int32_t n_rot) { return powf(freq_base, -2.0f / (float) n_rot); }

/* ---- per-head norm, NeoX partial RoPE, Q8_0 append.
 * Norm and rope: fn/kernels/qsa/attend.h:19-23 (semantics), attend.cu:153-197 (device form),
 * fn/kernels/qsa/qa2_test.cpp:230-259 (theta as an F32 product chain; pairs (i, i + n_rot/2);
 * x0 c - x1 s, x0 s + x1 c).  Text rows: every rope plane is the position (fn/kernels/qsa/imrope.cuh:7-9),
 * which is plain NeoX.  K = rope(norm(k)), V raw, both appended at the row's cell:
 * fn/kernels/qsa/qsa_prompt_attn.cu:77-122.  The cell format here is ggml Q8_0. ---- */
static void o_head(const float * x, const float * w, float eps, int hd, int n_rot, const float * cs, float * y) {
    if (w) {
        fnbo_rms_norm_f32(x, w, eps, y, 1, hd);
    } else {
        memcpy(y, x, (size_t) hd * sizeof(float));
    }
    const int half = n_rot / 2;
    for (int i = 0; i < half; ++i) {
        const float c = cs[2 * i], s = cs[2 * i + 1];
        const float x0 = y[i], x1 = y[i + half];
        y[i] = x0 * c - x1 * s;
        y[i + half] = x0 * s + x1 * c;
    }
}

void fnbo_rope_neox_q8_0_append(const fnbo_rope_kv_args * a) {
    const int hd = a->head_dim, half = a->n_rot / 2;
    const size_t row_blocks = (size_t) hd / 32;
    float cs[512];
    float tmp[1024];
    for (int64_t t = 0; t < a->rows; ++t) {
        const int64_t slot = a->slots ? a->slots[t] : a->pos[t];
        if (slot < 0 || slot >= a->cache_slots) {
            if (a->err) *a->err |= FNBO_ERR_SLOT;
            continue;
        }
        float theta = (float) a->pos[t];
        for (int i = 0; i < half; ++i) {
            if (a->planes) {
                /* fn/kernels/qsa/imrope.cuh:15-24 (imrope_plane, prompt_rope_pos) and qsa_prompt_attn.cu:56-60: pair i
                 * starts its chain at its own plane's position and multiplies by theta_scale i times */
                const int pl = i % 3 == 1 && i < 33 ? 1 : i % 3 == 2 && i < 30 ? 2 : i % 3 == 0 && i < 33 ? 0 : 3;
                theta = (float) a->planes[4 * t + pl];
                for (int c = 0; c < i; ++c) theta *= a->theta_scale;
            }
            cs[2 * i] = o_cosf(theta);
            cs[2 * i + 1] = o_sinf(theta);
            theta *= a->theta_scale;
        }
        for (int h = 0; h < a->n_q_heads; ++h) {
            const size_t off = ((size_t) t * a->n_q_heads + h) * hd;
            o_head(a->q + off, a->q_norm_w, a->eps, hd, a->n_rot, cs, a->q_out + off);
        }
        for (int h = 0; h < a->n_kv_heads; ++h) {
            const size_t off = ((size_t) t * a->n_kv_heads + h) * hd;
            const size_t cell = ((size_t) slot * a->n_kv_heads + h) * row_blocks * 34;
            o_head(a->k + off, a->k_norm_w, a->eps, hd, a->n_rot, cs, tmp);
            if (a->k_f32) memcpy(a->k_f32 + off, tmp, (size_t) hd * sizeof(float));
            fnbo_quantize_row_q8_0(tmp, (uint8_t *) a->k_cache + cell, hd);
            fnbo_quantize_row_q8_0(a->v + off, (uint8_t *) a->v_cache + cell, hd);
        }
    }
}

/* ---- the reference's own activation format: fn/kernels/act/act.h:8-15, fn/quant/act_ref.cpp:8-30.
 * d = amax/127, id = 127/amax (0 when amax is 0), q = nearest-even(x id) clamped to +-127, NaN -> 0,
 * s = d * (float) sum q. ---- */
void fnbo_act_quantize(const float * x, int64_t rows, int32_t k, int8_t * codes, float * scales) {
    const int64_t nb = rows * (k / 32);
    for (int64_t b = 0; b < nb; ++b) {
        const float * v = x + 32 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
        const float d = amax / 127.0f;
        const float id = amax > 0.0f ? 127.0f / amax : 0.0f;
        int32_t sum = 0;
        for (int j = 0; j < 32; ++j) {
            const float e = v[j] * id;
            int32_t q = 0;
            if (e == e) {
                float r = nearbyintf(e);
                r = r < -127.0f ? -127.0f : r > 127.0f ? 127.0f : r;
                q = (int32_t) r;
            }
            codes[32 * b + j] = (int8_t) q;
            sum += q;
        }
        scales[2 * b] = d;
        scales[2 * b + 1] = d * (float) sum;
    }
}

/* fn/kernels/experts/experts.cu:716-729 with experts_dev.cuh:196-213: the GLU, then the act format */
void fnbo_swiglu_act(const float * gate, const float * up, int8_t * codes, float * scales, float * f32_out,
                     int64_t rows, int32_t cols) {
    float tmp[32];
    const int64_t nb = rows * (cols / 32);
    for (int64_t b = 0; b < nb; ++b) {
        for (int j = 0; j < 32; ++j) tmp[j] = o_swiglu(gate[32 * b + j], up[32 * b + j]);
        if (f32_out) memcpy(f32_out + 32 * b, tmp, sizeof tmp);
        fnbo_act_quantize(tmp, 1, 32, codes + 32 * b, scales + 2 * b);
    }
}

/* ---- KV8: fn/kernels/qsa/kv_q8.cuh:29-52, fn/quant/kv_q8_ref.cpp:72-87.  Per 64 values:
 * scale = fp16_rn(amax/127), s its F32 value, code = clamp(nearest-even(x / s), +-127), 0 when s is 0. ---- */
void fnbo_kv8_quantize(const float * x, int64_t n, int8_t * codes, uint16_t * scales) {
    for (int64_t g = 0; g < n / 64; ++g) {
        const float * v = x + 64 * g;
        float amax = 0.0f;
        for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fabsf(v[j]));
        uint32_t hb = fnbo_bits_f32(amax / 127.0f);
        uint16_t h;
        if ((hb & 0x7fffffffu) > 0x7f800000u) {
            h = (uint16_t) (((hb >> 16) & 0x8000u) | 0x7e00u);
        } else {
            h = fnbo_f32_to_f16(amax / 127.0f);
        }
        scales[g] = h;
        const float s = fnbo_f16_to_f32(h);
        for (int j = 0; j < 64; ++j) {
            int32_t q = 0;
            if (s > 0.0f) {
                const float r = nearbyintf(v[j] / s);
                q = r < -127.0f ? -127 : r > 127.0f ? 127 : (int32_t) r;
            }
            codes[64 * g + j] = (int8_t) q;
        }
    }
}

/* ---- the routed experts' down mat-vec (fn/kernels/experts/cpu_kq_avx2.cpp) -------------------------------------------
 * The AVX2 kernels keep one vector of eight F32 lanes per (row, t); lane j of a block's integer products is the sum of
 * bytes 4 j .. 4 j + 3 (maddubs + madd, :133-139), converted exactly and fused-multiply-added with the block's scale
 * product (:314, :338).  The scalar side term of Q5_1 (m x s, :310) is `summs += xm * s`, which the reference's flags
 * (-mfma with GCC's default contraction) compile to one fused multiply-add; fmaf states that.  hsum_float_8 (:103-109)
 * adds lane i + 4 to lane i, then lanes 2, 3 to 0, 1, then lane 1 to lane 0. */
static float fnbo_hsum8(const float * a) {
    const float r0 = a[4] + a[0], r1 = a[5] + a[1], r2 = a[6] + a[2], r3 = a[7] + a[3];
    const float s0 = r0 + r2, s1 = r1 + r3;
    return s0 + s1;
}

void fnbo_expert_down_rows(int32_t fmt, const uint8_t * w, int64_t row_bytes, int32_t n, const uint8_t * act,
                           int64_t act_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1) {
    const int nb = n / 32;
    for (int64_t r = r0; r < r1; ++r) {
        const uint8_t * row = w + r * row_bytes;
        for (int t = 0; t < nt; ++t) {
            const uint8_t * a = act + (int64_t) t * act_stride;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float summs = 0.0f;
            for (int ib = 0; ib < nb; ++ib) {
                int qx[32];
                float xd, scale;
                const int8_t * qy;
                if (fmt == 0) { /* Q5_1 {d, m fp16; qh[4]; qs[16]} x Q8_1 {d, s fp16; qs[32]} */
                    const uint8_t * b = row + ib * 24;
                    uint16_t dh, mh, yd, ys;
                    uint32_t qh;
                    memcpy(&dh, b, 2), memcpy(&mh, b + 2, 2), memcpy(&qh, b + 4, 4);
                    for (int i = 0; i < 16; ++i) {
                        qx[i] = (b[8 + i] & 15) | (int) (((qh >> i) & 1u) << 4);
                        qx[i + 16] = (b[8 + i] >> 4) | (int) (((qh >> (i + 16)) & 1u) << 4);
                    }
                    const uint8_t * y = a + ib * 36;
                    memcpy(&yd, y, 2), memcpy(&ys, y + 2, 2);
                    qy = (const int8_t *) (y + 4);
                    xd = fnbo_f16_to_f32(dh);
                    summs = fmaf(fnbo_f16_to_f32(mh), fnbo_f16_to_f32(ys), summs);
                    scale = xd * fnbo_f16_to_f32(yd);
                } else if (fmt == 2) { /* IQ4_NL {d fp16; 16 nibble bytes -> kvalues_iq4nl} x Q8_0: cpu_iq_avx2.cpp:481-514 */
                    static const int8_t kvalues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
                    const uint8_t * b = row + ib * 18;
                    uint16_t dh, yd;
                    memcpy(&dh, b, 2);
                    const uint8_t * y = a + ib * 34;
                    memcpy(&yd, y, 2);
                    qy = (const int8_t *) (y + 2);
                    /* the kernel multiplies |w| by the code with w's sign applied (_mm256_sign_epi8: two's complement,
                     * -128 stays -128); stated here as w' x code with w' = w unless the code is -128 and w < 0 */
                    for (int i = 0; i < 16; ++i) {
                        qx[i] = kvalues[b[2 + i] & 15];
                        qx[i + 16] = kvalues[b[2 + i] >> 4];
                    }
                    for (int i = 0; i < 32; ++i) {
                        if (qy[i] == -128 && qx[i] < 0) qx[i] = -qx[i];
                    }
                    scale = fnbo_f16_to_f32(dh) * fnbo_f16_to_f32(yd);
                } else { /* Q8_0 {d fp16; qs[32]} x Q8_0 */
                    const uint8_t * b = row + ib * 34;
                    uint16_t dh, yd;
                    memcpy(&dh, b, 2);
                    for (int i = 0; i < 32; ++i) qx[i] = (int8_t) b[2 + i];
                    const uint8_t * y = a + ib * 34;
                    memcpy(&yd, y, 2);
                    qy = (const int8_t *) (y + 2);
                    scale = fnbo_f16_to_f32(dh) * fnbo_f16_to_f32(yd);
                }
                for (int j = 0; j < 8; ++j) {
                    int s = 0;
                    for (int i = 0; i < 4; ++i) s += qx[4 * j + i] * (int) qy[4 * j + i];
                    acc[j] = fmaf((float) s, scale, acc[j]);
                }
            }
            if (fmt == 2) { /* the IQ file's hsum8 (:187-193): lane i + 4 onto lane i, then two horizontal adds */
                const float s0 = acc[0] + acc[4], s1 = acc[1] + acc[5], s2 = acc[2] + acc[6], s3 = acc[3] + acc[7];
                out[(int64_t) t * out_stride + r] = (s0 + s1) + (s2 + s3);
                continue;
            }
            out[(int64_t) t * out_stride + r] = fnbo_hsum8(acc) + summs;
        }
    }
}

/* ---- Q8_K (ggml/src/ggml-quants.c:2844-2881; nearest_int :559-565) ---------------------------------------------------*/
void fnbo_quantize_row_q8_k(const float * x, void * vy, int64_t k) {
    uint8_t * y = (uint8_t *) vy;
    for (int64_t i = 0; i < k / 256; ++i, x += 256, y += 292) {
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < 256; ++j) {
            const float ax = fabsf(x[j]);
            if (ax > amax) amax = ax, max = x[j];
        }
        int8_t * qs = (int8_t *) (y + 4);
        int16_t bsums[16];
        if (!amax) {
            const float zero = 0.0f;
            memcpy(y, &zero, 4);
            memset(qs, 0, 256);
            /* the reference leaves bsums untouched here; the caller's buffer decides them.  Written as zeros so that the
             * block is a function of its input. */
            memset(y + 260, 0, 32);
            continue;
        }
        const float iscale = -127.0f / max;
        for (int j = 0; j < 256; ++j) {
            const float val = iscale * x[j] + 12582912.0f; /* nearest_int: the product rounds, then the sum */
            int32_t b;
            memcpy(&b, &val, 4);
            const int v = (b & 0x007fffff) - 0x00400000;
            qs[j] = (int8_t) (v < 127 ? v : 127);
        }
        for (int j = 0; j < 16; ++j) {
            int sum = 0;
            for (int ii = 0; ii < 16; ++ii) sum += qs[16 * j + ii];
            bsums[j] = (int16_t) sum;
        }
        memcpy(y + 260, bsums, 32);
        const float d = 1.0f / iscale;
        memcpy(y, &d, 4);
    }
}

/* ---- the reference's planar 32-value activation and its Q2_0 down rows (fn/kernels/experts/cpu_q2_avx2.cpp:180-226
 * quantize_act_q, :62-96 row_bp, :98-102 reduce1).  Quantiser: s = amax / 127, inv = 1 / s (both 0 for an all-zero
 * chunk), code = trunc(x inv +- 0.5) (half away from zero) clamped to +-127.  Q2_0: 64-weight blocks of 18 bytes (fp16
 * d, 16 code bytes: value 4 i + k at bits 2 k of byte i, weight d (c - 1)), taken in pairs.  Per pair eight lanes: lane
 * 4 h + m is block h's values 16 m .. 16 m + 15: sum(c q) - sum(q) exactly in integers, converted, TIMES the chunk
 * scale (one multiply), then one fused multiply-add by d into the lane; an output is
 * ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7)). ---- */
void fnbo_quantize_act_q(const float * x, int64_t n, int8_t * q, float * scale) {
    for (int64_t k = 0; k < n / 32; ++k) {
        const float * xb = x + 32 * k;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) {
            const float a = fabsf(xb[j]);
            if (a > amax) amax = a;
        }
        const float s = amax > 0.f ? amax / 127.f : 0.f;
        const float inv = s > 0.f ? 1.f / s : 0.f;
        for (int j = 0; j < 32; ++j) {
            const float t = xb[j] * inv;
            const float r = t + (t >= 0.f ? 0.5f : -0.5f);
            int32_t v = (r > -2147483648.0f && r < 2147483648.0f) ? (int32_t) r : INT32_MIN; /* cvttps */
            v = v < -127 ? -127 : v > 127 ? 127 : v;
            q[32 * k + j] = (int8_t) v;
        }
        scale[k] = s;
    }
}

void fnbo_expert_down_rows_q2_0(const uint8_t * w, int64_t row_bytes, int32_t n, const int8_t * q, int64_t q_stride,
                                const float * scale, int64_t scale_stride, int32_t nt, float * out, int64_t out_stride,
                                int64_t r0, int64_t r1) {
    const int npairs = n / 128;
    for (int64_t r = r0; r < r1; ++r) {
        const uint8_t * row = w + r * row_bytes;
        for (int t = 0; t < nt; ++t) {
            const int8_t * qt = q + (int64_t) t * q_stride;
            const float * st = scale + (int64_t) t * scale_stride;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int p = 0; p < npairs; ++p) {
                for (int h = 0; h < 2; ++h) {
                    const uint8_t * blk = row + 36 * p + 18 * h;
                    uint16_t dh;
                    memcpy(&dh, blk, 2);
                    const float d = fnbo_f16_to_f32(dh);
                    for (int m = 0; m < 4; ++m) {
                        int32_t dot = 0, sum = 0;
                        for (int v = 0; v < 16; ++v) {
                            const int idx = 16 * m + v; /* value idx of the block: byte idx / 4, bits 2 (idx % 4) */
                            const int c = (blk[2 + idx / 4] >> (2 * (idx % 4))) & 3;
                            const int qv = qt[128 * p + 64 * h + idx];
                            dot += c * qv, sum += qv;
                        }
                        const float val = (float) (dot - sum) * st[4 * p + 2 * h + m / 2];
                        acc[4 * h + m] = fmaf(d, val, acc[4 * h + m]);
                    }
                }
            }
            out[(int64_t) t * out_stride + r] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
        }
    }
}

/* ---- the routed experts' gate / up rows over Q8_K (fn/kernels/experts/cpu_kq_avx2.cpp:166-224, :362-380) ------------*/
static float fnbo_q4k_dot(const uint8_t * row, int nb, const uint8_t * act) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float acc_m[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + 144 * i;
        const uint8_t * y = act + 292 * i;
        uint16_t dh, mh;
        memcpy(&dh, x, 2), memcpy(&mh, x + 2, 2);
        const float xd = fnbo_f16_to_f32(dh), xdmin = fnbo_f16_to_f32(mh);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) o_scale_min_k4(j, x + 4, &sc[j], &mn[j]);
        float yd;
        memcpy(&yd, y, 4);
        const int8_t * q8 = (const int8_t *) (y + 4);
        int16_t bsums[16];
        memcpy(bsums, y + 260, 32);
        const float d = yd * xd, dmin = -yd * xdmin;
        for (int k = 0; k < 4; ++k) { /* madd_epi16 of the mins with the pairwise (16-bit) sums of the block sums */
            const int16_t s0 = (int16_t) (bsums[4 * k] + bsums[4 * k + 1]), s1 = (int16_t) (bsums[4 * k + 2] + bsums[4 * k + 3]);
            const int32_t prod = (int32_t) mn[2 * k] * s0 + (int32_t) mn[2 * k + 1] * s1;
            acc_m[k] = fmaf(dmin, (float) prod, acc_m[k]);
        }
        const uint8_t * q4 = x + 16;
        for (int l = 0; l < 8; ++l) {
            int32_t sumi = 0;
            for (int j = 0; j < 4; ++j) {
                int32_t lo = 0, hi = 0;
                for (int b = 4 * l; b < 4 * l + 4; ++b) {
                    lo += (q4[32 * j + b] & 15) * (int32_t) q8[64 * j + b];
                    hi += (q4[32 * j + b] >> 4) * (int32_t) q8[64 * j + 32 + b];
                }
                sumi += (int32_t) sc[2 * j] * lo + (int32_t) sc[2 * j + 1] * hi;
            }
            acc[l] = fmaf(d, (float) sumi, acc[l]);
        }
    }
    return fnbo_hsum8(acc) + ((acc_m[0] + acc_m[2]) + (acc_m[1] + acc_m[3]));
}

void fnbo_expert_gu_rows_q4_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                              int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                              int64_t r1) {
    const int nb = n / 256;
    for (int64_t r = r0; r < r1; ++r) {
        for (int t = 0; t < nt; ++t) {
            const float g = fnbo_q4k_dot(gate + r * row_bytes, nb, act + (int64_t) t * act_stride);
            const float u = fnbo_q4k_dot(up + r * row_bytes, nb, act + (int64_t) t * act_stride);
            ff[(int64_t) t * ff_stride + r] = (g / (1.0f + o_expf(-g))) * u;
            if (gu != NULL) {
                gu[(int64_t) t * ff_stride + r] = g;
                gu[((int64_t) nt + t) * ff_stride + r] = u;
            }
        }
    }
}

/* ---- the same rows with Q5_K weights (fn/kernels/experts/cpu_kq_avx2.cpp:226-290 q5k_dot, ggml's
 * ggml_vec_dot_q5_K_q8_K with the weight side hoisted).  Block: fp16 d, dmin, 12 scale bytes, qh[32], qs[128]; value
 * 64 j + b is (qs[32 j + b] & 15) + 16 bit 2 j of qh[b], value 64 j + 32 + b is (qs[32 j + b] >> 4) + 16 bit 2 j + 1.
 * Eight int32 lanes as for Q4_K; the mins are ONE scalar: summs += dmin x (sum over eight of min x 16-bit pair sum of
 * the block sums), which the reference's flags compile to a fused multiply-add; result hsum_float_8(acc) + summs. */
static float fnbo_q5k_dot(const uint8_t * row, int nb, const uint8_t * act) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float summs = 0.f;
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + 176 * i;
        const uint8_t * y = act + 292 * i;
        uint16_t dh, mh;
        memcpy(&dh, x, 2), memcpy(&mh, x + 2, 2);
        const float xd = fnbo_f16_to_f32(dh), xdmin = fnbo_f16_to_f32(mh);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) o_scale_min_k4(j, x + 4, &sc[j], &mn[j]);
        const uint8_t * qh = x + 16;
        const uint8_t * qs = x + 48;
        float yd;
        memcpy(&yd, y, 4);
        const int8_t * q8 = (const int8_t *) (y + 4);
        int16_t bsums[16];
        memcpy(bsums, y + 260, 32);
        const float d = yd * xd, dmin = -yd * xdmin;
        int32_t msum = 0;
        for (int k = 0; k < 8; ++k) msum += (int32_t) mn[k] * (int16_t) (bsums[2 * k] + bsums[2 * k + 1]);
        summs = fmaf(dmin, (float) msum, summs);
        for (int l = 0; l < 8; ++l) {
            int32_t sumi = 0;
            for (int j = 0; j < 4; ++j) {
                int32_t lo = 0, hi = 0;
                for (int b = 4 * l; b < 4 * l + 4; ++b) {
                    const int v0 = (qs[32 * j + b] & 15) + (((qh[b] >> (2 * j)) & 1) << 4);
                    const int v1 = (qs[32 * j + b] >> 4) + (((qh[b] >> (2 * j + 1)) & 1) << 4);
                    lo += v0 * (int32_t) q8[64 * j + b];
                    hi += v1 * (int32_t) q8[64 * j + 32 + b];
                }
                sumi += (int32_t) sc[2 * j] * lo + (int32_t) sc[2 * j + 1] * hi;
            }
            acc[l] = fmaf(d, (float) sumi, acc[l]);
        }
    }
    return fnbo_hsum8(acc) + summs;
}

void fnbo_expert_gu_rows_q5_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                              int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                              int64_t r1) {
    const int nb = n / 256;
    for (int64_t r = r0; r < r1; ++r) {
        for (int t = 0; t < nt; ++t) {
            const float g = fnbo_q5k_dot(gate + r * row_bytes, nb, act + (int64_t) t * act_stride);
            const float u = fnbo_q5k_dot(up + r * row_bytes, nb, act + (int64_t) t * act_stride);
            ff[(int64_t) t * ff_stride + r] = (g / (1.0f + o_expf(-g))) * u;
            if (gu != NULL) {
                gu[(int64_t) t * ff_stride + r] = g;
                gu[((int64_t) nt + t) * ff_stride + r] = u;
            }
        }
    }
}

/* ---- the same rows with IQ3_XXS weights (fn/kernels/experts/cpu_iq_avx2.cpp:256-271 fmt32<18>::decode, :305-337
 * row_dot, :429-445 gu_rows).  Per super-block eight int32 lanes: lane l collects, over the block's eight groups of 32
 * values, (2 s + 1) x the sum of four codebook bytes of the group's index byte l times the sign-applied Q8_K codes
 * 32 g + 4 l ..; _mm256_sign_epi8 negates a code in two's complement, so -128 stays -128.  maddubs_epi16's 16-bit
 * pair sums cannot saturate (2 x 62 x 128).  One fused multiply-add per super-block and lane with (x.d y.d), x.d
 * WITHOUT the format's 1/4; ggml's hsum_float_8 order; the 1/4 multiplies the reduced sum. */
static float fnbo_iq3xxs_dot(const uint8_t * row, int nb, const uint8_t * act) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + 98 * i;
        const uint8_t * y = act + 292 * i;
        uint16_t dh;
        memcpy(&dh, x, 2);
        float yd;
        memcpy(&yd, y, 4);
        const int8_t * q8 = (const int8_t *) (y + 4);
        int32_t acci[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int g = 0; g < 8; ++g) {
            uint32_t w;
            memcpy(&w, x + 66 + 4 * g, 4);
            const int32_t sc = 2 * (int32_t) (w >> 28) + 1;
            for (int l = 0; l < 8; ++l) {
                const unsigned code = o_grid_packed[x[2 + 8 * g + l]];
                const unsigned s7 = (w >> (7 * (l / 2))) & 127u;
                const unsigned signs = s7 | ((unsigned) (__builtin_popcount(s7) & 1) << 7);
                int32_t sum = 0;
                for (int b = 0; b < 4; ++b) {
                    const unsigned level = (code >> (3 * b)) & 7u;
                    const int32_t mag = level == 7 ? 62 : 4 + 8 * (int32_t) level;
                    const int8_t yv = q8[32 * g + 4 * l + b];
                    const int8_t ys = (signs >> (4 * (l & 1) + b)) & 1u ? (int8_t) (0u - (unsigned) yv) : yv;
                    sum += mag * (int32_t) ys;
                }
                acci[l] += sc * sum;
            }
        }
        const float dxy = fnbo_f16_to_f32(dh) * yd;
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(dxy, (float) acci[l], acc[l]);
    }
    return 0.25f * fnbo_hsum8(acc);
}

void fnbo_expert_gu_rows_iq3_xxs(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                                 int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                 int64_t r1) {
    const int nb = n / 256;
    for (int64_t r = r0; r < r1; ++r) {
        for (int t = 0; t < nt; ++t) {
            const float g = fnbo_iq3xxs_dot(gate + r * row_bytes, nb, act + (int64_t) t * act_stride);
            const float u = fnbo_iq3xxs_dot(up + r * row_bytes, nb, act + (int64_t) t * act_stride);
            ff[(int64_t) t * ff_stride + r] = (g / (1.0f + o_expf(-g))) * u;
            if (gu != NULL) {
                gu[(int64_t) t * ff_stride + r] = g;
                gu[((int64_t) nt + t) * ff_stride + r] = u;
            }
        }
    }
}

/* ---- and with IQ3_S weights (cpu_iq_avx2.cpp:273-290 fmt32<21>::decode through the same row_dot): 9-bit codebook
 * indices (qs byte | qh bit), sign bit i of a group's four sign bytes for value i, one 4-bit scale per 32 values
 * (2 s + 1), K = 1: x.d y.d per super-block, ggml's hsum_float_8 order. */
static float fnbo_iq3s_dot(const uint8_t * row, int nb, const uint8_t * act) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + 110 * i;
        const uint8_t * y = act + 292 * i;
        uint16_t dh;
        memcpy(&dh, x, 2);
        float yd;
        memcpy(&yd, y, 4);
        const int8_t * q8 = (const int8_t *) (y + 4);
        int32_t acci[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int g = 0; g < 8; ++g) {
            uint32_t signs;
            memcpy(&signs, x + 74 + 4 * g, 4);
            const unsigned s = x[106 + g / 2];
            const int32_t sc = 2 * (int32_t) ((g & 1) ? s >> 4 : s & 15u) + 1;
            for (int l = 0; l < 8; ++l) {
                const unsigned code = o_grid3s_packed[x[2 + 8 * g + l] | (((x[66 + g] >> l) & 1u) << 8)];
                int32_t sum = 0;
                for (int b = 0; b < 4; ++b) {
                    const int32_t mag = 2 * (int32_t) ((code >> (3 * b)) & 7u) + 1;
                    const int8_t yv = q8[32 * g + 4 * l + b];
                    const int8_t ys = (signs >> (4 * l + b)) & 1u ? (int8_t) (0u - (unsigned) yv) : yv;
                    sum += mag * (int32_t) ys;
                }
                acci[l] += sc * sum;
            }
        }
        const float dxy = fnbo_f16_to_f32(dh) * yd;
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(dxy, (float) acci[l], acc[l]);
    }
    return 1.0f * fnbo_hsum8(acc);
}

void fnbo_expert_gu_rows_iq3_s(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                               int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                               int64_t r1) {
    const int nb = n / 256;
    for (int64_t r = r0; r < r1; ++r) {
        for (int t = 0; t < nt; ++t) {
            const float g = fnbo_iq3s_dot(gate + r * row_bytes, nb, act + (int64_t) t * act_stride);
            const float u = fnbo_iq3s_dot(up + r * row_bytes, nb, act + (int64_t) t * act_stride);
            ff[(int64_t) t * ff_stride + r] = (g / (1.0f + o_expf(-g))) * u;
            if (gu != NULL) {
                gu[(int64_t) t * ff_stride + r] = g;
                gu[((int64_t) nt + t) * ff_stride + r] = u;
            }
        }
    }
}

/* ---- and with the three IQ2 formats (fn/kernels/experts/cpu_iq_avx2.cpp:225-254 fmt32<16> and fmt32<22>, :341-414
 * row_dot_iq2xs, :305-337 row_dot).  The lane structure is the IQ3 kernels': per super-block eight int32 lanes, lane l of
 * a 32-value half collecting scale x (four codebook magnitudes times four sign-applied Q8_K codes); a codebook entry
 * holds EIGHT magnitudes (8, 25 or 43), so it serves two lanes.
 *   IQ2_XXS (66 bytes): per half four index bytes, then a word of 4 x 7-bit sign index + 4-bit scale s: 2 s + 1.
 *   IQ2_XS  (74 bytes): 32 x u16 = 9-bit index | 7-bit sign index << 9; scales[8], low nibble for a half's first 16
 *                       values, high nibble for its last 16; its two accumulators a block add as integers.
 *   IQ2_S   (82 bytes): qs[32] index low bytes, 32 plain sign bytes, qh[8] (two more index bits a value group),
 *                       scales[8] as IQ2_XS.
 * K = 1/8: IQ2_XXS and IQ2_XS fold it into the block's d (d * 0.125f, exact) and reduce pairwise (hsum8: lo + hi halves,
 * then two horizontal adds); IQ2_S applies it to the reduced sum in ggml's hsum_float_8 order. */
static const uint16_t o_grid2xxs_packed[256] = {
#include "../fnfl_v100_b200/csrc/iq2xxs_grid_packed.inc"
};
static const uint16_t o_grid2xs_packed[512] = {
#include "../fnfl_v100_b200/csrc/iq2xs_grid_packed.inc"
};
static const uint16_t o_grid2s_packed[1024] = {
#include "../fnfl_v100_b200/csrc/iq2s_grid_packed.inc"
};

static float fnbo_hsum8_pairwise(const float * a) {
    const float s0 = a[0] + a[4], s1 = a[1] + a[5], s2 = a[2] + a[6], s3 = a[3] + a[7];  /* lo + hi */
    const float h0 = s0 + s1, h1 = s2 + s3;                                               /* hadd */
    return h0 + h1;                                                                       /* hadd */
}

/* fmt: 16 IQ2_XXS, 17 IQ2_XS, 22 IQ2_S (ggml's type numbers, as the reference's templates) */
static float fnbo_iq2_dot(int fmt, const uint8_t * row, int nb, const uint8_t * act) {
    const int bytes = fmt == 16 ? 66 : fmt == 17 ? 74 : 82;
    static const int32_t mags[4] = {8, 25, 43, 0};
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < nb; ++i) {
        const uint8_t * x = row + (size_t) bytes * i;
        const uint8_t * y = act + 292 * i;
        uint16_t dh;
        memcpy(&dh, x, 2);
        float yd;
        memcpy(&yd, y, 4);
        const int8_t * q8 = (const int8_t *) (y + 4);
        int32_t acci[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int h = 0; h < 8; ++h) {            /* the eight 32-value halves */
            for (int k = 0; k < 4; ++k) {        /* a codebook entry: values 8 k .. 8 k + 7 of the half, lanes 2 k, 2 k + 1 */
                unsigned code, signs;
                int32_t sc;
                if (fmt == 16) {
                    uint32_t w;
                    memcpy(&w, x + 2 + 8 * h + 4, 4);
                    code = o_grid2xxs_packed[x[2 + 8 * h + k]];
                    const unsigned s7 = (w >> (7 * k)) & 127u;
                    signs = s7 | ((unsigned) (__builtin_popcount(s7) & 1) << 7);
                    sc = 2 * (int32_t) (w >> 28) + 1;
                } else if (fmt == 17) {
                    uint16_t q;
                    memcpy(&q, x + 2 + 2 * (4 * h + k), 2);
                    code = o_grid2xs_packed[q & 511u];
                    const unsigned s7 = q >> 9;
                    signs = s7 | ((unsigned) (__builtin_popcount(s7) & 1) << 7);
                    const unsigned sn = x[66 + h];
                    sc = 2 * (int32_t) (k < 2 ? sn & 15u : sn >> 4) + 1;
                } else {
                    code = o_grid2s_packed[x[2 + 4 * h + k] | (((x[66 + h] >> (2 * k)) & 3u) << 8)];
                    signs = x[34 + 4 * h + k];
                    const unsigned sn = x[74 + h];
                    sc = 2 * (int32_t) (k < 2 ? sn & 15u : sn >> 4) + 1;
                }
                for (int half = 0; half < 2; ++half) {   /* lanes 2 k and 2 k + 1: four values each */
                    int32_t sum = 0;
                    for (int b = 0; b < 4; ++b) {
                        const int v = 4 * half + b;
                        const int32_t mag = mags[(code >> (2 * v)) & 3u];
                        const int8_t yv = q8[32 * h + 8 * k + v];
                        const int8_t ys = (signs >> v) & 1u ? (int8_t) (0u - (unsigned) yv) : yv;
                        sum += mag * (int32_t) ys;
                    }
                    acci[2 * k + half] += sc * sum;
                }
            }
        }
        const float dx = fmt == 22 ? fnbo_f16_to_f32(dh) : fnbo_f16_to_f32(dh) * 0.125f;
        const float dxy = dx * yd;
        for (int l = 0; l < 8; ++l) acc[l] = fmaf(dxy, (float) acci[l], acc[l]);
    }
    return fmt == 22 ? 0.125f * fnbo_hsum8(acc) : fnbo_hsum8_pairwise(acc);
}

void fnbo_expert_gu_rows_iq2(int32_t fmt, const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n,
                             const uint8_t * act, int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu,
                             int64_t r0, int64_t r1) {
    const int nb = n / 256;
    for (int64_t r = r0; r < r1; ++r) {
        for (int t = 0; t < nt; ++t) {
            const float g = fnbo_iq2_dot(fmt, gate + r * row_bytes, nb, act + (int64_t) t * act_stride);
            const float u = fnbo_iq2_dot(fmt, up + r * row_bytes, nb, act + (int64_t) t * act_stride);
            ff[(int64_t) t * ff_stride + r] = (g / (1.0f + o_expf(-g))) * u;
            if (gu != NULL) {
                gu[(int64_t) t * ff_stride + r] = g;
                gu[((int64_t) nt + t) * ff_stride + r] = u;
            }
        }
    }
}

/* fn/kernels/qsa/attend.h:17-19 (o = softmax(q . K / 16) . V, out = o sigmoid(gate)), every sum in double, the
 * maximum subtracted before the exponentials: the FP64 statement the reference's qa2-test checks its kernel against
 * (fn/kernels/qsa/qa2_test.cpp:469-520) */
void fnbo_attend_f64(const float * q, const float * gate, const float * k, const float * v, const int32_t * first,
                     const int32_t * count, int32_t rows, int32_t n_q, int32_t n_kv, int32_t hd, double scale, double * out) {
    const int rep = n_q / n_kv;
    for (int t = 0; t < rows; ++t) {
        const int64_t c0 = first[t], n = count[t];
        double * s = (double *) malloc(sizeof(double) * (size_t) (n > 0 ? n : 1));
        for (int h = 0; h < n_q; ++h) {
            const int g = h / rep;
            const float * qr = q + ((size_t) t * n_q + h) * hd;
            double * o = out + ((size_t) t * n_q + h) * hd;
            for (int d = 0; d < hd; ++d) o[d] = 0.0;
            if (n <= 0) continue;
            double mx = -INFINITY;
            for (int64_t c = 0; c < n; ++c) {
                const float * kr = k + ((size_t) (c0 + c) * n_kv + g) * hd;
                double acc = 0.0;
                for (int d = 0; d < hd; ++d) acc += (double) qr[d] * (double) kr[d];
                s[c] = acc * scale;
                if (s[c] > mx) mx = s[c];
            }
            double l = 0.0;
            for (int64_t c = 0; c < n; ++c) {
                s[c] = exp(s[c] - mx);
                l += s[c];
            }
            for (int64_t c = 0; c < n; ++c) {
                const float * vr = v + ((size_t) (c0 + c) * n_kv + g) * hd;
                const double p = s[c] / l;
                for (int d = 0; d < hd; ++d) o[d] += p * (double) vr[d];
            }
            if (gate) {
                const float * gr = gate + ((size_t) t * n_q + h) * hd;
                for (int d = 0; d < hd; ++d) o[d] *= 1.0 / (1.0 + exp(-(double) gr[d]));
            }
        }
        free(s);
    }
}
