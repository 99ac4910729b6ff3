// TEST INFRASTRUCTURE.  C entry points over the reference's own CPU sources, compiled where they lie in the
// reference tree (see Makefile: nothing is copied).  The ggml (de)quantisers are exported by ggml-quants.c
// itself under their own names (quantize_row_q8_0_ref, quantize_row_q8_1_ref, dequantize_row_q4_K,
// dequantize_row_iq3_xxs, dequantize_row_q8_0); this file adds the four symbols ggml-quants.c leaves undefined
// when built alone, and C wrappers for the C++ references under fn/quant.
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "fn/quant/act_ref.h"
#include "fn/quant/decode.h"
#include "fn/quant/formats.h"
#include "fn/quant/kv_q8_ref.h"
#include "fn/kernels/experts/cpu_kernels.h"
#include "fn/quant/synth.h"

extern "C" {

// ggml-quants.c's unresolved externals: only reached from quantisation paths the oracle never calls
void ggml_abort(const char * file, int line, const char * fmt, ...) {
    std::fprintf(stderr, "ggml_abort %s:%d: ", file, line);
    va_list ap;
    va_start(ap, fmt);
    std::vfprintf(stderr, fmt, ap);
    va_end(ap);
    std::fputc('\n', stderr);
    std::abort();
}
size_t ggml_row_size(int, int64_t) { std::abort(); }
const char * ggml_type_name(int) { return "?"; }
size_t ggml_type_size(int) { std::abort(); }

void ref_act_quantize(const float * x, int32_t rows, int32_t k, int8_t * codes, float * scales) {
    fn::quant::act_quantize_ref(x, rows, k, codes, scales);
}

void ref_kv_q8_quantize(const float * x, int32_t n, int8_t * codes, uint16_t * scales) {
    fn::quant::kv_q8_quantize(x, n, codes, scales);
}

// the value a KV8 code stands for under its group's scale bits (fn/quant/kv_q8_ref.cpp:95-97), n values, group of 64
void ref_kv_q8_values(const int8_t * codes, const uint16_t * scales, int64_t n, float * out) {
    for (int64_t i = 0; i < n; ++i) out[i] = fn::quant::kv_q8_value(codes[i], scales[i / fn::quant::kv_q8_group]);
}

// the KV8 stress rows (fn/quant/kv_q8_ref.cpp:99-169): returns the value count; copies up to cap values
int64_t ref_kv_q8_stress_rows(uint64_t seed, int32_t random_rows, float * out, int64_t cap) {
    const std::vector<float> v = fn::quant::kv_q8_stress_rows(seed, random_rows);
    const int64_t n = int64_t(v.size());
    if (out != nullptr) {
        std::memcpy(out, v.data(), size_t(n < cap ? n : cap) * sizeof(float));
    }
    return n;
}

static bool fmt_of(const char * name, fn::quant::wfmt & f) { return fn::quant::wfmt_of_name(name, f); }

int32_t ref_block_bytes(const char * fmt) {
    fn::quant::wfmt f;
    return fmt_of(fmt, f) ? fn::quant::info(f).block_bytes : -1;
}

int32_t ref_decode_row(const char * fmt, const void * src, float * dst, int64_t n) {
    fn::quant::wfmt f;
    return fmt_of(fmt, f) && fn::quant::decode_row(f, src, dst, n) ? 0 : 1;
}

int32_t ref_synth_blocks(const char * fmt, uint64_t seed, int64_t n_blocks, uint8_t * dst) {
    fn::quant::wfmt f;
    return fmt_of(fmt, f) && fn::quant::synth_blocks(f, seed, n_blocks, dst) ? 0 : 1;
}

uint16_t ref_f32_to_f16(float f) { return fn::quant::f32_to_f16(f); }
float ref_f16_to_f32(uint16_t h) { return fn::quant::f16_to_f32(h); }

// the routed experts' gate / up rows with the GLU (fn/kernels/experts/cpu_kq_avx2.cpp:362-380), fmt q4_k
void ref_kq_gu_rows_q4_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                         int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, int32_t r0, int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = ff + int64_t(t) * ff_stride;
    fn::experts::cpu::kq_gu_rows(fn::experts::fmt::q4_k, gate, up, size_t(row_bytes), n, a, nt, o, r0, r1);
}

// the same rows for Q5_K weights (fn/kernels/experts/cpu_kq_avx2.cpp:226-290 through kq_gu_rows)
void ref_kq_gu_rows_q5_k(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                         int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, int32_t r0, int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = ff + int64_t(t) * ff_stride;
    fn::experts::cpu::kq_gu_rows(fn::experts::fmt::q5_k, gate, up, size_t(row_bytes), n, a, nt, o, r0, r1);
}

// the same rows for IQ3_XXS weights (fn/kernels/experts/cpu_iq_avx2.cpp:429-445 through iq_gu_rows)
void ref_iq_gu_rows_iq3_xxs(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                            int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, int32_t r0, int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = ff + int64_t(t) * ff_stride;
    fn::experts::cpu::iq_gu_rows(fn::experts::fmt::iq3_xxs, gate, up, size_t(row_bytes), n, a, nt, o, r0, r1);
}

// and for IQ3_S weights
void ref_iq_gu_rows_iq3_s(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n, const uint8_t * act,
                          int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, int32_t r0, int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = ff + int64_t(t) * ff_stride;
    fn::experts::cpu::iq_gu_rows(fn::experts::fmt::iq3_s, gate, up, size_t(row_bytes), n, a, nt, o, r0, r1);
}

// and for the three IQ2 formats (fmt: ggml's type number 16 IQ2_XXS, 17 IQ2_XS, 22 IQ2_S)
void ref_iq_gu_rows_iq2(int32_t fmt, const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int32_t n,
                        const uint8_t * act, int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, int32_t r0,
                        int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = ff + int64_t(t) * ff_stride;
    const fn::experts::fmt f = fmt == 16 ? fn::experts::fmt::iq2_xxs : fmt == 17 ? fn::experts::fmt::iq2_xs : fn::experts::fmt::iq2_s;
    fn::experts::cpu::iq_gu_rows(f, gate, up, size_t(row_bytes), n, a, nt, o, r0, r1);
}

// the planar 32-value activation (fn/kernels/experts/cpu_q2_avx2.cpp:180-226): codes and chunk scales of n <= 640 values
void ref_quantize_act_q(const float * x, int32_t n, int8_t * q, float * scale) {
    fn::experts::cpu::act_q a;
    fn::experts::cpu::quantize_act_q(x, n, a);
    for (int i = 0; i < n; ++i) q[i] = a.q[i];
    for (int i = 0; i < n / 32; ++i) scale[i] = a.scale[i];
}

// Q2_0 down rows (:150-178) of nt <= 8 activation rows given as floats (quantised by the reference's own quantiser)
void ref_q2_down_rows(const uint8_t * w, int64_t row_bytes, int32_t n, const float * x, int32_t nt, float * out,
                      int64_t out_stride, int32_t r0, int32_t r1) {
    static fn::experts::cpu::act_q acts[8];
    const fn::experts::cpu::act_q * a[8];
    float * o[8];
    for (int t = 0; t < nt && t < 8; ++t) {
        fn::experts::cpu::quantize_act_q(x + int64_t(t) * n, n, acts[t]);
        a[t] = &acts[t], o[t] = out + int64_t(t) * out_stride;
    }
    fn::experts::cpu::q2_down_rows(w, size_t(row_bytes), n / 64, a, nt, o, r0, r1);
}

// Q8_K activations: the reference's AVX2 form (fn/kernels/experts/cpu_iq_avx2.cpp:583-646); ggml's scalar form
// quantize_row_q8_K_ref is exported by ggml-quants.c itself
void ref_quantize_q8_k_avx2(const float * x, void * y, int64_t k) { fn::experts::cpu::quantize_q8_k(x, y, k); }

// the routed experts' down rows (fn/kernels/experts/cpu_kq_avx2.cpp:382-394): fmt 0 = Q5_1 x Q8_1, 1 = Q8_0 x Q8_0
void ref_kq_down_rows(int32_t f, const uint8_t * w, int64_t row_bytes, int32_t n, const uint8_t * act, int64_t act_stride,
                      int32_t nt, float * out, int64_t out_stride, int32_t r0, int32_t r1) {
    const void * a[64];
    float * o[64];
    for (int t = 0; t < nt && t < 64; ++t) a[t] = act + int64_t(t) * act_stride, o[t] = out + int64_t(t) * out_stride;
    if (f == 2) {  // IQ4_NL x Q8_0 (fn/kernels/experts/cpu_iq_avx2.cpp:571-578)
        fn::experts::cpu::iq4nl_down_rows(w, size_t(row_bytes), n, a, nt, o, r0, r1);
        return;
    }
    fn::experts::cpu::kq_down_rows(f == 0 ? fn::experts::fmt::q5_1 : fn::experts::fmt::q8_0, w, size_t(row_bytes), n, a, nt,
                                   o, r0, r1);
}

}  // extern "C"
