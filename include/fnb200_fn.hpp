// Header-only C++ shims over the C ABI (fnb200.h) in the reference engine's launcher convention:
//
//     namespace <family> { struct <op>_args { raw device pointers, PODs }; bool <op>(const <op>_args &, void * stream); }
//
// `false` means nothing was enqueued (argument outside the contract) or the launch was refused (the CUDA error is left
// for cudaPeekAtLastError), exactly as fn::act::quantize (fn/kernels/act/act.h:64-66), fn::embed::embed_rows
// (fn/kernels/embed/embed.h:85), fn::qsa::qsp_kv (fn/kernels/qsa/qsa_prompt.h:105), fn::experts::glu_finish
// (fn/kernels/experts/experts.h:277) and fn::draft::dcp_norm (fn/kernels/draft/draft_prompt.h:34) behave.  `stream` is a
// cudaStream_t passed as void * so this header stays CUDA-free, as the reference's headers do; null is the default
// stream.  The launchers own nothing, allocate nothing and never synchronise.
//
// The families keep the reference's names; the operators carry the formats this library implements (ggml Q8_0 / Q8_1 /
// Q4_K / IQ3_XXS next to the reference's own activation and KV8 formats).
#pragma once

#include <cstdint>

#include "fnb200.h"

namespace fnb {

constexpr uint32_t err_token = FNB_ERR_TOKEN;      // fn::xchg::err_token's role
constexpr uint32_t err_slot = FNB_ERR_SLOT;
constexpr uint32_t err_timeout = FNB_ERR_TIMEOUT;

namespace draft {  // hidden RMSNorm: fn::draft::dcp_norm's arithmetic, F32 out

struct norm_args {
    int64_t rows = 0;
    int32_t cols = 0;
    const float * x = nullptr;  // [rows][cols]
    const float * w = nullptr;  // [cols] or null
    float eps = 1e-6f;
    float * y = nullptr;        // [rows][cols]
};
inline bool dcp_norm(const norm_args & a, void * stream) {
    return fnb_rms_norm_f32(a.x, a.w, a.eps, a.y, a.rows, a.cols, stream) == FNB_OK;
}

}  // namespace draft

namespace act {  // fn::act::quantize and its ggml-format siblings

constexpr int32_t run = 32;

struct out_view {  // fn::act::out_view: codes int8 [rows][k], scales F32 [rows][k / 32][2]
    int8_t * codes = nullptr;
    float * scales = nullptr;
    int32_t rows = 0;
    int32_t k = 0;
    uint32_t * err = nullptr;  // not in fn::act::out_view: optional device error word (FNB_ERR_TIMEOUT)
};
inline bool quantize(const float * x, const out_view & o, void * stream) {
    return fnb_act_quantize(x, o.codes, o.scales, o.rows, o.k, o.err, stream) == FNB_OK;
}
inline bool quantize_q8_1(const float * x, void * blocks, int64_t rows, int32_t k, void * stream,
                          uint32_t * err = nullptr) {
    return fnb_quantize_q8_1(x, blocks, rows, k, err, stream) == FNB_OK;
}
inline bool quantize_q8_0(const float * x, void * blocks, int64_t rows, int32_t k, void * stream,
                          uint32_t * err = nullptr) {
    return fnb_quantize_q8_0(x, blocks, rows, k, err, stream) == FNB_OK;
}

}  // namespace act

namespace experts {  // SwiGLU + requantisation: fn::experts::glu_finish

// gs, us: F32 [n][cols] gate and up sums; the GLU leaves in the reference's activation format
// (err, not in the reference's signature: optional device error word for FNB_ERR_TIMEOUT)
inline bool glu_finish(const float * gs, const float * us, int64_t n, int32_t cols, int8_t * codes, float * scales,
                       void * stream, uint32_t * err = nullptr) {
    return fnb_swiglu_act(gs, us, codes, scales, nullptr, n, cols, err, stream) == FNB_OK;
}
// the same GLU as ggml Q8_1 blocks [n][cols / 32]; glu_f32 (optional) receives the F32 GLU the codes were made from
inline bool glu_finish_q8_1(const float * gs, const float * us, int64_t n, int32_t cols, void * blocks, float * glu_f32,
                            void * stream, uint32_t * err = nullptr) {
    return fnb_swiglu_q8_1(gs, us, blocks, glu_f32, n, cols, err, stream) == FNB_OK;
}

// the experts' gate / up mat-vec with the GLU over a decode window (fn::experts::cpu::kq_gu_rows for fmt q4_k, same
// bits): ff[t][r] = silu(gate row r . act[t]) * (up row r . act[t]); Q4_K rows back to back, Q8_K activation rows
inline bool gate_up_rows_q4_k(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                              int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_q4_k(gate, up, int64_t(n / 256) * 144, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                        r1, stream) == FNB_OK;
}
// the same for fmt q5_k (176-byte super-blocks)
inline bool gate_up_rows_q5_k(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                              int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_q5_k(gate, up, int64_t(n / 256) * 176, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                        r1, stream) == FNB_OK;
}
// the same for fmt iq3_xxs (fn::experts::cpu::iq_gu_rows, same bits); IQ3_XXS rows of n / 256 x 98 bytes back to back
inline bool gate_up_rows_iq3_xxs(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                                 int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_iq3_xxs(gate, up, int64_t(n / 256) * 98, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                           r1, stream) == FNB_OK;
}
// and for fmt iq3_s (rows of n / 256 x 110 bytes)
inline bool gate_up_rows_iq3_s(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                               int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_iq3_s(gate, up, int64_t(n / 256) * 110, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                         r1, stream) == FNB_OK;
}
// and for the IQ2 formats (66-, 74-, 82-byte super-blocks), as fn::experts::cpu::iq_gu_rows dispatches them
inline bool gate_up_rows_iq2_xxs(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                                 int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_iq2_xxs(gate, up, int64_t(n / 256) * 66, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                           r1, stream) == FNB_OK;
}
inline bool gate_up_rows_iq2_xs(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                                int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_iq2_xs(gate, up, int64_t(n / 256) * 74, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                          r1, stream) == FNB_OK;
}
inline bool gate_up_rows_iq2_s(const uint8_t * gate, const uint8_t * up, int32_t n, const void * act, int64_t act_stride,
                               int32_t nt, float * ff, int64_t ff_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_gate_up_rows_iq2_s(gate, up, int64_t(n / 256) * 82, n, act, act_stride, nt, ff, ff_stride, nullptr, r0,
                                         r1, stream) == FNB_OK;
}
inline bool quantize_q8_k(const float * x, void * blocks, int64_t rows, int32_t k, void * stream) {
    return fnb_quantize_q8_k(x, blocks, rows, k, stream) == FNB_OK;
}

// the experts' down mat-vec over a decode window (fn::experts::cpu::kq_down_rows for fmt q5_1, same bits): out[t][r] =
// Q5_1 weight row r . Q8_1 activation row t, r in [r0, r1); w rows back to back, act rows act_stride bytes apart
inline bool down_rows_q5_1(const uint8_t * w, int32_t n, const void * act, int64_t act_stride, int32_t nt, float * out,
                           int64_t out_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_down_rows_q5_1(w, int64_t(n / 32) * 24, n, act, act_stride, nt, out, out_stride, r0, r1, stream) == FNB_OK;
}

// the same with Q8_0 weights against Q8_0 activations (n a multiple of 128)
inline bool down_rows_q8_0(const uint8_t * w, int32_t n, const void * act, int64_t act_stride, int32_t nt, float * out,
                           int64_t out_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_down_rows_q8_0(w, int64_t(n / 32) * 34, n, act, act_stride, nt, out, out_stride, r0, r1, stream) == FNB_OK;
}
// fmt iq4_nl (fn::experts::cpu::iq4nl_down_rows, same bits): IQ4_NL weight rows against Q8_0 activation rows
inline bool down_rows_iq4_nl(const uint8_t * w, int32_t n, const void * act, int64_t act_stride, int32_t nt, float * out,
                             int64_t out_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_down_rows_iq4_nl(w, int64_t(n / 32) * 18, n, act, act_stride, nt, out, out_stride, r0, r1, stream) == FNB_OK;
}
// Q2_0 weights against the planar activation (fn::experts::cpu::quantize_act_q, q2_down_rows; same bits)
inline bool quantize_act_q(const float * x, int8_t * codes, float * scales, int64_t rows, int32_t n, void * stream) {
    return fnb_quantize_act_q(x, codes, scales, rows, n, stream) == FNB_OK;
}
inline bool down_rows_q2_0(const uint8_t * w, int32_t n, const int8_t * codes, const float * scales, int32_t nt, float * out,
                           int64_t out_stride, int64_t r0, int64_t r1, void * stream) {
    return fnb_expert_down_rows_q2_0(w, int64_t(n / 64) * 18, n, codes, n, scales, n / 32, nt, out, out_stride, r0, r1, stream) ==
           FNB_OK;
}

}  // namespace experts

namespace qsa {  // per-head norm + NeoX partial RoPE + KV append: fn::qsa::qsp_kv and attend's prepare phase

struct qsp_kv_args {
    const float * q = nullptr;        // [rows][n_q_heads][head_dim]; n_q_heads may be 0 (K/V only, as qsp_kv)
    const float * kv_k = nullptr;     // [rows][n_kv_heads][head_dim]
    const float * kv_v = nullptr;
    const float * q_norm = nullptr;   // [head_dim] or null
    const float * k_norm = nullptr;
    const int32_t * pos = nullptr;    // [rows] device: rotary position
    const int32_t * cells = nullptr;  // [rows] device: cache cell, or null = the position
    int64_t rows = 0, max_cells = 0;
    int32_t n_q_heads = 0, n_kv_heads = 1, head_dim = 256, n_rot = 64;
    float theta_scale = 0.0f;         // fnb_rope_theta_scale(freq_base, n_rot)
    float eps = 1e-6f;
    float * q_out = nullptr;          // [rows][n_q_heads][head_dim]
    void * k_cache = nullptr;         // Q8_0 cells, or int8 codes when k_scale / v_scale are set (KV8)
    void * v_cache = nullptr;
    uint16_t * k_scale = nullptr;     // KV8: both set, FP16 scales [max_cells][n_kv_heads][head_dim / 64]
    uint16_t * v_scale = nullptr;
    float * k_f32 = nullptr;          // optional: k after norm and rope, before quantising
    uint32_t * err = nullptr;
    const int32_t * planes = nullptr; // fn::qsa::qsp_kv_args::planes: device [rows][4] rotary planes of image rows
};
inline bool qsp_kv(const qsp_kv_args & a, void * stream) {
    fnb_rope_kv8_args w{};
    w.base.q = a.q, w.base.k = a.kv_k, w.base.v = a.kv_v, w.base.pos = a.pos, w.base.slots = a.cells;
    w.base.q_norm_w = a.q_norm, w.base.k_norm_w = a.k_norm, w.base.q_out = a.q_out;
    w.base.k_cache = a.k_cache, w.base.v_cache = a.v_cache, w.base.k_f32 = a.k_f32, w.base.err = a.err;
    w.base.rows = a.rows, w.base.cache_slots = a.max_cells;
    w.base.n_q_heads = a.n_q_heads, w.base.n_kv_heads = a.n_kv_heads, w.base.head_dim = a.head_dim;
    w.base.n_rot = a.n_rot, w.base.theta_scale = a.theta_scale, w.base.eps = a.eps, w.base.planes = a.planes;
    w.k_scale = a.k_scale, w.v_scale = a.v_scale;
    if ((a.k_scale != nullptr) != (a.v_scale != nullptr)) return false;  // KV8 needs both planes, as the reference
    return (a.k_scale != nullptr ? fnb_rope_neox_kv8_append(&w, stream) : fnb_rope_neox_q8_0_append(&w.base, stream)) ==
           FNB_OK;
}


// cache rows widened to F32 exactly as attention widens them (fn::qsa::kv8::decode4 for KV8, ggml's Q8_0 decode else);
// scale null: Q8_0 cells.  cells null: rows cell0 .. cell0 + rows - 1.
inline bool kv_read(const void * cache, const uint16_t * scale, const int32_t * cells, int64_t cell0, int64_t rows,
                    int64_t max_cells, int32_t n_kv_heads, int32_t head_dim, float * out, uint32_t * err, void * stream) {
    fnb_kv_read_args a{};
    a.cache = cache, a.scale = scale, a.cells = cells, a.out = out, a.err = err;
    a.rows = rows, a.cache_slots = max_cells, a.cell0 = cell0, a.n_kv_heads = n_kv_heads, a.head_dim = head_dim;
    return fnb_kv_read_f32(&a, stream) == FNB_OK;
}

}  // namespace qsa

namespace embed {  // token-embedding get_rows: fn::embed::embed_rows / check_tokens

enum class table_fmt : int32_t { q4_k, iq3_xxs, q8_0 };

struct rows_args {
    const void * table = nullptr;   // [n_vocab][row bytes], ggml block layout
    table_fmt fmt = table_fmt::q4_k;
    int64_t n_vocab = 0;
    const int32_t * tok = nullptr;  // [rows] device
    int64_t rows = 0;
    int32_t cols = 0;
    float * out = nullptr;          // [rows][cols]
    uint32_t * err = nullptr;       // err_token is OR-ed in for an id outside [0, n_vocab); that row stays unwritten
};
inline bool embed_rows(const rows_args & a, void * stream) {
    switch (a.fmt) {
        case table_fmt::q4_k: return fnb_get_rows_q4_k(a.table, a.n_vocab, a.tok, a.out, a.err, a.rows, a.cols, stream) == FNB_OK;
        case table_fmt::iq3_xxs: return fnb_get_rows_iq3_xxs(a.table, a.n_vocab, a.tok, a.out, a.err, a.rows, a.cols, stream) == FNB_OK;
        case table_fmt::q8_0: return fnb_get_rows_q8_0(a.table, a.n_vocab, a.tok, a.out, a.err, a.rows, a.cols, stream) == FNB_OK;
    }
    return false;
}
// embed_rows and the hidden RMSNorm of each row in one launch (Q4_K and IQ3_XXS tables): normed = (out * scale) * w
inline bool embed_rows_norm(const rows_args & a, const float * w, float eps, float * normed, void * stream) {
    if (a.fmt == table_fmt::q4_k) {
        return fnb_get_rows_rms_norm_q4_k(a.table, a.n_vocab, a.tok, w, eps, a.out, normed, a.err, a.rows, a.cols, stream) == FNB_OK;
    }
    if (a.fmt == table_fmt::iq3_xxs) {
        return fnb_get_rows_rms_norm_iq3_xxs(a.table, a.n_vocab, a.tok, w, eps, a.out, normed, a.err, a.rows, a.cols, stream) == FNB_OK;
    }
    return false;
}
// The reference's own layout (fn::embed::rows_args, fn/kernels/embed/embed.h:70-87): a card's IQ3_S or Q8_0 table of
// n_own features per token, decoded into own [rows][n_own], the card's columns of full [rows][n_full] and of all
// n_streams streams [rows][n_streams][n_full].  The reference's constants (1280, 2560, 4) are the defaults.
struct card_rows_args {
    const uint8_t * table = nullptr;  // the card's token_embd slice
    const int32_t * tok = nullptr;    // [rows] device
    int64_t n_vocab = 0;
    int32_t rows = 0;
    int32_t card = 0;
    float * own = nullptr;            // [rows][n_own]
    float * full = nullptr;           // [rows][n_full]
    float * streams = nullptr;        // [rows][n_streams][n_full]
    uint32_t * err = nullptr;
    bool q8 = false;                  // the table is Q8_0 instead of IQ3_S
    int32_t n_own = 1280, n_full = 2560, n_streams = 4;
};
inline fnb_embed_args to_c(const card_rows_args & a) {
    fnb_embed_args c{};
    c.table = a.table, c.tok = a.tok, c.own = a.own, c.full = a.full, c.streams = a.streams, c.err = a.err;
    c.n_vocab = a.n_vocab, c.rows = a.rows, c.fmt = a.q8 ? FNB_TABLE_Q8_0 : FNB_TABLE_IQ3_S;
    c.n_own = a.n_own, c.n_full = a.n_full, c.col0 = a.card * a.n_own, c.n_streams = a.n_streams;
    return c;
}
inline bool embed_rows(const card_rows_args & a, void * stream) {
    const fnb_embed_args c = to_c(a);
    return fnb_embed_rows(&c, stream) == FNB_OK;
}
// peer: the received [rows][n_own] of the other card (two-card layout: its columns are (1 - card) * n_own ..)
inline bool embed_join(const card_rows_args & a, const float * peer, void * stream) {
    const fnb_embed_args c = to_c(a);
    return fnb_embed_join(&c, peer, (1 - a.card) * a.n_own, stream) == FNB_OK;
}
// rows row0 .. row0 + n - 1 of the chunk take src [n][n_own] in own, full and every stream
inline bool embed_supply(const card_rows_args & a, const float * src, int32_t row0, int32_t n, void * stream) {
    const fnb_embed_args c = to_c(a);
    return fnb_embed_supply(&c, src, row0, n, stream) == FNB_OK;
}

// host check before upload: true when every id is in [0, n_vocab)
inline bool check_tokens(const int32_t * tok_host, int64_t rows, int64_t n_vocab) {
    return fnb_check_tokens(tok_host, rows, n_vocab) == 0;
}

}  // namespace embed
}  // namespace fnb
