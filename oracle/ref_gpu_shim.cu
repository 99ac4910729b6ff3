// TEST INFRASTRUCTURE.  C entry points over three of the REFERENCE'S OWN GPU launchers, whose translation units are
// compiled where they lie for sm_100a (oracle/Makefile, target ref-gpu) into oracle/_ref/libfnb_ref_gpu.so:
//
//   fn::draft::dcp_norm       fn/kernels/draft/draft_prompt.cu:26-68, :159-167   hidden RMSNorm, FP16 out
//   fn::experts::glu_finish   fn/kernels/experts/experts.cu:716-729, :1506-1513  SwiGLU + the activation format
//   fn::qsa::qsp_kv           fn/kernels/qsa/qsa_prompt_attn.cu:77-122, :440-454 K norm + rope, K / V into the KV8 cache
//
// They are the only executable statements of these three operations the reference holds (it has no CPU code for
// them), so GPU tests hold this library's kernels to them within the reference tests' bounds and report how many
// codes differ (their sincosf / expf / fmaf chains are the device's, not the C library's, so the bits are not expected
// to be equal everywhere).  Each launcher enqueues one plain kernel: no device-side wait, no cooperative launch.
// Nothing else of those translation units is called; the other launchers they reference are satisfied by the
// stubs below, which refuse.  Nothing in the product links this file.
#include <cmath>
#include <cstdint>

#include "fn/kernels/draft/draft_prompt.h"
#include "fn/kernels/experts/experts.h"
#include "fn/kernels/experts/experts_inst.h"
#include "fn/kernels/qsa/qsa_prompt.h"

// ---- what the three translation units reference but this library never calls ------------------------------------
namespace fn::qsa::attn {
float rope_theta_scale() { return powf(10000000.0f, -2.0f / 64.0f); }  // as fn/kernels/qsa/attend.cu:830-832
}  // namespace fn::qsa::attn

namespace fn::experts::detail {
#define FNB_REFUSE_GU(name)                                                                                        \
    bool name(fn::dense::fmt, fn::dense::fmt, int32_t, const gate_up_args &, cudaStream_t) { return false; }
FNB_REFUSE_GU(gate_up_q2_0)
FNB_REFUSE_GU(gate_up_q4_k)
FNB_REFUSE_GU(gate_up_q5_k)
FNB_REFUSE_GU(gate_up_q8_0)
FNB_REFUSE_GU(gate_up_iq2_s)
FNB_REFUSE_GU(gate_up_iq3_s)
FNB_REFUSE_GU(gate_up_iq2_xs)
FNB_REFUSE_GU(gate_up_iq2_xxs)
FNB_REFUSE_GU(gate_up_iq3_xxs)
#undef FNB_REFUSE_GU
bool gate_up_pair_iq2(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, const gate_up_pair_args &, cudaStream_t) { return false; }
bool gate_up_pair_iq3(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, const gate_up_pair_args &, cudaStream_t) { return false; }
bool gate_up_lanes_iq2(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, int32_t, const gate_up_lanes_args &, cudaStream_t) { return false; }
bool gate_up_lanes_iq3(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, int32_t, const gate_up_lanes_args &, cudaStream_t) { return false; }
bool gate_up_lanes_q4_k(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, int32_t, const gate_up_lanes_args &, cudaStream_t) { return false; }
bool gate_up_lanes_q5_k(fmt, fn::dense::fmt, fn::dense::fmt, int32_t, int32_t, const gate_up_lanes_args &, cudaStream_t) { return false; }
}  // namespace fn::experts::detail

// ---- the three launchers --------------------------------------------------------------------------------------------
extern "C" {

// rows <= 4096 positions of width 2560: e16 [rows][2560] = f16((emb enorm) rs), h16 [rows][4][2560] likewise from
// pred (row 0) and hidden rows t - 1; err bit 0: an FP16 overflow
int32_t fnbr_dcp_norm(int32_t rows, const float * emb, const float * hidden, const float * pred, const float * enorm,
                      const float * hnorm, uint16_t * e16, uint16_t * h16, uint32_t * err, void * stream) {
    fn::draft::norm_args a;
    a.rows = rows, a.emb = emb, a.hidden = hidden, a.pred = pred, a.enorm = enorm, a.hnorm = hnorm;
    a.e16 = e16, a.h16 = h16, a.err = err;
    return fn::draft::dcp_norm(a, stream) ? 0 : 1;
}

// n <= 50 rows of 320: codes int8 [n][320], scales {d, s} F32 [n][10][2]
int32_t fnbr_glu_finish(const float * gs, const float * us, int32_t n, int8_t * codes, float * scales, void * stream) {
    return fn::experts::glu_finish(gs, us, n, codes, scales, stream) ? 0 : 1;
}

// rows <= 4096 rows of 256 at cells pos0 .. pos0 + rows - 1: k = rope(norm(kv_k) k_norm) and v into int8 codes
// [max_cells][256] with FP16 scales [max_cells][64] (the first four of a cell are this layer's groups); rotary position
// pos0 + rope_off + t, or planes [rows][4] when given
int32_t fnbr_qsp_kv8(const float * kv_k, const float * kv_v, const float * k_norm, int32_t rows, int32_t pos0,
                     int32_t max_cells, int8_t * k_codes, int8_t * v_codes, uint16_t * k_scale, uint16_t * v_scale,
                     int32_t rope_off, const int32_t * planes, void * stream) {
    fn::qsa::qsp_kv_args a;
    a.kv_k = kv_k, a.kv_v = kv_v, a.k_norm = k_norm, a.rows = rows, a.pos0 = pos0, a.max_cells = max_cells;
    a.k_cache = reinterpret_cast<uint16_t *>(k_codes), a.v_cache = reinterpret_cast<uint16_t *>(v_codes);
    a.k_scale = k_scale, a.v_scale = v_scale, a.rope_off = rope_off, a.planes = planes;
    return fn::qsa::qsp_kv(a, stream) ? 0 : 1;
}

float fnbr_rope_theta_scale(void) { return fn::qsa::attn::rope_theta_scale(); }

}  // extern "C"
