/*
 * fnb200 - B200 (sm_100a) kernels for the FNFL engine's fused per-layer row-wise path, C ABI.
 *
 * The reference engine has no extern "C" layer: fn/model and fn/runtime call fn/kernels through one C++
 * convention, `bool fn::<family>::<op>(const <op>_args &, void * stream)` with raw device pointers, "false
 * and nothing enqueued" for an argument outside the contract, and a device error word for data-dependent
 * faults (fn/kernels/act/act.h:64-66, fn/kernels/embed/embed.h:56-60, fn/kernels/qsa/qsa_prompt.h:90-105,
 * fn/kernels/experts/experts.h:277, fn/kernels/draft/draft_prompt.h:34).  Each entry point below replaces one
 * of those launchers and keeps that convention: plain pointers and sizes, the caller owns every buffer, the
 * call only enqueues work on `stream` (a cudaStream_t passed as void *, null = the default stream), never
 * synchronises and never allocates, so it is legal inside stream capture.  include/fnb200_fn.hpp restores the
 * `bool op(args, stream)` spelling on top of these.
 *
 * Return value: FNB_OK (enqueued), FNB_REJECTED (argument outside the contract, nothing enqueued) or
 * FNB_LAUNCH_FAILED (the launch was refused; the CUDA error is left for cudaPeekAtLastError).
 * Device error word (`err`, optional): bits are OR-ed in by the kernel; the offending row is left unwritten.
 *
 * Numerics: built with --fmad=false; every product and sum that the CPU definition rounds separately is
 * rounded separately here.  Block layouts are ggml's (Q8_0 34 B, Q8_1 36 B, Q4_K 144 B, IQ3_XXS 98 B).
 */
#ifndef FNB200_H
#define FNB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FNB_OK 0
#define FNB_REJECTED 1
#define FNB_LAUNCH_FAILED 2

#define FNB_ERR_TOKEN 1u /* a token id outside [0, n_vocab): as fn::xchg::err_token in fn/kernels/embed/embed.h:37 */
#define FNB_ERR_SLOT 2u  /* a cache slot outside [0, cache_slots): fn/kernels/qsa/attend.h:109-110 */
#define FNB_ERR_TIMEOUT 4u /* a bounded in-kernel wait gave up (the reference's device waits do the same:
                              fn/kernels/qsa/attend.cu:264-281); the launch's outputs are incomplete */

#define FNB_Q8_0_BLOCK_BYTES 34
#define FNB_Q8_1_BLOCK_BYTES 36
#define FNB_Q4_K_BLOCK_BYTES 144
#define FNB_IQ3_XXS_BLOCK_BYTES 98

/* Library version (major * 10000 + minor * 100 + patch) and the name of a return code. */
int32_t fnb_version(void);
const char * fnb_status_name(int32_t status);

/*
 * Hidden RMSNorm, one row per token: y = (x * scale) * w, scale = 1 / sqrtf(mean(x^2) + eps), the sum of
 * squares accumulated in double.  w may be null (no weight).  x, y: F32 [rows][cols], 16-byte aligned, cols a
 * multiple of 4 in [4, 65536]; rows in [1, 2^31).  x and y may be the same buffer.
 * Replaces fn::draft::dcp_norm (fn/kernels/draft/draft_prompt.h:22-34, draft_prompt.cu:26-68) and the norm half
 * of draft_in_send / draft_in_recv (fn/kernels/draft/draft.h:110-139).
 */
int32_t fnb_rms_norm_f32(const float * x, const float * w, float eps, float * y, int64_t rows, int32_t cols,
                         void * stream);

/*
 * Per-head Q/K RMSNorm: the same norm over each head_dim-wide head of x [rows][n_heads][head_dim] with one
 * weight vector [head_dim] shared by all heads.  Stand-alone form of the norm that
 * fnb_rope_neox_q8_0_append fuses.  Replaces the norm half of norm_rope
 * (fn/kernels/qsa/attend.cu:153-171, fn/kernels/qsa/qsa_prompt_attn.cu:33-55).
 */
int32_t fnb_rms_norm_heads_f32(const float * x, const float * w, float eps, float * y, int64_t rows,
                               int32_t n_heads, int32_t head_dim, void * stream);

/*
 * SwiGLU fused with Q8_1 requantisation: v = (gate / (1 + expf(-gate))) * up in F32, then each run of 32
 * values becomes one ggml block_q8_1 {fp16 d, fp16 s = d * sum(q), int8 q[32]} with d = amax / 127,
 * id = 1 / d, q = roundf(v * id) (ggml/src/ggml-quants.c:300-333).  gate, up: F32 [rows][cols], 16-byte
 * aligned, cols a multiple of 32; out_q8_1: [rows][cols / 32] blocks, 16-byte aligned; out_f32 (optional,
 * F32 [rows][cols]) receives v before quantisation, which is how the reference's own tests pin the codes
 * (fn/kernels/experts/experts.h:45-47).  expf is evaluated exactly as glibc 2.39's non-FMA expf.
 * As with the rope entry points, the first call of each SwiGLU / requantiser variant on a device raises its
 * kernel's dynamic shared-memory limit (cudaFuncSetAttribute): make that first call outside a stream capture.
 * err (optional device error word, 4-byte aligned; the same for every SwiGLU / requantiser / fused-norm entry point
 * below): these kernels stage their input through a ring of shared-memory stages filled by bulk copies and every
 * wait on that ring is bounded; a wait that gives up sets FNB_ERR_TIMEOUT in *err, the launch ends by itself and
 * its outputs are incomplete.  With err null such a launch ends the same way, unreported.
 * Replaces fn::experts::glu_finish (fn/kernels/experts/experts.h:273-277, experts.cu:716-729) and the GLU
 * epilogues glu_out / glu_run (experts_gu.cuh:308-340, experts_dev.cuh:196-213).
 */
int32_t fnb_swiglu_q8_1(const float * gate, const float * up, void * out_q8_1, float * out_f32, int64_t rows,
                        int32_t cols, uint32_t * err, void * stream);

/*
 * The same GLU into the reference's own activation format: int8 codes [rows][cols] and F32 {d, s} pairs
 * [rows][cols / 32][2], d = amax / 127, id = 127 / amax, q = nearest-even(v * id) clamped to +-127,
 * s = d * (float) sum q (fn/kernels/act/act.h:8-15).  codes 16-byte aligned, scales 8-byte aligned.
 * Bitwise drop-in for fn::experts::glu_finish's outputs.
 */
int32_t fnb_swiglu_act(const float * gate, const float * up, int8_t * codes, float * scales, float * out_f32,
                       int64_t rows, int32_t cols, uint32_t * err, void * stream);

/*
 * Stand-alone requantisers of F32 [rows][cols] (cols a multiple of 32): ggml Q8_1 blocks, ggml Q8_0 blocks, and
 * the reference's activation format.  fnb_act_quantize replaces fn::act::quantize
 * (fn/kernels/act/act.h:57-66, act.cu:17-49); the Q8 forms replace the CPU quantize_q8_1 / quantize_q8_0 of
 * the expert miss path (fn/kernels/experts/experts_cpu.cpp:359-367) with ggml's reference rounding rule.
 */
int32_t fnb_quantize_q8_1(const float * x, void * out_q8_1, int64_t rows, int32_t cols, uint32_t * err, void * stream);
int32_t fnb_quantize_q8_0(const float * x, void * out_q8_0, int64_t rows, int32_t cols, uint32_t * err, void * stream);
int32_t fnb_act_quantize(const float * x, int8_t * codes, float * scales, int64_t rows, int32_t cols, uint32_t * err,
                         void * stream);

/*
 * Hidden RMSNorm fused with the requantisation of its output (the activation the next quantised mat-vec reads):
 * y as fnb_rms_norm_f32, then every 32 values of y become one Q8_1 / Q8_0 block or the reference's activation
 * format, exactly as the stand-alone requantisers would produce from y.  cols a multiple of 32, at most 4096;
 * out_f32 (optional, F32 [rows][cols]) receives y.  The reference fuses the same pair in its split hidden norm
 * (fn/kernels/draft/draft_in.cu:85-132, which writes the activation format: fn/kernels/draft/draft.h:110-139).
 * First call per device and variant sets a kernel attribute (see fnb_swiglu_q8_1).
 */
int32_t fnb_rms_norm_q8_1(const float * x, const float * w, float eps, void * out_q8_1, float * out_f32, int64_t rows,
                          int32_t cols, uint32_t * err, void * stream);
int32_t fnb_rms_norm_q8_0(const float * x, const float * w, float eps, void * out_q8_0, float * out_f32, int64_t rows,
                          int32_t cols, uint32_t * err, void * stream);
int32_t fnb_rms_norm_act(const float * x, const float * w, float eps, int8_t * codes, float * scales, float * out_f32,
                         int64_t rows, int32_t cols, uint32_t * err, void * stream);

/*
 * Optional per-head RMSNorm, NeoX partial-rotary RoPE, and Q8_0 quantise-and-append of K and V into the cache.
 * Per token t at rotary position pos[t] and cache slot slots[t] (or pos[t] when slots is null):
 *   q_out[t][h] = rope(norm(q[t][h]))            F32, all head_dim values (dims >= n_rot pass through)
 *   k_cache[slot][h] = Q8_0(rope(norm(k[t][h])))  8 blocks of 34 bytes per 256-wide head
 *   v_cache[slot][h] = Q8_0(v[t][h])
 * rope: pair i = (dim i, dim i + n_rot/2), angle = (float) pos * theta_scale^i built as an F32 product chain,
 * cosf / sinf evaluated exactly as glibc 2.39's non-FMA forms; y0 = x0 c - x1 s, y1 = x0 s + x1 c.
 * norm: as fnb_rms_norm_f32 over head_dim with q_norm_w / k_norm_w [head_dim]; null = no norm for that tensor.
 * k_f32 (optional, F32 [rows][n_kv_heads][head_dim]) receives k after norm and rope, before quantising.
 * A slot outside [0, cache_slots) sets FNB_ERR_SLOT in *err and nothing is written for that token.
 * head_dim in {64, 128, 256}; n_rot a multiple of 2 * (head_dim / 32), 0 <= n_rot <= head_dim; all pointers
 * 16-byte aligned (pos, slots 4-byte).  q_out may alias q.
 * The first call on a device raises the kernel's dynamic shared-memory limit (cudaFuncSetAttribute, once per
 * device and head_dim): make that first call outside a stream capture.  Shapes whose token tile does not fit in
 * shared memory, or whose n_rot is not a multiple of 64, run a slower row-per-warp kernel with the same results.
 * A bounded in-kernel wait that gives up sets FNB_ERR_TIMEOUT in *err.
 * planes (optional, n_rot 64 only): the reference's interleaved multi-section rotary positions for image rows
 * (fn/kernels/qsa/imrope.cuh:15-24, qsa_prompt.h:100-102): row t's rotary pair i takes its position from
 * planes[4 t + p(i)], p(i) = 1 for i % 3 == 1 below 33, 2 for i % 3 == 2 below 30, 0 for i % 3 == 0 below 33, else 3,
 * instead of pos[t]; the angle is that position times theta_scale^i by the same F32 product chain.  pos[t] is then
 * only the cache slot when slots is null.  Text rows hold one integer in all four planes, which is plain NeoX.
 * Replaces fn::qsa::qsp_kv (fn/kernels/qsa/qsa_prompt.h:90-105, qsa_prompt_attn.cu:77-122), the prepare phase
 * of fn::qsa::attn::attend (fn/kernels/qsa/attend.cu:153-260) and fn::draft::dcp_prepare
 * (fn/kernels/draft/draft_prompt.h:44-59).
 */
typedef struct fnb_rope_kv_args {
    const float * q;
    const float * k;
    const float * v;
    const int32_t * pos;
    const int32_t * slots;
    const float * q_norm_w;
    const float * k_norm_w;
    float * q_out;
    void * k_cache;
    void * v_cache;
    float * k_f32;
    uint32_t * err;
    int64_t rows;
    int64_t cache_slots;
    int32_t n_q_heads;
    int32_t n_kv_heads;
    int32_t head_dim;
    int32_t n_rot;
    float theta_scale;
    float eps;
    const int32_t * planes; /* optional, device [rows][4]: rotary position planes of image rows (see above); null = text */
} fnb_rope_kv_args;

int32_t fnb_rope_neox_q8_0_append(const fnb_rope_kv_args * args, void * stream);

/*
 * The same step into the reference's KV8 cache format: int8 codes [cache_slots][n_kv_heads][head_dim] and FP16
 * scales per 64 values [cache_slots][n_kv_heads][head_dim / 64] (fn/kernels/qsa/kv_q8.cuh:8-14, :29-52):
 * scale = fp16_rn(amax / 127), code = clamp(nearest-even(x / f32(scale)), +-127), 0 when the scale is 0.
 * k_cache / v_cache hold the codes, k_scale / v_scale the scales.  head_dim in {64, 128, 256}.
 */
typedef struct fnb_rope_kv8_args {
    fnb_rope_kv_args base;
    uint16_t * k_scale;
    uint16_t * v_scale;
} fnb_rope_kv8_args;

int32_t fnb_rope_neox_kv8_append(const fnb_rope_kv8_args * args, void * stream);

/* theta_scale = powf(freq_base, -2 / n_rot), the host-side constant of fn/kernels/qsa/attend.cu:830-832. */
float fnb_rope_theta_scale(float freq_base, int32_t n_rot);

/*
 * Token-embedding get_rows: out[t] = the dequantised row ids[t] of a quantised table [n_vocab][cols], F32,
 * bit-exact with ggml's row decoders (ggml/src/ggml-quants.c:1527-1549 Q4_K, :2573-2601 IQ3_XXS, :551-565
 * Q8_0).  table, out 16-byte aligned; cols a multiple of 256 (Q4_K, IQ3_XXS) or of 32 (Q8_0), at most 16384;
 * ids I32 [rows] on the device.  An id outside [0, n_vocab) sets
 * FNB_ERR_TOKEN in *err and leaves that output row unwritten.
 * Replaces fn::embed::embed_rows / fn::embed::embed (fn/kernels/embed/embed.h:56-87, embed_prompt.cu:26-107).
 */
int32_t fnb_get_rows_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                          int64_t rows, int32_t cols, void * stream);

/*
 * fnb_get_rows_q4_k (or _iq3_xxs) and the RMSNorm of the row in one pass: out[t] = the dequantised row ids[t] (the same bytes
 * fnb_get_rows_q4_k writes) and normed[t] = (out[t] * scale) * w, scale = 1 / sqrtf(mean(out[t]^2) + eps), the definition
 * of fnb_rms_norm_f32 (w may be null).  At cols = 2048 the decoded row never leaves the warp's registers between the two
 * steps, which saves the norm's read of the row (17.5 KB instead of 25.7 KB of traffic a token); other widths run the
 * two kernels in turn.  out and normed are distinct F32 [rows][cols] buffers, 16-byte aligned; the other arguments are
 * fnb_get_rows_q4_k's and fnb_rms_norm_f32's.  An id outside [0, n_vocab) sets FNB_ERR_TOKEN and leaves both rows
 * unwritten (other widths: the normalised row is then formed from whatever out held).
 * Replaces fn::embed::embed_rows followed by the hidden norm that reads its output (fn/kernels/embed/embed.h:56-87,
 * fn/kernels/draft/draft_prompt.cu:26-68).
 */
int32_t fnb_get_rows_rms_norm_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, const float * w, float eps,
                                   float * out, float * normed, uint32_t * err, int64_t rows, int32_t cols, void * stream);
/* the same for an IQ3_XXS table (row bytes a multiple of 2, as fnb_get_rows_iq3_xxs) */
int32_t fnb_get_rows_rms_norm_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, const float * w, float eps,
                                      float * out, float * normed, uint32_t * err, int64_t rows, int32_t cols, void * stream);
int32_t fnb_get_rows_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                             uint32_t * err, int64_t rows, int32_t cols, void * stream);
int32_t fnb_get_rows_q8_0(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err,
                          int64_t rows, int32_t cols, void * stream);

/*
 * The reference engine's own embedding layouts (fn/kernels/embed/embed.h:70-105, embed_prompt.cu:26-146): the table
 * holds `n_own` features of every token (one card's share) in IQ3_S (110-byte super-blocks, ggml-quants.c:2605-2644) or
 * Q8_0; each decoded row is written to own [rows][n_own], to columns col0 .. col0 + n_own - 1 of full [rows][n_full] and
 * to the same columns of each of n_streams streams [rows][n_streams][n_full] (null destinations are skipped; at least
 * one must be given).  The reference's fixed widths are arguments: its card r passes n_own 1280, n_full 2560,
 * col0 1280 r, n_streams 4; one GPU holding whole rows passes n_own = n_full, col0 = 0.
 *   fnb_embed_rows    decode (replaces fn::embed::embed_rows); a bad id sets FNB_ERR_TOKEN, its row stays unwritten
 *   fnb_embed_join    the peer card's F32 half [rows][n_own] into columns peer_col0 .. of full and the streams, skipping
 *                     rows whose id is bad (replaces fn::embed::embed_join)
 *   fnb_embed_supply  rows row0 .. row0 + n - 1 overwritten from src [n][n_own] in own, full and the streams
 *                     (replaces fn::embed::embed_supply)
 * All F32 pointers 16-byte aligned, n_own / n_full / col0 multiples of 4, n_own a multiple of 256 (IQ3_S) or 32 (Q8_0).
 */
#define FNB_TABLE_Q4_K 0
#define FNB_TABLE_IQ3_XXS 1
#define FNB_TABLE_Q8_0 2
#define FNB_TABLE_IQ3_S 3

typedef struct fnb_embed_args {
    const void * table;
    const int32_t * tok;
    float * own;
    float * full;
    float * streams;
    uint32_t * err;
    int64_t n_vocab;
    int64_t rows;
    int32_t fmt; /* FNB_TABLE_IQ3_S or FNB_TABLE_Q8_0 */
    int32_t n_own;
    int32_t n_full;
    int32_t col0;
    int32_t n_streams;
} fnb_embed_args;

int32_t fnb_embed_rows(const fnb_embed_args * args, void * stream);
int32_t fnb_embed_join(const fnb_embed_args * args, const float * peer, int32_t peer_col0, void * stream);
int32_t fnb_embed_supply(const fnb_embed_args * args, const float * src, int64_t row0, int64_t n, void * stream);

/*
 * Host-only: a minimal GGUF (v2 / v3) tensor-directory reader, so that a quantised table such as token_embd.weight can
 * be found in a model file and read row by row into host memory for upload.  It covers what this path needs of the
 * reference's fn/borrowed/gguf_tensors.h and fn/loader row slicing (fn/loader/loader.h); metadata is skipped except
 * general.alignment.  `type` is the ggml type number (0 F32, 1 F16, 8 Q8_0, 12 Q4_K, 18 IQ3_XXS, 21 IQ3_S); row_bytes
 * is 0 for a type this library does not decode.  fnb_gguf_open returns null for a missing or malformed file.
 */
typedef struct fnb_gguf fnb_gguf;
typedef struct fnb_gguf_tensor {
    int64_t ne[4];     /* extents, ne[0] = values per row; unused dims are 1 */
    int64_t offset;    /* from the start of the file's data section */
    int64_t row_bytes; /* ne[0] values in the tensor's block format */
    int64_t n_rows;    /* ne[1] * ne[2] * ne[3] */
    int32_t n_dims;
    int32_t type;
} fnb_gguf_tensor;

fnb_gguf * fnb_gguf_open(const char * path);
void fnb_gguf_close(fnb_gguf * g);
int64_t fnb_gguf_n_tensors(const fnb_gguf * g);
int32_t fnb_gguf_find(const fnb_gguf * g, const char * name, fnb_gguf_tensor * out);
int32_t fnb_gguf_read_rows(fnb_gguf * g, const fnb_gguf_tensor * t, int64_t row0, int64_t n_rows, void * dst_host);

/*
 * Reads cache rows back as F32, exactly as a consumer of the cache widens them: out[t][h][:] = the head_dim values of
 * cell cells[t] (or cell0 + t when cells is null), kv head h.  Q8_0 cells (scale null): value = fp16 d x code, ggml's
 * dequantize_row_q8_0 (ggml/src/ggml-quants.c:551-565).  KV8 (scale = the FP16 scale plane, cache = the int8 codes):
 * value = float(code) x f32(scale of its group of 64), exact in F32: fn::qsa::kv8::decode4
 * (fn/kernels/qsa/kv_q8.cuh:61-67), CPU fn::quant::kv_q8_value (fn/quant/kv_q8_ref.h).  The reference has no
 * stand-alone launcher for this (its attention widens cells in place); it is the read side of the append above, for
 * consumers that want F32 rows and for checking a cache.  A cell outside [0, cache_slots) sets FNB_ERR_SLOT and
 * leaves its row untouched.  head_dim in {64, 128, 256}; cache, out 16-byte aligned.
 */
typedef struct fnb_kv_read_args {
    const void * cache;
    const uint16_t * scale;
    const int32_t * cells;
    float * out;
    uint32_t * err;
    int64_t rows;
    int64_t cache_slots;
    int64_t cell0;
    int32_t n_kv_heads;
    int32_t head_dim;
} fnb_kv_read_args;

int32_t fnb_kv_read_f32(const fnb_kv_read_args * args, void * stream);

/*
 * Decode attention over the cache the append entry points write: for each of `rows` query rows t and query head h,
 *   out[t][h] = softmax over the row's cells c of (scale q[t][h] . K[c][g]) applied to V[c][g],  g = h / (n_q_heads / n_kv_heads),
 * times sigmoid(gate[t][h]) when gate is given (the reference's output gate).  q [rows][n_q_heads][head_dim] F32 is the
 * q_out of fnb_rope_neox_*_append (normed and roped); K and V are widened from the cache exactly as fnb_kv_read_f32
 * widens them: Q8_0 cells (k_scale and v_scale null) or KV8 codes with their FP16 scale planes.  Row t attends cells
 * first_cell[t] .. first_cell[t] + n_cells[t] - 1 (device arrays; null: every row attends the whole range); every row's
 * cells must lie inside [range_begin, range_end), a host-known bound from which the split over cells is laid out (cells
 * of the bound outside a row's own range are masked); a row range outside the cache sets FNB_ERR_SLOT and the row
 * attends nothing; a row with no cell gives zeros.  F32 softmax statistics; the products run on the 5th-generation
 * tensor cores (tcgen05.mma, F32 accumulators in tensor memory) with every operand split into two FP16 halves (q into a
 * rounded value and its rounded residual; K and V = d x code into the rounded product and its exact residual), which
 * keeps the reference's bound: max |error| / max |reference| <= 1e-5 per row and head against an FP64 evaluation over
 * the decoded cache (fn/kernels/qsa/qa2_test.cpp:469-520), for ranges of any length.  Values whose magnitude exceeds
 * FP16's range (65504) are outside the contract, and cache scales d below about 2^-10 lose low bits of d x code to
 * FP16 subnormals.  A kernel of this call holds all 512 columns of its SMs' tensor memory while it runs.
 * head_dim 128 or 256; rows x (n_q_heads / n_kv_heads) <= 64; n_kv_heads <= 1024; q, gate, out, caches 16-byte, scale
 * planes 8-byte aligned.
 * workspace: device memory of at least fnb_attend_workspace_bytes(args) bytes (16-byte aligned), the partial results of
 * the split over cells, folded by a second kernel of the same call; its contents need no initialisation and mean
 * nothing afterwards.  Calls that share a workspace must not overlap on the GPU.  The first call per device and shape
 * class raises a kernel attribute (fnb_prepare_device covers it).
 * Replaces the attention phase of fn::qsa::attn::attend for dense contiguous cell ranges (fn/kernels/qsa/attend.h:9-23,
 * :141; cache decode fn/kernels/qsa/kv_q8.cuh:61-67); the reference's selection format, and its fused prepare phase
 * (which fnb_rope_neox_*_append covers), are separate.
 */
typedef struct fnb_attend_args {
    const float * q;
    const float * gate;
    const void * k_cache;
    const void * v_cache;
    const uint16_t * k_scale;
    const uint16_t * v_scale;
    const int32_t * first_cell;
    const int32_t * n_cells;
    float * out;
    void * workspace;
    size_t workspace_bytes;
    uint32_t * err;
    int64_t cache_slots;
    int64_t range_begin;
    int64_t range_end;
    int32_t rows;
    int32_t n_q_heads;
    int32_t n_kv_heads;
    int32_t head_dim;
    float scale; /* the softmax scale, 1 / sqrt(head_dim) in the reference */
} fnb_attend_args;

size_t fnb_attend_workspace_bytes(const fnb_attend_args * args); /* 0 for a shape outside the contract */
int32_t fnb_attend(const fnb_attend_args * args, void * stream);

/*
 * fnb_attend for callers that have no workspace to pass and cannot allocate one.  It has no counterpart in the
 * reference (whose attention takes a caller-carved workspace, fn/kernels/qsa/attend.h:84-96).  Who needs it: an engine
 * that reserves all its device memory once at load and has none left to carve from; a plug-in whose host forbids
 * device allocation on the serving path, where an allocation stalls every stream of the device and may fail long after
 * start-up.  The partial results of the split over cells go into a fixed 16 MiB array inside the library's device
 * image instead of args->workspace (workspace and workspace_bytes are ignored): every GPU that loads the library holds
 * those 16 MiB until the process exits, used or not.  Same arguments, results (bit for bit) and return codes as
 * fnb_attend otherwise.
 *   - A shape whose partial results need more than 16 MiB (fnb_attend_workspace_bytes(args) > 16 << 20: very many KV
 *     heads or rows on a long range) is refused with FNB_REJECTED and one line on stderr; use fnb_attend for those.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current, checked); make that first call before any stream capture.  No call allocates or frees anything.
 *   - All calls share the one array per device and it keeps whatever the last call left there.  Nothing in it has to
 *     start at zero (every partial a call reads, that call wrote), so nothing is cleared; but two calls that overlap
 *     on the GPU (different streams, or one stream's graph branches) race on it.  Serialise them, or give all but one a
 *     workspace of their own through fnb_attend.
 */
int32_t fnb_attend_static(const fnb_attend_args * args, void * stream);

/*
 * F32 rows to ggml Q8_K blocks (292 bytes per 256 values: F32 d, 256 int8 codes, 16 int16 sums of 16 codes), the
 * activation format the routed experts' gate / up mat-vec reads on the reference's CPU tier.  Replaces
 * fn::experts::cpu::quantize_q8_k (fn/kernels/experts/cpu_kernels.h; cpu_iq_avx2.cpp:583-646) and ggml's
 * quantize_row_q8_K_ref (ggml/src/ggml-quants.c:2844-2881), same bytes: the value of largest magnitude (the first one
 * on ties) maps to -127, codes nearest-even capped at 127, d = 1 / iscale.  An all-zero block comes out as zeros,
 * sums included.  cols a multiple of 256; x 16-byte, out 4-byte aligned; out [rows][cols / 256] blocks.
 */
int32_t fnb_quantize_q8_k(const float * x, void * out_q8_k, int64_t rows, int32_t cols, void * stream);

/*
 * The routed experts' gate / up mat-vec for a decode window with the GLU fused: ff[t * ff_stride + r] = silu(g) u,
 * g = gate row r . act[t], u = up row r . act[t], for t < nt and r in [r0, r1).  ggml Q4_K weights (n / 256
 * super-blocks of 144 bytes a row, rows back to back: row_bytes = n / 256 * 144; row r of either matrix at
 * base + r row_bytes) against the Q8_K activations fnb_quantize_q8_k writes (row t at act + t act_stride).  Replaces
 * fn::experts::cpu::kq_gu_rows for fmt q4_k (fn/kernels/experts/cpu_kernels.h; cpu_kq_avx2.cpp:166-224, :362-380) and
 * returns the SAME BITS (lane structure, fused multiply-adds and reduction order of the AVX2 kernel; expf as the host C
 * library's generic build evaluates it).  gu (optional, windows of up to eight rows): [2][nt][ff_stride], g then u.
 * nt <= 64; the window's activations (nt x n / 256 x 292 bytes per pass of eight rows) must fit in 47 KB of shared
 * memory (n <= 5120 at eight rows); gate, up 16-byte, act, ff 4-byte aligned.
 */
int32_t fnb_expert_gate_up_rows_q4_k(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                     int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                     int64_t r1, void * stream);

/*
 * The same mat-vec with ggml Q5_K weights (n / 256 super-blocks of 176 bytes a row: row_bytes = n / 256 * 176): replaces
 * fn::experts::cpu::kq_gu_rows for fmt q5_k (cpu_kq_avx2.cpp:226-290 q5k_dot, :362-380) and returns the SAME BITS - the
 * Q4_K lane structure over 5-bit values, the mins as one scalar fused multiply-add a super-block.  Arguments and limits
 * as fnb_expert_gate_up_rows_q4_k.
 */
int32_t fnb_expert_gate_up_rows_q5_k(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                     int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                     int64_t r1, void * stream);

/*
 * The same mat-vec with ggml IQ3_XXS weights (n / 256 super-blocks of 98 bytes a row, rows back to back:
 * row_bytes = n / 256 * 98): replaces fn::experts::cpu::iq_gu_rows for fmt iq3_xxs (fn/kernels/experts/cpu_kernels.h:67;
 * cpu_iq_avx2.cpp:256-271, :305-337, :429-445) and returns the SAME BITS - eight int32 lanes a super-block of
 * (2 s + 1) x codebook bytes x sign-applied codes, one fused multiply-add a super-block with x.d y.d, ggml's
 * hsum_float_8 order, the format's 1/4 on the reduced sum, g / (1 + expf(-g)) * u - including for activation codes of
 * -128, which the reference's sign step leaves as they are.  Arguments as fnb_expert_gate_up_rows_q4_k.  n a multiple
 * of 512 up to 16384 (rows on 4-byte boundaries); nt <= 64 in passes of up to eight rows; gu only for windows of one
 * pass.  Uses more than the default shared memory: fnb_prepare_device covers it.
 */
int32_t fnb_expert_gate_up_rows_iq3_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                        int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                        int64_t r1, void * stream);

/*
 * And with ggml IQ3_S weights (110-byte super-blocks: row_bytes = n / 256 * 110): fn::experts::cpu::iq_gu_rows for fmt
 * iq3_s (cpu_iq_avx2.cpp:273-290 through the same row kernel), same bits - 9-bit codebook indices, plain sign bits, one
 * 4-bit scale per 32 values, K = 1.  Arguments and limits as fnb_expert_gate_up_rows_iq3_xxs.
 */
int32_t fnb_expert_gate_up_rows_iq3_s(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                      int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                      int64_t r1, void * stream);

/*
 * And with the three IQ2 formats (66-, 74- and 82-byte super-blocks: row_bytes = n / 256 * 66 / 74 / 82): fn::experts::cpu::
 * iq_gu_rows for fmt iq2_xxs, iq2_xs and iq2_s (cpu_iq_avx2.cpp:225-254, :341-414 row_dot_iq2xs, :551-565 the dispatch), same
 * bits - codebook entries of eight magnitudes (ggml/src/ggml-common.h:605, :672, :803), 7-bit sign indices with their
 * parity bit (IQ2_XXS, IQ2_XS) or plain sign bits (IQ2_S), a scale per 32 values (IQ2_XXS) or per 16 (IQ2_XS, IQ2_S), the
 * format's 1/8 folded into d with the pairwise reduction order (IQ2_XXS, IQ2_XS) or on the reduced sum in ggml's order
 * (IQ2_S).  Arguments and limits as fnb_expert_gate_up_rows_iq3_xxs.
 */
int32_t fnb_expert_gate_up_rows_iq2_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                        int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                        int64_t r1, void * stream);
int32_t fnb_expert_gate_up_rows_iq2_xs(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                       int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                       int64_t r1, void * stream);
int32_t fnb_expert_gate_up_rows_iq2_s(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act,
                                      int64_t act_stride, int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0,
                                      int64_t r1, void * stream);

/*
 * The consumer of the Q8_1 blocks fnb_swiglu_q8_1 writes: the routed experts' down mat-vec for a decode window,
 * out[t * out_stride + r] = weight row r . act[t] for t < nt and r in [r0, r1).  Weights are ggml Q5_1 rows (n / 32
 * blocks of 24 bytes: fp16 d, fp16 m, 32 high bits, 16 nibble bytes; value = d q + m), rows back to back
 * (row_bytes = n / 32 * 24), row r at w + r row_bytes; activations are nt rows of n / 32 Q8_1 blocks, row t at
 * act + t act_stride.  Replaces fn::experts::cpu::kq_down_rows for fmt q5_1 (fn/kernels/experts/cpu_kernels.h,
 * cpu_kq_avx2.cpp:293-320, :382-394) and returns the SAME BITS: eight F32 accumulators per (row, t) in the AVX2
 * kernel's lane order, one fused multiply-add per block and lane, the m x s side sum fused, hsum_float_8's reduction
 * order.  nt <= 64 (passes of eight rows, as the reference's); w 8-byte, act and out 4-byte aligned; act_stride a multiple
 * of 4; out_stride >= r1.  First call per device raises a kernel attribute (see fnb_prepare_device).
 */
int32_t fnb_expert_down_rows_q5_1(const void * w, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                                  int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1, void * stream);

/*
 * The same mat-vec with ggml Q8_0 weights (34-byte blocks) against Q8_0 activations (fnb_quantize_q8_0 /
 * fnb_rms_norm_q8_0 blocks): fn::experts::cpu::kq_down_rows for fmt q8_0 (cpu_kq_avx2.cpp:322-344), same bits (eight
 * accumulators, one fused multiply-add per block and lane with the product of the two block scales, no side sum).
 * The same bits hold for activation codes in [-127, 127], which is every code ggml's Q8_0 quantiser and
 * fnb_quantize_q8_0 emit; a hand-made -128 code under a negative weight differs (the AVX2 kernel's sign step leaves
 * -128 as it is; only the IQ4_NL and IQ gate / up entry points reproduce that corner).
 * n a multiple of 128 (rows are whole 8-byte pairs); row_bytes = n / 32 * 34; w 8-byte, act 2-byte aligned.
 */
int32_t fnb_expert_down_rows_q8_0(const void * w, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                                  int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1, void * stream);

/*
 * The same mat-vec with ggml IQ4_NL weights (18-byte blocks: fp16 d, 16 nibble bytes indexing kvalues_iq4nl) against
 * Q8_0 activations: fn::experts::cpu::iq4nl_down_rows (fn/kernels/experts/cpu_kernels.h:73; cpu_iq_avx2.cpp:481-514,
 * :571-578), same bits - eight accumulators, one fused multiply-add per block and lane with the product of the two block
 * scales, |w| times the code with w's sign applied (a -128 code stays -128, as _mm256_sign_epi8 leaves it), that file's
 * hsum8 order.  n a multiple of 64 up to 8192 (rows on 4-byte boundaries, blocks in pairs); row_bytes = n / 32 * 18;
 * w 16-byte, act 2-byte, out 4-byte aligned; act_stride even.  Uses more than the default shared memory:
 * fnb_prepare_device covers it.
 */
int32_t fnb_expert_down_rows_iq4_nl(const void * w, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                                    int32_t nt, float * out, int64_t out_stride, int64_t r0, int64_t r1, void * stream);

/*
 * The reference engine's planar 32-value activation: per chunk of 32 values s = amax / 127 and codes
 * trunc(x / s +- 0.5) in +-127 (half away from zero; inv = 1 / s is what multiplies).  codes int8 [rows][n], scales F32
 * [rows][n / 32], both dense.  Replaces fn::experts::cpu::quantize_act_q (fn/kernels/experts/cpu_kernels.h:45-62;
 * cpu_q2_avx2.cpp:180-226) for codes and scales, same bits on finite inputs.  n a multiple of 32; x, codes 16-byte aligned.
 */
int32_t fnb_quantize_act_q(const float * x, int8_t * codes, float * scales, int64_t rows, int32_t n, void * stream);

/*
 * The down mat-vec with the reference engine's Q2_0 weights (64-weight blocks of 18 bytes: fp16 d, 16 bytes of 2-bit
 * codes, value 4 i + k at bits 2 k of byte i, weight d (c - 1); rows back to back, row_bytes = n / 64 * 18) against the
 * planar activation fnb_quantize_act_q writes (row t's codes at codes + t codes_stride, its chunk scales at
 * scales + t scales_stride): replaces fn::experts::cpu::q2_down_rows (cpu_kernels.h:78-81; cpu_q2_avx2.cpp:62-146),
 * same bits - per pair of blocks eight lanes of sum(c q) - sum(q) in integers, times the chunk scale, one fused
 * multiply-add by d, an output reduced as ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7)).  n a multiple of 128 up to
 * 8192; codes 16-byte aligned, codes_stride a multiple of 16; other arguments as fnb_expert_down_rows_q5_1.
 */
int32_t fnb_expert_down_rows_q2_0(const void * w, int64_t row_bytes, int32_t n, const int8_t * codes, int64_t codes_stride,
                                  const float * scales, int64_t scales_stride, int32_t nt, float * out, int64_t out_stride,
                                  int64_t r0, int64_t r1, void * stream);

/*
 * Host-side check before upload: 0 when every id is in [0, n_vocab), else 1 + the index of the first bad id.
 * Replaces fn::embed::check_tokens (fn/kernels/embed/embed.h:56).
 */
int64_t fnb_check_tokens(const int32_t * ids_host, int64_t rows, int64_t n_vocab);

/*
 * Optional, once per device (the current one): performs the one-time kernel attribute set-up (cudaFuncSetAttribute for
 * the kernels that use more than 48 KB of shared memory) that the SwiGLU / requantiser, fused-norm and rope entry
 * points otherwise perform on their first call.  After it every entry point is legal inside a stream capture from
 * its first call on.  No counterpart in the reference (its launchers have the same first-call rule and the engine
 * warms them before recording its graphs).  FNB_OK, or FNB_LAUNCH_FAILED when a CUDA call fails.
 */
int32_t fnb_prepare_device(void);

#ifdef __cplusplus
}
#endif
#endif
