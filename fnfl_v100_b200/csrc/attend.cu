// Decode attention over the 8-bit KV cache this library appends: the consumer of fnb_rope_neox_*_append's outputs.
//
//   out[t][h] = softmax_c(scale q[t][h] . K[c][g]) . V[c][g]  over row t's cells c,  g = h / (n_q_heads / n_kv_heads)
//               (optionally times sigmoid(gate[t][h]), the reference's output gate)
//
// with K and V widened from the cache exactly as fnb_kv_read_f32 widens them (Q8_0: fp16 d x code; KV8: code x scale
// of its group of 64), F32 softmax statistics and accumulators.  It replaces the attention phase of
// fn::qsa::attn::attend (fn/kernels/qsa/attend.h:9-23, :141) for dense, contiguous cell ranges (the reference's cell
// selection format is not part of this path) and keeps its bound: max |error| / max |reference| <= 1e-5 per row and
// head against an FP64 reference over the decoded cache (fn/kernels/qsa/qa2_test.cpp:469-520).
//
// Roofline: the cache is read once, 2 x 272 bytes per cell and KV head (Q8_0), shared by every query row of the
// head's group; the work per byte is a contraction (M = rows x heads per group query rows against every cell), so both
// products run on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory) and everything else is
// shaped around feeding them:
//
//   * Split precision.  The 1e-5 bound needs products far more exact than 11-bit operands give, so every operand is
//     two FP16 operands, value = hi + lo (about 22 bits):  q = q_hi + q_lo (rounded residual);  K and V = d x code,
//     split EXACTLY (hi = the rounded product, lo = the fused residual, one half2 instruction each per two values);
//     p = p_hi + p_lo (scaled by 2^12 to stay clear of FP16's subnormals).
//   * Stacked rows.  A group has at most 64 query rows and the MMA is 128 rows tall: row 2 r of the A operand holds
//     query row r's hi part and row 2 r + 1 its lo part, so ONE pass over the B operand gives hi . B and lo . B in
//     adjacent accumulator rows (adjacent lanes of tensor memory: a shuffle adds them).  Scores: S = [q_hi; q_lo] .
//     (K_lo + K_hi)^T, the small K_lo products first.  Outputs: row 2 r: p_hi . V_hi; row 2 r + 1: p_lo . V_hi +
//     p_hi . V_lo, through an alternate probability operand whose even rows are zero.  The order matters: the tensor
//     core adds into its F32 accumulator by truncation (about 0.7 x 2^-24 of relative bias per accumulating MMA), so
//     the large accumulator rows take as few steps as possible (16 per score tile, 4 per tile of outputs) and a work
//     unit is capped at 24 tiles (make_plan); partial results of units are combined in round-to-nearest F32.
//   * The stacked operands (query rows, probabilities) live in TENSOR memory, a row per lane, two FP16 values per
//     column, written by tcgen05.st straight from the registers that made them; only the cell operands are in shared
//     memory.  Tensor-memory columns: 64 scores | head_dim outputs | head_dim / 2 query | 32 + 32 probabilities = 512
//     at head_dim 256, all there are.
//   * Cell operand tiles in shared memory are written directly in the MMA's canonical layout: 64-dim blocks of
//     [cell][128 bytes] with the 16-byte chunks XOR-swizzled by the cell's low three bits (the 128-byte swizzle).  The
//     same bytes serve as a K-major operand (rows = cells, for the scores) and as an MN-major operand (contiguous =
//     dims, for the outputs), so K and V are widened by the same code: a thread takes one Q8_0 block (or 32 KV8 codes)
//     of one cell and stores four 16-byte chunks each of hi and lo; consecutive lanes take consecutive cells, so the
//     eight lanes of a store phase fall on eight different chunks.
//   * Cells arrive in a two-stage ring of raw tiles, a tile or two ahead.  One thread of a warp of its own asks for
//     them: ONE tensor-map copy (cp.async.bulk.tensor) per tensor and tile, completion counted in bytes on the stage's
//     mbarrier.  Q8_0 at head_dim 256: box = 64 cells x one head's 272 bytes, laid out densely (68 words a cell: the
//     raw loads of eight consecutive cells fall on different banks).  KV8: a cell is one or two rows of 128 bytes, box =
//     64 cells x one head's rows with the copy's 128-byte swizzle, which the raw loads undo (two-way conflicts instead
//     of the eight-way ones of dense 256-byte cells); its scales, 8 bytes a cell, stay 8-byte asynchronous copies by
//     64 workers.  Q8_0 at head_dim 128 (136 bytes a cell: no 16-byte stride) and drivers without the encoder use
//     16-byte asynchronous copies issued by the workers, consecutive threads taking consecutive pieces so that the
//     copies cover whole cache lines (a thread reading its own cell straight from the cache touched 32 lines per warp
//     instruction and kept the L1 pipe busy 80 % of the time).  Those 2 x 1088 copies a tile cost each worker 0.29 us
//     per tensor - more than widening its item - because they are bound by the load / store unit's rate; the
//     tensor-map copies do not pass through it (Q8_0 0.142 -> 0.123 ms, KV8 0.138 -> 0.130).
//   * Sixteen worker warps and one that only issues the MMAs; completion comes back through mbarriers
//     (tcgen05.commit).  A worker's tile: read the tile's scores into registers; widen the NEXT tile's K (its operand
//     is free, and with S read the next scores can run at once); then this tile's softmax and its V.  The issuer sends
//     the next tile's scores before this tile's outputs, so both products run under the workers' arithmetic (a
//     timeline of one CTA showed the old order - K, V, softmax, each tile's scores waited for - spending a third of a
//     tile waiting on the score MMAs).  Softmax: warps w, w + 4, w + 8, w + 12 share tensor-memory quarter w & 3 and take a
//     quarter of the tile's cells each; a lane pair is one query row (hi lane, lo lane), a thread 8 cells of it.  The
//     row maximum crosses the quarter's four warps through shared memory and a 128-thread barrier.  The maximum is
//     lazy: the reference point moves only when a row's maximum has outgrown it by more than 2^3, and only then are the
//     row's accumulators rescaled in tensor memory.
//   * Split over cells (flash decoding): a work unit is (KV head, range of cells), about two per SM; a unit writes
//     (reference point, sum, unnormalised output) partials into a caller-supplied workspace, and a second small kernel
//     folds them in a fixed order, divides, gates and writes the rows.  The workspace is the only global memory beyond
//     inputs and outputs; its size is a function of the shape (fnb_attend_workspace_bytes).
//
// Every wait is bounded (bulk_pipe.cuh): one that runs out ORs FNB_ERR_TIMEOUT into the error word and the kernel
// carries on to its end, where tensor memory is freed.  No kernel here waits on another: the fold is a second launch
// on the same stream.  Nothing here reads another GPU's memory.
#include <atomic>
#include <cstdio>

#include <cuda.h>  // CUtensorMap and the type of cuTensorMapEncodeTiled (reached through cudaGetDriverEntryPoint: nothing links to the driver library)
#include <cuda_fp16.h>

#include "bulk_pipe.cuh"
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kThreads = 512;  // sixteen worker warps: four per scheduler hide each other's latencies
constexpr int kLaunchThreads = kThreads + 32;
constexpr int kLaunchThreadsTma = kLaunchThreads + 32;  // + the warp whose first lane asks for the tiles (tensor-map copies)  // and a warp that only issues the MMAs (a thread that issues them waits on the tensor core's queue: as a worker it held up every barrier)
constexpr int kTile = 64;   // cells per tile: the N of the score MMA, four K steps of the output MMA
constexpr int kMaxM = 64;   // query rows of one KV head's group: rows x (n_q_heads / n_kv_heads)
constexpr float kPScale = 4096.0f, kPUnscale = 1.0f / 4096.0f;
constexpr float kLazy = 3.0f;  // log2 units a row's maximum may exceed its reference point: p <= 8, p x 2^12 fits FP16
constexpr float kLog2e = 1.4426950408889634f;

struct attend_plan {
    int m, parts;            // query rows per group; partial results a unit writes (1)
    int64_t unit_cells;      // cells per work unit (a multiple of kTile)
    int n_units;             // units per KV head
    int64_t slots;           // partial results in the workspace: n_kv x n_units x parts
};

// The split the launcher and the workspace size agree on: about two units per SM over all KV heads, never shorter than
// 256 cells and never longer than 24 tiles.  The cap is a matter of accuracy, not speed: the tensor core adds into its
// F32 accumulator by truncation, about 0.7 x 2^-24 of relative bias per accumulation step, and a unit's output rows take
// four such steps per tile; 24 tiles keep that below 5e-6 of the 1e-5 bound.  Partials are combined by the fold kernel
// in round-to-nearest F32.
constexpr int kMaxUnitTiles = 24;
inline attend_plan make_plan(int rows, int n_q, int n_kv, int64_t range) {
    attend_plan p;
    p.m = rows * (n_q / n_kv);
    p.parts = 1;
    int64_t want = (2 * int64_t(kSmCount) + n_kv - 1) / n_kv;
    int64_t cells = (range + want - 1) / want;
    cells = cells < 256 ? 256 : cells;
    cells = cells > int64_t(kMaxUnitTiles) * kTile ? int64_t(kMaxUnitTiles) * kTile : cells;
    p.unit_cells = (cells + kTile - 1) / kTile * kTile;
    p.n_units = int((range + p.unit_cells - 1) / p.unit_cells);
    if (p.n_units < 1) p.n_units = 1;
    p.slots = int64_t(n_kv) * p.n_units * p.parts;
    return p;
}
// workspace: (reference point, sum) pairs, padded to 16 bytes so that the outputs behind them take 128-bit stores, then
// the outputs
inline size_t plan_ml_floats(const attend_plan & p) { return (size_t(p.slots) * p.m * 2 + 3) / 4 * 4; }
inline size_t plan_bytes(const attend_plan & p, int head_dim) {
    return (plan_ml_floats(p) + size_t(p.slots) * p.m * head_dim) * 4;
}

struct attend_params {
    const float * q;
    const float * gate;
    const uint8_t * k_cache;
    const uint8_t * v_cache;
    const uint16_t * k_scale;
    const uint16_t * v_scale;
    const int32_t * first_cell;
    const int32_t * n_cells;
    float * out;
    float * ws_ml;   // [slots][m][2]: reference point (in log2 units) and sum
    float * ws_acc;  // [slots][m][head_dim]
    uint32_t * err;
    int64_t cache_slots, range_begin, range_end, unit_cells;
    int rows, n_q, n_kv, n_rep, m, parts, n_units;
    float scale_log2;  // softmax scale x log2(e)
};

// ---- small wrappers -------------------------------------------------------------------------------------------------
// 16 (or 8) bytes global -> shared; src_bytes = 0 writes zeros instead (cells past the end of a unit)
__device__ __forceinline__ void cp_async16(void * dst, const void * src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async8(void * dst, const void * src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 8 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(void * dst, const void * src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 4 : 0) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// four int8 codes of a word -> two half2 of their exact values: each biased byte under FP16's 2^10 exponent is
// 1024 + 128 + code, less 1152 the code
__device__ __forceinline__ void codes_to_h2(uint32_t w, __half2 & lo, __half2 & hi) {
    const uint32_t b = w ^ 0x80808080u;
    const __half2 bias = bits_h2(0x64806480u);
    lo = __hsub2(bits_h2(__byte_perm(b, 0x64646464u, 0x4140u)), bias);
    hi = __hsub2(bits_h2(__byte_perm(b, 0x64646464u, 0x4342u)), bias);
}

// one tile of a 3-D tensor (box given by the tensor map) global -> shared, completion counted in bytes on `bar`; x, y, z
// from the innermost dimension out (x times the element size must be a multiple of 16 bytes: it is always 0 here)
__device__ __forceinline__ void tensor_g2s(void * dst_smem, const CUtensorMap * map, int x, int y, int z, uint64_t * bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst_smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tensor_g2s4(void * dst_smem, const CUtensorMap * map, int x, int y, int z, int w, uint64_t * bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
            smem_u32(dst_smem)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
        : "memory");
}

// ---- tensor memory and the MMA --------------------------------------------------------------------------------------
// Shared-memory matrix descriptor of an operand in the 128-byte-swizzled canonical layout: start address, leading and
// stride byte offsets (in 16-byte units), descriptor version 1, layout type 2 (128-byte swizzle).
//   K-major (rows of 128 bytes = 64 FP16 along K): stride offset = bytes between 8-row groups; leading offset unused.
//   MN-major (rows of 128 bytes = 64 FP16 along MN, one row per K index): stride offset = bytes between groups of 8 K
//   indices, leading offset = bytes between 64-element blocks along MN.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return uint64_t((saddr & 0x3ffffu) >> 4) | (uint64_t(leading_bytes >> 4) << 16) | (uint64_t(stride_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::f16: F32 accumulator, FP16 A and B, A K-major, B K-major or MN-major, M = 128, N
__host__ __device__ constexpr uint32_t umma_idesc(int n, bool b_mn_major) {
    return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}
// D (+)= A . B: the A operand in tensor memory (one operand row per lane, two FP16 values per column), B in shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the barrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// generic-proxy writes to shared memory made visible to the tensor core's (async proxy) reads
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t * slot, uint32_t cols) {  // one whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {  // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// 32 consecutive columns of this thread's lane (the warp's quarter of tensor memory: lanes 32 (warp % 4) ..)
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const float (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                   "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
                   "r"(__float_as_uint(v[7]))
                 : "memory");
}
// barrier among `threads` threads on hardware barrier `id` chosen at run time
__device__ __forceinline__ void named_barrier_id(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- shared and tensor memory ---------------------------------------------------------------------------------------
// Cell operand tiles in shared memory: 64-dim blocks of [cell][128 bytes]; chunk c of cell r sits at chunk c ^ (r & 7).
// The stacked operands (query rows, probabilities) live in TENSOR memory, one operand row per lane, two FP16 values per
// 32-bit column: the tensor core then reads only the cell operand from shared memory (with the stacked operand there
// too, its 4 KB per MMA made shared-memory bandwidth the bound).  Stacked rows interleave the parts: lane 2 r holds
// query row r's hi part, lane 2 r + 1 its lo part, so a query row's two accumulator rows sit in adjacent lanes of one
// 32-lane quarter.
template <int HD, bool KV8, bool TMA = false>
struct tc_layout {
    static constexpr int kBlocks = HD / 64;
    static constexpr int kCBlock = kTile * 128;               // a block of a cell operand
    static constexpr int kCell = KV8 ? HD : HD / 32 * 34;     // raw bytes of a cell
    // a cell's stride in the raw tile: a multiple of 16 bytes (the copies) that is NOT a multiple of 128, so that the
    // 16-byte loads of eight consecutive cells fall on different banks (KV8's 256 put all eight on the same four).
    // A tensor-map copy lays the box out densely; KV8's cells are then kept apart by the copy's own 128-byte swizzle
    // (16-byte chunk c of the 128-byte row at address a sits at chunk c ^ ((a >> 7) & 7)), which wants the tile's base
    // on a 1024-byte boundary.
    static constexpr bool kSwizzled = KV8 && TMA;
    static constexpr int kRawCell = kSwizzled ? kCell : kCell % 128 == 0 ? kCell + 16 : kCell;
    static constexpr int kRawTensor = kSwizzled ? (kTile * kCell + kTile * 8 + 1023) / 1024 * 1024
                                                : kTile * kRawCell + (KV8 ? kTile * 8 : 0);  // a tensor's raw tile (KV8: + scales, 8-byte slots)
    static constexpr int kRawStage = 2 * kRawTensor;          // K raw | V raw
    static constexpr int k_hi = 0;
    static constexpr int k_lo = k_hi + kBlocks * kCBlock;
    static constexpr int v_hi = k_lo + kBlocks * kCBlock;
    static constexpr int v_lo = v_hi + kBlocks * kCBlock;
    static constexpr int raw = v_lo + kBlocks * kCBlock;      // [2 stages][K raw | V raw]: the cells as they lie in the cache
    static constexpr int part_max = raw + 2 * kRawStage;      // float [2][4][64]: a row's maximum over each quarter of a tile, by tile parity
    static constexpr int bars = part_max + 2 * 4 * kMaxM * 4; // ten mbarriers
    static constexpr int misc = bars + 128;                    // tensor-memory base, the give-up flag
    static constexpr int total = misc + 16 + 1024;            // + slack to align the base to 1024 bytes
    // tensor-memory columns: scores | outputs | stacked query rows | stacked probabilities | the alternate probabilities
    static constexpr uint32_t t_s = 0, t_o = 64, t_q = t_o + HD, t_p = t_q + HD / 2, t_alt = t_p + 32;
    static constexpr uint32_t kTmemCols = 512;
    static_assert(t_alt + 32 <= kTmemCols, "tensor memory of one SM");
    static_assert(total <= 232448, "shared memory of one CTA");
};
__device__ __forceinline__ uint32_t op_at(int row, int chunk) { return uint32_t(row) * 128u + (uint32_t(chunk ^ (row & 7)) << 4); }

// ---- a thread's share of a tile of raw cells, in registers ----------------------------------------------------------
// Q8_0: one pair of blocks of a cell, 68 bytes = 17 aligned words: d0 | 32 codes | d1 | 32 codes.  KV8: 64 codes and
// their group's scale.  Cells past the end of the unit read as zeros.
template <bool KV8>
struct raw_item {
    uint32_t w[KV8 ? 8 : 9];
    uint32_t scale;  // KV8: the group's FP16 scale bits
};
// blk: the item's 32-dim block of the cell.  Q8_0: the block's 34 bytes lie in nine aligned words of its pair of blocks
// (68 bytes = 17 words): words 0 .. 8 for the pair's first block (d in the low half of word 0, codes from its high
// half on), words 8 .. 16 for the second (d in the high half of word 8, codes in words 9 .. 16).
// from the staged raw tile: `cell_raw` the cell's bytes, `cell_scales` (KV8) its FP16 group scales
// SWZ: the raw tile was laid out by a tensor-map copy with the 128-byte swizzle (its base on a 1024-byte boundary):
// chunk c of a cell's 128-byte row number `row` (counted from the tile's base) sits at chunk c ^ (row & 7).
template <int HD, bool KV8, bool SWZ = false>
__device__ __forceinline__ void load_item(raw_item<KV8> & r, const uint8_t * cell_raw, const uint8_t * cell_scales, int blk, int cell = 0) {
    if (KV8) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            int at = 32 * blk + 16 * j;
            if (SWZ) {
                const int row = cell * (HD / 128) + (blk >> 2), chunk = (2 * (blk & 3) + j) ^ (row & 7);
                at = 128 * (blk >> 2) + 16 * chunk;
            }
            const uint4 v = *reinterpret_cast<const uint4 *>(cell_raw + at);
            r.w[4 * j] = v.x, r.w[4 * j + 1] = v.y, r.w[4 * j + 2] = v.z, r.w[4 * j + 3] = v.w;
        }
        r.scale = reinterpret_cast<const uint16_t *>(cell_scales)[blk >> 1];
    } else {
        const uint32_t * src = reinterpret_cast<const uint32_t *>(cell_raw + 68 * (blk >> 1)) + 8 * (blk & 1);
#pragma unroll
        for (int j = 0; j < 9; ++j) r.w[j] = src[j];
        r.scale = 0;
    }
}
// widen the item into the hi and lo operand tiles: value = d x code, hi = rn(value), lo = value - hi.  SECOND: the
// item is the second block of its pair (the same for every thread of a warp).
template <bool KV8, bool SECOND>
__device__ __forceinline__ void widen_half(const raw_item<KV8> & r, int cell, int blk, uint8_t * t_hi, uint8_t * t_lo) {
    const __half d = __ushort_as_half(uint16_t(KV8 ? r.scale : SECOND ? r.w[0] >> 16 : r.w[0] & 0xffffu));
    const __half2 d2 = __half2half2(d);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t c0, c1;
        if (KV8) {
            c0 = r.w[2 * j], c1 = r.w[2 * j + 1];
        } else if (!SECOND) {
            c0 = __funnelshift_r(r.w[2 * j], r.w[2 * j + 1], 16), c1 = __funnelshift_r(r.w[2 * j + 1], r.w[2 * j + 2], 16);
        } else {
            c0 = r.w[2 * j + 1], c1 = r.w[2 * j + 2];
        }
        __half2 c[4], h[4], l[4];
        codes_to_h2(c0, c[0], c[1]);
        codes_to_h2(c1, c[2], c[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            h[e] = __hmul2(d2, c[e]);
            l[e] = __hfma2(d2, c[e], __hneg2(h[e]));
        }
        const uint32_t at = uint32_t(blk >> 1) * (kTile * 128) + op_at(cell, 4 * (blk & 1) + j);
        *reinterpret_cast<uint4 *>(t_hi + at) = make_uint4(h2_bits(h[0]), h2_bits(h[1]), h2_bits(h[2]), h2_bits(h[3]));
        *reinterpret_cast<uint4 *>(t_lo + at) = make_uint4(h2_bits(l[0]), h2_bits(l[1]), h2_bits(l[2]), h2_bits(l[3]));
    }
}
template <bool KV8>
__device__ __forceinline__ void widen_item(const raw_item<KV8> & r, int cell, int blk, uint8_t * t_hi, uint8_t * t_lo) {
    if (blk & 1) {  // uniform in a warp
        widen_half<KV8, true>(r, cell, blk, t_hi, t_lo);
    } else {
        widen_half<KV8, false>(r, cell, blk, t_hi, t_lo);
    }
}

// ---- the attention kernel -------------------------------------------------------------------------------------------
// Waits of this kernel: bounded, and once one has run out every other wait of the CTA returns at its next look (the
// CTA then runs to its end on whatever data it has, with FNB_ERR_TIMEOUT set).
__device__ __forceinline__ bool tc_wait(uint64_t * bar, uint32_t parity, volatile uint32_t * gave_up, uint32_t * err) {
    for (uint32_t i = 0; i < kPrimarySpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && *gave_up != 0) return false;
    }
    *gave_up = 1;
    if (err != nullptr) atomicOr(err, FNB_ERR_TIMEOUT);
    return false;
}
// the barrier gets one of its expected arrivals when this thread's asynchronous copies issued so far have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t * bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Roles.  Sixteen worker warps stage, widen and run the softmax; the last warp's first lane issues the MMAs.  Nothing
// in the tile loop is a block-wide barrier: every hand-over is an mbarrier, so warps drift apart by as much as the
// data allows and widening, softmax and tensor work overlap.
//   raw_k[2], raw_v[2]  (512 arrivals)  a stage of the raw ring has landed: each worker's copies arrive on completion
//   k_ready             (512)           every worker has widened its share of a tile's K - on a unit's first tile after
//                                       storing its share of the query operand, on the others after reading the
//                                       previous tile's scores: the issuer starts the tile's score MMAs
//   bar_s               (commit)        the score MMAs are done: S readable, the K operand free and - because k_ready
//                                       needed every worker - its raw stage read by all
//   pv_ready            (512)           every worker has stored its probabilities and widened its share of V
//   bar_o               (commit)        the output MMAs are done: O, P and the V operand are free
// Tile g (counted over the CTA's units) uses stage g & 1 of both rings and phase g of the four tile barriers.  Within a
// unit K runs a tile ahead: tile g + 1's K is widened, and its scores issued, during tile g.
// TMA: the raw tiles are asked for by one thread, one tensor-map copy per tensor and tile (box: 64 cells x one head's
// bytes of a cell), instead of 2 x 1088 16-byte copies issued by the workers, which cost each worker more than widening
// its item: the copies then bypass the load / store unit.  For every shape whose cells lie a multiple of 16 bytes apart
// in the cache (all but Q8_0 at head_dim 128).
template <int HD, bool KV8, bool TMA>
__global__ void __launch_bounds__(kLaunchThreadsTma, 1)
    attend_kernel(const attend_params p, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
    using L = tc_layout<HD, KV8, TMA>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t * k_hi = smem + L::k_hi;
    uint8_t * k_lo = smem + L::k_lo;
    uint8_t * v_hi = smem + L::v_hi;
    uint8_t * v_lo = smem + L::v_lo;
    uint8_t * raw = smem + L::raw;
    float * part_max = reinterpret_cast<float *>(smem + L::part_max);
    uint64_t * bar_s = reinterpret_cast<uint64_t *>(smem + L::bars);
    uint64_t * bar_o = bar_s + 1;
    uint64_t * k_ready = bar_s + 2;   // [2]
    uint64_t * pv_ready = bar_s + 4;  // [2]
    uint64_t * raw_k = bar_s + 6;     // [2]
    uint64_t * raw_v = bar_s + 8;     // [2]
    // Without the copier k_ready and pv_ready are one barrier each, phase g for tile g.  With it they are split by tile
    // parity (tile g on barrier g & 1, phase g >> 1): the copier waits for the tile two back, and a waiter may be one
    // phase behind its barrier, never two.
    const auto kr = [&](uint32_t g) { return k_ready + (TMA ? g & 1u : 0u); };
    const auto pr = [&](uint32_t g) { return pv_ready + (TMA ? g & 1u : 0u); };
    const auto par = [&](uint32_t g) { return TMA ? (g >> 1) & 1u : g & 1u; };
    uint32_t * tmem_slot = reinterpret_cast<uint32_t *>(smem + L::misc);
    volatile uint32_t * gave_up = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const bool worker = wid < kThreads / 32, copier = TMA && wid == kThreads / 32 + 1;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_ready + i, kThreads), mbar_init(pv_ready + i, kThreads);
            // a raw stage hears of every worker's copies, or of the copier's one arrival and its bytes (KV8: and of the
            // 64 threads that copy the cells' scales, 8 bytes each)
            mbar_init(raw_k + i, TMA ? 1 + (KV8 ? kTile : 0) : kThreads), mbar_init(raw_v + i, TMA ? 1 + (KV8 ? kTile : 0) : kThreads);
        }
        *gave_up = 0;
        mbar_init_fence();
    }
    if (wid == 0) tmem_alloc(tmem_slot, L::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem + L::t_s, tmem_o = tmem + L::t_o, tmem_q = tmem + L::t_q, tmem_p = tmem + L::t_p,
                   tmem_alt = tmem + L::t_alt;
    constexpr uint32_t kIdescS = umma_idesc(kTile, false), kIdescO = umma_idesc(HD, true);
    const int total_units = p.n_kv * p.n_units;
    const auto tiles_of = [&](int unit, int & head, int & u, int64_t & c_begin, int64_t & c_end) {
        head = unit / p.n_units, u = unit - head * p.n_units;
        c_begin = p.range_begin + int64_t(u) * p.unit_cells;
        c_end = c_begin + p.unit_cells < p.range_end ? c_begin + p.unit_cells : p.range_end;
        return int((c_end - c_begin + kTile - 1) / kTile);
    };

    if (copier) {
        // ---- the copier: every tile of this CTA in order, tile g's K and V into stage g & 1 of the raw rings, one
        //      tensor-map copy each.  A stage is free when every worker has read it, which is what its tile's k_ready /
        //      pv_ready phase says.  The box is always 64 cells: cells past the unit's end come along (the workers widen
        //      them as zeros), cells past the cache's end are filled with zeros by the copy. ----
        if (lane == 0) {
            uint32_t g = 0;
            for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
                int head, u;
                int64_t c_begin, c_end;
                const int n_tiles = tiles_of(unit, head, u, c_begin, c_end);
                for (int tile = 0; tile < n_tiles; ++tile, ++g) {
                    const int st = g & 1;
                    const int t0 = int(c_begin + int64_t(tile) * kTile);
                    if (g >= 2) tc_wait(kr(g), par(g - 2), gave_up, p.err);
                    mbar_expect_tx(raw_k + st, kTile * L::kCell);
                    if (KV8) {
                        tensor_g2s4(raw + st * L::kRawStage, &map_k, 0, 0, head, t0, raw_k + st);
                    } else {
                        tensor_g2s(raw + st * L::kRawStage, &map_k, 0, head, t0, raw_k + st);
                    }
                    mbar_arrive(raw_k + st);
                    if (g >= 2) tc_wait(pr(g), par(g - 2), gave_up, p.err);
                    mbar_expect_tx(raw_v + st, kTile * L::kCell);
                    if (KV8) {
                        tensor_g2s4(raw + st * L::kRawStage + L::kRawTensor, &map_v, 0, 0, head, t0, raw_v + st);
                    } else {
                        tensor_g2s(raw + st * L::kRawStage + L::kRawTensor, &map_v, 0, head, t0, raw_v + st);
                    }
                    mbar_arrive(raw_v + st);
                }
            }
            // every copy issued has landed before the CTA's shared memory can go to another CTA (at once when the
            // workers ran to the end; after a wait that gave up, this is what keeps the exit safe)
            for (uint32_t back = 1; back <= 2 && back <= g; ++back) {
                const uint32_t gg = g - back;
                mbar_wait_landed(raw_k + (gg & 1), (gg >> 1) & 1);
                mbar_wait_landed(raw_v + (gg & 1), (gg >> 1) & 1);
            }
        }
    } else if (!worker) {
        // ---- the issuer: S = [q_hi; q_lo] . (K_lo + K_hi)^T, the small products first, so that only the sixteen K_hi
        //      steps round a large accumulator; then lane 2 r: p_hi . V_hi only (four roundings of the large
        //      accumulator per tile), lane 2 r + 1: p_lo . V_hi + p_hi . V_lo (small) ----
        if (lane == 0) {
            // the operand tiles never move: their descriptors are made once, and an MMA's is its tile's plus a constant
            // (byte offset / 16 in the address field; no offset here carries out of it)
            const uint64_t d_kh = umma_desc(smem_u32(k_hi), 16, 1024), d_kl = umma_desc(smem_u32(k_lo), 16, 1024);
            const uint64_t d_vh = umma_desc(smem_u32(v_hi), L::kCBlock, 1024), d_vl = umma_desc(smem_u32(v_lo), L::kCBlock, 1024);
            uint32_t g = 0;
            for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
                int head, u;
                int64_t c_begin, c_end;
                const int n_tiles = tiles_of(unit, head, u, c_begin, c_end);
                const auto scores = [&]() {
#pragma unroll
                    for (int kb = 0; kb < L::kBlocks; ++kb) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            umma_f16_ts(tmem_s, tmem_q + 32 * kb + 8 * ks, d_kl + uint64_t((kb * L::kCBlock + 32 * ks) >> 4), kIdescS, (kb | ks) != 0);
                        }
                    }
#pragma unroll
                    for (int kb = 0; kb < L::kBlocks; ++kb) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            umma_f16_ts(tmem_s, tmem_q + 32 * kb + 8 * ks, d_kh + uint64_t((kb * L::kCBlock + 32 * ks) >> 4), kIdescS, 1);
                        }
                    }
                    umma_commit(bar_s);
                };
                // the unit's first scores; then, tile by tile, the NEXT tile's scores before this tile's outputs: the
                // workers widen the next K as soon as they have read this tile's scores, and only then run its softmax
                tc_wait(kr(g), par(g), gave_up, p.err);
                tc_fence_after();
                scores();
                for (int tile = 0; tile < n_tiles; ++tile, ++g) {
                    if (tile + 1 < n_tiles) {
                        tc_wait(kr(g + 1), par(g + 1), gave_up, p.err);
                        tc_fence_after();
                        scores();
                    }
                    tc_wait(pr(g), par(g), gave_up, p.err);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {  // 16 cells a step: two groups of eight 128-byte rows, 8 columns of P
                        umma_f16_ts(tmem_o, tmem_p + 8 * ks, d_vh + uint64_t((2048 * ks) >> 4), kIdescO, (tile | ks) != 0);
                        umma_f16_ts(tmem_o, tmem_alt + 8 * ks, d_vl + uint64_t((2048 * ks) >> 4), kIdescO, 1);
                    }
                    umma_commit(bar_o);
                }
            }
        }
    } else {
        // ---- the workers ----
        // widening: a thread's item is (cell, 32-dim block).  A warp takes eight consecutive cells (the eight lanes of a
        // 16-byte store phase: eight different chunks of the swizzle) times four blocks of one parity (the parity picks
        // the code path, so it is the same in a warp).  The four blocks start 17 words apart in a raw cell and the
        // cells 68 words: the 32 lanes of every raw load then fall on 32 different banks (32 consecutive cells of one
        // block fell on eight).  head_dim 128 has two blocks a parity: a warp takes two groups of eight cells.
        const bool has_item = tid < kTile * (HD / 32);
        constexpr int kPairs = HD / 64, kItemWarps = 2 * (HD / 32);  // block pairs of a cell; warps that hold items
        const int wq = lane >> 3, wparity = wid / (kItemWarps / 2);
        const int cell = 8 * ((wid % (kItemWarps / 2)) * (4 / kPairs) + wq / kPairs) + (lane & 7);
        const int blk = 2 * (wq % kPairs) + wparity;
        // tensor memory: warps w, w + 4, w + 8, w + 12 share quarter w & 3 (lanes 32 (w & 3) ..); a lane pair is one
        // query row (even lane: the hi operand / accumulator row, odd lane: the lo row).  Softmax: each of the
        // quarter's warps takes a quarter of the tile's cells, this thread 8 of the tile's 64 cells of its row.
        const int quarter = wid & 3, col_q = wid >> 2, part = lane & 1;
        const int row = 16 * quarter + (lane >> 1);
        const int col0 = 16 * col_q + 8 * part;  // first cell (of the tile) this thread owns
        const uint32_t lane_base = uint32_t(32 * quarter) << 16;
        // a quarter holds 16 query rows: one with no live row (rows past m) has no softmax to run; its probability
        // lanes are zeroed once per unit and its warps only stage and widen
        const bool quarter_live = 16 * quarter < p.m;

        // a thread's pieces of a raw tile are the same in every tile: (cell of the tile, piece of the cell), for K
        // and for V alike; consecutive threads take consecutive pieces, so a warp's copies cover whole cells
        constexpr int kPiece = L::kCell % 16 == 0 ? 16 : 8;
        constexpr int kPieces = L::kCell / kPiece;
        constexpr int kMine = (kTile * kPieces + kThreads - 1) / kThreads;
        int piece_cell[kMine];      // cell of the tile, or -1: no such piece
        uint32_t piece_src[kMine];  // byte offset from the tile's first cell of this head
        int piece_dst[kMine];       // byte offset in a raw tensor tile
#pragma unroll
        for (int k = 0; k < kMine; ++k) {
            const int i = tid + k * kThreads;
            const int cl = i / kPieces, piece = i - cl * kPieces;
            piece_cell[k] = i < kTile * kPieces ? cl : -1;
            piece_src[k] = uint32_t(cl) * uint32_t(p.n_kv) * L::kCell + kPiece * piece;  // < 64 cells x n_kv x 272
            piece_dst[k] = cl * L::kRawCell + kPiece * piece;
        }

        uint32_t g = 0;
        for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
            int head, u;
            int64_t c_begin, c_end;
            const int n_tiles = tiles_of(unit, head, u, c_begin, c_end);

            // ---- raw tiles of one tensor into stage `st` of its ring; the stage's barrier hears of this thread's
            //      copies when they land ----
            const auto issue = [&](int tile, int st, int tensor) {
                if (TMA && !KV8) return;  // the copier asks for the tiles; KV8: for the cells, the scales are copied here
                uint8_t * base = raw + st * L::kRawStage + tensor * L::kRawTensor;
                const uint8_t * cache = tensor == 0 ? p.k_cache : p.v_cache;
                const int64_t t0 = c_begin + int64_t(tile) * kTile;
                const int64_t head_at = (t0 * p.n_kv + head) * L::kCell;
                if (!TMA) {
#pragma unroll
                    for (int k = 0; k < kMine; ++k) {
                        if (piece_cell[k] >= 0) {
                            const bool valid = t0 + piece_cell[k] < c_end;
                            const uint8_t * src = cache + (valid ? head_at + piece_src[k] : 0);
                            if (kPiece == 16) {
                                cp_async16(base + piece_dst[k], src, valid);
                            } else {
                                cp_async8(base + piece_dst[k], src, valid);
                            }
                        }
                    }
                }
                if (KV8 && tid < kTile) {
                    const int64_t c = t0 + tid;
                    const bool valid = c < c_end;
                    const uint16_t * src = (tensor == 0 ? p.k_scale : p.v_scale) + ((valid ? c : c_begin) * p.n_kv + head) * (HD / 64);
                    uint8_t * dst = base + kTile * L::kRawCell + tid * 8;
                    if (HD == 256) {
                        cp_async8(dst, src, valid);
                    } else {  // two scales a cell
                        cp_async4(dst, src, valid);
                    }
                }
                if (!TMA || tid < kTile) cp_async_arrive((tensor == 0 ? raw_k : raw_v) + st);
            };
            // this thread's item of a staged tensor, widened into the operand tiles
            const auto widen = [&](int tile, int st, int tensor, uint8_t * t_hi, uint8_t * t_lo) {
                if (has_item) {
                    const uint8_t * t = raw + st * L::kRawStage + tensor * L::kRawTensor;
                    raw_item<KV8> r;
                    load_item<HD, KV8, L::kSwizzled>(r, t + cell * L::kRawCell, t + kTile * L::kRawCell + cell * 8, blk, cell);
                    if (TMA && c_begin + int64_t(tile) * kTile + cell >= c_end) {  // the box brought a cell past the unit's end
#pragma unroll
                        for (int j = 0; j < (KV8 ? 8 : 9); ++j) r.w[j] = 0u;
                        r.scale = 0u;
                    }
                    widen_item<KV8>(r, cell, blk, t_hi, t_lo);
                }
            };

            // ---- this thread's row: its live cells [lo, hi) within the unit, an empty range for rows past m ----
            int64_t r_lo = 0, r_hi = 0;
            if (row < p.m) {
                const int t = row / p.n_rep;
                r_lo = p.first_cell != nullptr ? int64_t(__ldg(p.first_cell + t)) : p.range_begin;
                r_hi = p.n_cells != nullptr ? r_lo + int64_t(__ldg(p.n_cells + t)) : p.range_end;
                if (r_lo < 0 || r_hi > p.cache_slots || r_hi < r_lo) {
                    if (p.err != nullptr && col_q == 0 && part == 0) atomicOr(p.err, FNB_ERR_SLOT);
                    r_lo = r_hi = 0;
                }
                r_lo = r_lo < c_begin ? c_begin : r_lo;
                r_hi = r_hi > c_end ? c_end : r_hi;
            }

            // ---- the unit's first tile on its way (both stages are free: the previous unit's last tile was waited
            //      for by every worker before its partial result) ----
            issue(0, g & 1, 0);
            issue(0, g & 1, 1);
            if (n_tiles > 1) issue(1, (g & 1) ^ 1, 0);

            // ---- the group's query rows into tensor memory: lane 2 r the hi part of row r, lane 2 r + 1 the rounded
            //      residual, rows past m zero; this warp the 64 dims of its column quarter (the previous unit's score
            //      MMAs are done) ----
            if (col_q < HD / 64) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {  // 32 dims = 16 columns at a time
                    float w[16];
                    if (row < p.m) {
                        const int t = row / p.n_rep, rr = row - t * p.n_rep;
                        const float4 * src = reinterpret_cast<const float4 *>(p.q + (int64_t(t) * p.n_q + head * p.n_rep + rr) * HD +
                                                                              64 * col_q + 32 * h);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 x = __ldg(src + j);
                            const __half2 a = __floats2half2_rn(x.x, x.y), b = __floats2half2_rn(x.z, x.w);
                            if (part) {
                                const float2 fa = __half22float2(a), fb = __half22float2(b);
                                w[2 * j] = __uint_as_float(h2_bits(__floats2half2_rn(x.x - fa.x, x.y - fa.y)));
                                w[2 * j + 1] = __uint_as_float(h2_bits(__floats2half2_rn(x.z - fb.x, x.w - fb.y)));
                            } else {
                                w[2 * j] = __uint_as_float(h2_bits(a)), w[2 * j + 1] = __uint_as_float(h2_bits(b));
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) w[j] = 0.0f;
                    }
                    tmem_st16(tmem_q + lane_base + uint32_t(32 * col_q + 16 * h), w);
                }
                tmem_wait_st();
            }
            if (!quarter_live) {  // the previous unit's output MMAs, the last readers of P, were waited for
                float z[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                tmem_st8(tmem_p + lane_base + uint32_t(8 * col_q), z);
                tmem_st8(tmem_alt + lane_base + uint32_t(8 * col_q), z);
                tmem_wait_st();
            }

            // the reference point (the same in the row's eight threads) and the sum over this thread's cells
            float m_ref = -INFINITY, l_run = 0.0f;

            // ---- K of the unit's first tile (the operand is free: the previous unit's last scores were read by all) ----
            tc_wait(raw_k + (g & 1), (g >> 1) & 1, gave_up, p.err);
            widen(0, g & 1, 0, k_hi, k_lo);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(kr(g));

            for (int tile = 0; tile < n_tiles; ++tile, ++g) {
                const int st = g & 1;
                float * pm = part_max + st * (4 * kMaxM);  // by tile parity: a warp a tile ahead writes the other half
                // ---- the tile's scores into registers: every thread 8 cells of one query row ----
                tc_wait(bar_s, g & 1, gave_up, p.err);
                tc_fence_after();
                float s[8];
                if (quarter_live) {
                    float mine[16];
                    tmem_ld16(tmem_s + lane_base + 16 * col_q, mine);
                    // the pair's other lane holds the row's other part: keep my 8 cells, hand over the other 8
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float keep = part ? mine[8 + j] : mine[j], give = part ? mine[j] : mine[8 + j];
                        s[j] = keep + __shfl_xor_sync(kFull, give, 1);
                    }
                }
                // ---- K of the NEXT tile: the operand is free (this tile's scores are done) and S has been read, so the
                //      next scores can run under this tile's softmax.  The raw K after that takes this tile's stage,
                //      which every worker read before the scores just waited for could be issued ----
                if (tile + 1 < n_tiles) {
                    tc_wait(raw_k + (st ^ 1), ((g + 1) >> 1) & 1, gave_up, p.err);
                    if (tile + 2 < n_tiles) issue(tile + 2, st, 0);
                    widen(tile + 1, st ^ 1, 0, k_hi, k_lo);
                    fence_proxy_async();
                    tc_fence_before();
                    mbar_arrive(kr(g + 1));
                }
                float a_row = 1.0f;
                if (quarter_live) {
                const int64_t c0 = c_begin + int64_t(tile) * kTile + col0;
                const int lo = int(r_lo - c0), hi = int(r_hi - c0);  // this thread's live cells: lo <= j < hi
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    s[j] = j >= lo && j < hi ? s[j] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, s[j]);
                }
                mx = fmaxf(mx, __shfl_xor_sync(kFull, mx, 1));
                if (part == 0) pm[col_q * kMaxM + row] = mx;
                named_barrier_id(2 + quarter, 128);  // the four warps of this quarter
                mx = fmaxf(fmaxf(pm[row], pm[kMaxM + row]), fmaxf(pm[2 * kMaxM + row], pm[3 * kMaxM + row]));
                // lazy reference point: it moves only when the row's maximum has outgrown it by more than 2^kLazy
                if (mx > m_ref + kLazy || (m_ref == -INFINITY && mx > -INFINITY)) {
                    if (m_ref != -INFINITY) a_row = fast_exp2(m_ref - mx);
                    m_ref = mx;
                }
                }
                // ---- the previous tile's output MMAs: after them O may be rescaled, P overwritten and the V operand
                //      refilled ----
                if (g > 0) {
                    tc_wait(bar_o, (g - 1) & 1, gave_up, p.err);
                    tc_fence_after();
                }
                if (quarter_live) {
                if (__any_sync(kFull, a_row != 1.0f)) {  // this warp's quarter of the output columns of its lanes' rows
#pragma unroll 1
                    for (int cb = 0; cb < HD / 128; ++cb) {
                        float o[32];
                        const uint32_t at = tmem_o + lane_base + uint32_t(HD / 4 * col_q + 32 * cb);
                        tmem_ld32(at, o);
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] *= a_row;
                        tmem_st32(at, o);
                    }
                }
                {
                    // probabilities of this thread's 8 cells as four words each of hi and lo parts (x 2^12)
                    const float ref = m_ref == -INFINITY ? 0.0f : m_ref;
                    float sum = 0.0f;
                    uint32_t hi4[4], lo4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float p0 = fast_exp2(s[2 * e] - ref), p1 = fast_exp2(s[2 * e + 1] - ref);
                        sum += p0 + p1;
                        const float x0 = p0 * kPScale, x1 = p1 * kPScale;
                        const __half2 hv = __floats2half2_rn(x0, x1);
                        const float2 back = __half22float2(hv);
                        hi4[e] = h2_bits(hv);
                        lo4[e] = h2_bits(__floats2half2_rn(x0 - back.x, x1 - back.y));
                    }
                    l_run = l_run * a_row + sum;
                    // The warp's 16 cells of a row are 8 columns of the row's two operand lanes.  Even lane (the hi lane,
                    // owner of the first 8 cells): P = hi of all 16, alternate P = zeros.  Odd lane (the lo lane, owner
                    // of the last 8): P = lo of all 16, alternate P = hi of all 16.
                    float w_op[8], w_alt[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t other_hi = __shfl_xor_sync(kFull, hi4[e], 1), other_lo = __shfl_xor_sync(kFull, lo4[e], 1);
                        w_op[e] = __uint_as_float(part ? other_lo : hi4[e]);
                        w_op[4 + e] = __uint_as_float(part ? lo4[e] : other_hi);
                        w_alt[e] = __uint_as_float(part ? other_hi : 0u);
                        w_alt[4 + e] = __uint_as_float(part ? hi4[e] : 0u);
                    }
                    tmem_st8(tmem_p + lane_base + uint32_t(8 * col_q), w_op);
                    tmem_st8(tmem_alt + lane_base + uint32_t(8 * col_q), w_alt);
                    tmem_wait_st();
                }
                }
                // ---- V of the tile; the next tile's raw V takes the stage of tile g - 1's, which every worker read
                //      before the output MMAs just waited for could be issued ----
                tc_wait(raw_v + st, (g >> 1) & 1, gave_up, p.err);
                if (tile + 1 < n_tiles) issue(tile + 1, st ^ 1, 1);
                widen(tile, st, 1, v_hi, v_lo);
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(pr(g));
            }

            // ---- the unit's partial result: (reference point, sum, (O[2 r] + O[2 r + 1]) / 2^12) of its rows ----
            tc_wait(bar_o, (g - 1) & 1, gave_up, p.err);
            tc_fence_after();
            if (quarter_live) {
            const int64_t slot = int64_t(head) * p.n_units + u;
            float * ml = p.ws_ml + slot * p.m * 2;
            float * acc = p.ws_acc + slot * p.m * HD;
            // the row's sum: its eight threads' shares (two lanes in each of the quarter's four warps)
            const float l_pair = l_run + __shfl_xor_sync(kFull, l_run, 1);
            float * pm = part_max + (g & 1) * (4 * kMaxM);
            if (part == 0) pm[col_q * kMaxM + row] = l_pair;
            named_barrier_id(2 + quarter, 128);
            if (col_q == 0 && part == 0 && row < p.m) {
                ml[2 * row] = m_ref;
                ml[2 * row + 1] = (pm[row] + pm[kMaxM + row]) + (pm[2 * kMaxM + row] + pm[3 * kMaxM + row]);
            }
#pragma unroll 1
            for (int cb = 0; cb < HD / 128; ++cb) {
                float o[32];
                const int col = HD / 4 * col_q + 32 * cb;
                tmem_ld32(tmem_o + lane_base + uint32_t(col), o);
#pragma unroll
                for (int j = 0; j < 32; ++j) o[j] += __shfl_xor_sync(kFull, o[j], 1);
                // the pair's even lane writes the first 16 columns, the odd lane the other 16
                if (row < p.m) {
                    float4 * dst = reinterpret_cast<float4 *>(acc + int64_t(row) * HD + col + 16 * part);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int b = 4 * j;
                        dst[j] = part ? make_float4(o[16 + b] * kPUnscale, o[17 + b] * kPUnscale, o[18 + b] * kPUnscale, o[19 + b] * kPUnscale)
                                      : make_float4(o[b] * kPUnscale, o[b + 1] * kPUnscale, o[b + 2] * kPUnscale, o[b + 3] * kPUnscale);
                    }
                }
            }
            }
            // the sums in part_max are read before any warp of the quarter can write a maximum there: that write
            // follows the next tile's scores, which need this warp's arrival on k_ready
            tc_fence_before();
        }
    }
    __syncthreads();
    if (wid == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, L::kTmemCols);
    }
}

// ---- the fold: one CTA a (row, query head), one thread a value ------------------------------------------------------
// M = max m_j, L = sum l_j 2^(m_j - M), A = sum acc_j 2^(m_j - M) over the row's partials j in slot order.  The weights
// are formed once per CTA in shared memory (slots in parallel), then every thread streams its column of the partials
// with independent loads.
constexpr int kFoldMaxSlots = 4096;
constexpr int kFoldLanes = 4;  // threads a value: each streams every fourth partial

template <int HD>
__global__ void __launch_bounds__(HD * kFoldLanes) attend_fold_kernel(const attend_params p) {
    __shared__ float w_of[kFoldMaxSlots];
    __shared__ float red[HD * kFoldLanes / 32];
    __shared__ float part_a[kFoldLanes][HD];
    const int t = blockIdx.x / p.n_q, h = blockIdx.x - t * p.n_q;
    const int head = h / p.n_rep, row = t * p.n_rep + (h - head * p.n_rep);
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int d = tid % HD, q = tid / HD;
    constexpr int kThreadsF = HD * kFoldLanes, kWarpsF = kThreadsF / 32;
    const int n = p.n_units * p.parts;
    const int64_t slot0 = int64_t(head) * n;
    float big = -INFINITY;
    for (int j = tid; j < n; j += kThreadsF) {
        const float mj = __ldg(p.ws_ml + ((slot0 + j) * p.m + row) * 2);
        w_of[j] = mj;
        big = fmaxf(big, mj);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(kFull, big, o));
    if (lane == 0) red[wid] = big;
    __syncthreads();
    big = red[0];
#pragma unroll
    for (int i = 1; i < kWarpsF; ++i) big = fmaxf(big, red[i]);
    __syncthreads();
    // weights (0 for a partial with no live cell for this row, and for every partial of a row with none at all)
    float part_sum = 0.0f;
    for (int j = tid; j < n; j += kThreadsF) {
        const float mj = w_of[j];
        const float w = mj == -INFINITY ? 0.0f : fast_exp2(mj - big);
        w_of[j] = w;
        part_sum = fmaf(__ldg(p.ws_ml + ((slot0 + j) * p.m + row) * 2 + 1), w, part_sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part_sum += __shfl_xor_sync(kFull, part_sum, o);
    if (lane == 0) red[wid] = part_sum;
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kWarpsF; ++i) sum += red[i];
    float a = 0.0f;
    const float * col = p.ws_acc + (slot0 * p.m + row) * HD + d;
    const int64_t stride = int64_t(p.m) * HD;
#pragma unroll 8
    for (int j = q; j < n; j += kFoldLanes) a = fmaf(__ldg(col + j * stride), w_of[j], a);
    part_a[q][d] = a;
    __syncthreads();
    if (q != 0) return;
    a = (part_a[0][d] + part_a[1][d]) + (part_a[2][d] + part_a[3][d]);
    float y = sum > 0.0f ? a / sum : 0.0f;  // a row with no cell at all gives zeros
    const int64_t at = (int64_t(t) * p.n_q + h) * HD + d;
    if (p.gate != nullptr) y *= 1.0f / (1.0f + expf(-__ldg(p.gate + at)));
    p.out[at] = y;
}

template <int HD, bool KV8, bool TMA>
bool configure() {
    static std::atomic<bool> done[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!done[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(attend_kernel<HD, KV8, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tc_layout<HD, KV8, TMA>::total) != cudaSuccess) {
            return false;
        }
        done[dev].store(true, std::memory_order_release);
    }
    return true;
}

// The tensor map of one cache tensor as the copier reads it: [cache_slots][n_kv][cell bytes] seen as 16-bit elements, a
// box of 64 cells x one head x the whole cell.  Encoded on the host by the driver's cuTensorMapEncodeTiled, looked up
// once through the runtime (no link against the driver library); false when the driver does not offer it or refuses
// the shape, and the caller then launches the kernel whose workers copy the cells themselves.
using encode_tiled_fn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                     const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline encode_tiled_fn encode_tiled() {
    static const encode_tiled_fn fn = [] {
        void * f = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            (void) cudaGetLastError();
            return encode_tiled_fn(nullptr);
        }
        return reinterpret_cast<encode_tiled_fn>(f);
    }();
    return fn;
}
// Q8_0 (swizzled = false): three dimensions, [slots][heads][cell as u16], the box one head's whole cell of 64 slots, laid
// out densely.  KV8 (swizzled = true): a cell is one or two rows of 128 bytes, four dimensions [slots][heads][rows][64 x
// u16], the box 64 slots x one head x its rows, with the 128-byte swizzle.
inline bool make_cell_map(CUtensorMap * map, const uint8_t * cache, int64_t cache_slots, int n_kv, int cell_bytes, bool swizzled) {
    const encode_tiled_fn enc = encode_tiled();
    if (enc == nullptr || cell_bytes % 16 != 0) return false;
    const cuuint32_t elem[4] = {1u, 1u, 1u, 1u};
    if (swizzled) {
        if (cell_bytes % 128 != 0) return false;
        const cuuint64_t dims[4] = {64u, cuuint64_t(cell_bytes / 128), cuuint64_t(n_kv), cuuint64_t(cache_slots)};
        const cuuint64_t strides[3] = {128u, cuuint64_t(cell_bytes), cuuint64_t(n_kv) * cuuint64_t(cell_bytes)};
        const cuuint32_t box[4] = {64u, cuuint32_t(cell_bytes / 128), 1u, cuuint32_t(kTile)};
        return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<uint8_t *>(cache), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (cell_bytes / 2 > 256) return false;
    const cuuint64_t dims[3] = {cuuint64_t(cell_bytes / 2), cuuint64_t(n_kv), cuuint64_t(cache_slots)};
    const cuuint64_t strides[2] = {cuuint64_t(cell_bytes), cuuint64_t(n_kv) * cuuint64_t(cell_bytes)};  // bytes, from the second dimension on
    const cuuint32_t box[3] = {cuuint32_t(cell_bytes / 2), 1u, cuuint32_t(kTile)};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<uint8_t *>(cache), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int HD, bool KV8>
int32_t launch_hd(const attend_params & p, cudaStream_t s) {
    const int units = p.n_kv * p.n_units;
    const int grid = units < kSmCount ? units : kSmCount;
    CUtensorMap map_k = {}, map_v = {};
    // the tensor-map copies want a cell's stride in the cache a multiple of 16 bytes: every shape but Q8_0 at head_dim 128
    constexpr int kCell = tc_layout<HD, KV8, false>::kCell;
    constexpr bool kTmaShape = kCell % 16 == 0;
    if (kTmaShape && make_cell_map(&map_k, p.k_cache, p.cache_slots, p.n_kv, kCell, KV8) &&
        make_cell_map(&map_v, p.v_cache, p.cache_slots, p.n_kv, kCell, KV8)) {
        if (!configure<HD, KV8, kTmaShape>()) return FNB_LAUNCH_FAILED;
        attend_kernel<HD, KV8, kTmaShape><<<grid, kLaunchThreadsTma, tc_layout<HD, KV8, kTmaShape>::total, s>>>(p, map_k, map_v);
    } else {
        if (!configure<HD, KV8, false>()) return FNB_LAUNCH_FAILED;
        attend_kernel<HD, KV8, false><<<grid, kLaunchThreads, tc_layout<HD, KV8, false>::total, s>>>(p, map_k, map_v);
    }
    if (cudaPeekAtLastError() != cudaSuccess) return FNB_LAUNCH_FAILED;
    attend_fold_kernel<HD><<<p.rows * p.n_q, HD * kFoldLanes, 0, s>>>(p);
    return launch_status();
}

bool shape_ok(const fnb_attend_args * a) {
    if (a == nullptr) return false;
    if (a->head_dim != 128 && a->head_dim != 256) return false;
    if (a->rows < 1 || a->n_q_heads < 1 || a->n_kv_heads < 1 || a->n_kv_heads > 1024 || a->n_q_heads % a->n_kv_heads != 0) return false;
    if (int64_t(a->rows) * (a->n_q_heads / a->n_kv_heads) > kMaxM) return false;
    if (a->cache_slots < 1 || a->cache_slots > INT32_MAX) return false;
    if (a->range_begin < 0 || a->range_end <= a->range_begin || a->range_end > a->cache_slots) return false;
    return true;
}

}  // namespace

bool attend_prepare_device() {
    (void) encode_tiled();
    return configure<256, false, false>() && configure<256, false, true>() && configure<256, true, false>() &&
           configure<256, true, true>() && configure<128, false, false>() && configure<128, true, false>() &&
           configure<128, true, true>();
}

// shared by the two entry points: everything but where the workspace lives
int32_t attend_launch(const fnb_attend_args * a, void * ws, size_t ws_bytes, cudaStream_t s) {
    if (!shape_ok(a)) return FNB_REJECTED;
    const bool kv8 = a->k_scale != nullptr || a->v_scale != nullptr;
    if (kv8 && (!ok_ptr(a->k_scale, 8) || !ok_ptr(a->v_scale, 8))) return FNB_REJECTED;
    if (!ok_ptr(a->q, 16) || !ok_opt(a->gate, 16) || !ok_ptr(a->out, 16) || !ok_ptr(a->k_cache, 16) || !ok_ptr(a->v_cache, 16)) {
        return FNB_REJECTED;
    }
    if (!ok_opt(a->first_cell, 4) || !ok_opt(a->n_cells, 4) || !ok_opt(a->err, 4)) return FNB_REJECTED;
    if (!(a->scale > 0.0f) || !(a->scale < INFINITY)) return FNB_REJECTED;
    const attend_plan plan = make_plan(a->rows, a->n_q_heads, a->n_kv_heads, a->range_end - a->range_begin);
    if (plan.n_units * plan.parts > kFoldMaxSlots) return FNB_REJECTED;  // cannot happen with the plan's one unit an SM
    if (!ok_ptr(ws, 16) || ws_bytes < plan_bytes(plan, a->head_dim)) return FNB_REJECTED;

    attend_params p;
    p.q = a->q, p.gate = a->gate;
    p.k_cache = static_cast<const uint8_t *>(a->k_cache), p.v_cache = static_cast<const uint8_t *>(a->v_cache);
    p.k_scale = a->k_scale, p.v_scale = a->v_scale, p.first_cell = a->first_cell, p.n_cells = a->n_cells;
    p.out = a->out, p.err = a->err;
    p.ws_ml = static_cast<float *>(ws);
    p.ws_acc = p.ws_ml + plan_ml_floats(plan);
    p.cache_slots = a->cache_slots, p.range_begin = a->range_begin, p.range_end = a->range_end, p.unit_cells = plan.unit_cells;
    p.rows = a->rows, p.n_q = a->n_q_heads, p.n_kv = a->n_kv_heads, p.n_rep = a->n_q_heads / a->n_kv_heads;
    p.m = plan.m, p.parts = plan.parts, p.n_units = plan.n_units;
    p.scale_log2 = a->scale * kLog2e;
    if (a->head_dim == 256) return kv8 ? launch_hd<256, true>(p, s) : launch_hd<256, false>(p, s);
    return kv8 ? launch_hd<128, true>(p, s) : launch_hd<128, false>(p, s);
}

size_t attend_workspace_bytes(const fnb_attend_args * a) {
    if (!shape_ok(a)) return 0;
    return plan_bytes(make_plan(a->rows, a->n_q_heads, a->n_kv_heads, a->range_end - a->range_begin), a->head_dim);
}

}  // namespace fnb

// ---- the same attention for callers with no workspace to give ----------------------------------------------------------
// Some callers cannot hand in a workspace and cannot get one: an engine that reserves all of its device memory once at
// load and has nothing left to carve from, a plug-in whose host forbids device allocation on the serving path (an
// allocation synchronises the whole device and can fail long after start-up).  For them the partial results live in
// this fixed array, part of the library's image: every GPU that loads the library holds these bytes until the process
// ends, whether or not this entry point is ever called.
#define FNB_ATTEND_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_attend_scratch[FNB_ATTEND_STATIC_SCRATCH_BYTES];

namespace fnb {
namespace {

// The array's name is only a host-side handle here: its device address has to be asked for, once per device, with
// that device current.  nullptr when the runtime refuses.
void * attend_static_scratch() {
    static std::atomic<void *> addr_of[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    void * p = addr_of[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (cudaGetSymbolAddress(&p, g_attend_scratch) != cudaSuccess || p == nullptr) {
            (void) cudaGetLastError();
            return nullptr;
        }
        addr_of[dev].store(p, std::memory_order_release);
    }
    return p;
}

}  // namespace
}  // namespace fnb

extern "C" size_t fnb_attend_workspace_bytes(const fnb_attend_args * args) { return fnb::attend_workspace_bytes(args); }

extern "C" int32_t fnb_attend_static(const fnb_attend_args * args, void * stream) {
    if (args == nullptr) return FNB_REJECTED;
    const size_t need = fnb::attend_workspace_bytes(args);
    if (need == 0) return FNB_REJECTED;
    if (need > size_t(FNB_ATTEND_STATIC_SCRATCH_BYTES)) {
        fprintf(stderr, "fnb_attend_static: this shape needs %zu bytes of partial results, the built-in scratch holds %u; "
                        "use fnb_attend with a workspace\n", need, unsigned(FNB_ATTEND_STATIC_SCRATCH_BYTES));
        return FNB_REJECTED;
    }
    void * scratch = fnb::attend_static_scratch();
    if (scratch == nullptr) return FNB_LAUNCH_FAILED;
    return fnb::attend_launch(args, scratch, size_t(FNB_ATTEND_STATIC_SCRATCH_BYTES), static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_attend(const fnb_attend_args * args, void * stream) {
    if (args == nullptr) return FNB_REJECTED;
    return fnb::attend_launch(args, args->workspace, args->workspace_bytes, static_cast<cudaStream_t>(stream));
}
