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
// head's group; the work per byte is a contraction (M = rows x heads per group query rows against every cell), so the
// products run on the tensor pipe and everything else is shaped around feeding it:
//
//   * Split precision.  The 1e-5 bound needs products far more exact than 11-bit operands give, so every F32 operand
//     becomes two FP16 operands (value = hi + lo, about 22 bits):  q = q_hi + q_lo;  K stays the INTEGER codes (exact in
//     FP16) and each 32-dim block's partial dot product is multiplied by the block's scale in F32 afterwards, so
//     q . K costs two tensor products, not three;  V = d x code is split exactly (hi = the rounded product, lo = the
//     fused residual, both one half2 instruction per two values) and p = p_hi + p_lo (scaled by 2^12 to stay clear of
//     FP16's subnormals), so p . V costs three (the lo x lo term is below 2^-22).
//   * A PAIR of warps owns 16 query rows (an m16n8k16 tile row): both form the rows' scores and softmax statistics (the
//     same instructions on the same data, so the same bits), and each accumulates one half of the head_dim output
//     columns, so that running maximum, sum and output accumulators never leave registers and eight warps (two per
//     scheduler) hide each other's latencies.  A CTA's four pairs take up to four such row tiles; with one or two row
//     tiles the pairs split the CTA's 64-cell tile four or two ways instead, each part an independent partial result,
//     so that all four tensor cores work whatever the number of rows.  A warp walks its cells in steps of 16 (two
//     score tiles, one step of the output product), with the online-softmax update per step.
//   * Cells arrive by 16-byte cp.async into a two-stage ring of raw tiles (the next tile's copies are in flight while
//     this one is computed); all 128 threads widen a raw tile into the operand tiles (XOR-swizzled rows, so that
//     ldmatrix is conflict-free), K first, then V into the same shared memory once the scores are done.
//   * Split over cells (flash decoding): a work unit is (KV head, range of cells); units and tile parts write
//     (max, sum, unnormalised output) partials into a caller-supplied workspace, and a second small kernel folds them
//     in a fixed order, divides, gates and writes the rows.  The workspace is the only global memory beyond inputs and
//     outputs; its size is a function of the shape (fnb_attend_workspace_bytes).
//
// No kernel here waits on another: the fold is a second launch on the same stream.
#include <atomic>
#include <cstdio>

#include <cuda_fp16.h>

#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarps = 8;  // four score / step owners x two halves of the output columns
constexpr int kThreads = kWarps * 32;
constexpr int kStep = 16;  // cells of one step of a warp: two 8-cell score tiles, one k-step of the output product
constexpr int kTile = 64;  // cells a CTA stages at once: four steps
constexpr int kMaxM = 64;  // query rows of one KV head's group: rows x (n_q_heads / n_kv_heads)
constexpr float kPScale = 4096.0f, kPUnscale = 1.0f / 4096.0f;
constexpr float kLog2e = 1.4426950408889634f;

struct attend_plan {
    int m, m_tiles, parts;   // query rows per group, their 16-row tiles, partial results a unit writes (1, 2 or 4)
    int64_t unit_cells;      // cells per work unit (a multiple of kTile)
    int n_units;             // units per KV head
    int64_t slots;           // partial results in the workspace: n_kv x n_units x parts
};

// the split the launcher and the workspace size agree on: about two units per SM over all KV heads, never shorter
// than 256 cells
inline attend_plan make_plan(int rows, int n_q, int n_kv, int64_t range) {
    attend_plan p;
    p.m = rows * (n_q / n_kv);
    p.m_tiles = (p.m + 15) / 16;
    p.parts = p.m_tiles == 1 ? 4 : p.m_tiles == 2 ? 2 : 1;
    int64_t want = (2 * int64_t(kSmCount) + n_kv - 1) / n_kv;
    int64_t cells = (range + want - 1) / want;
    cells = cells < 256 ? 256 : cells;
    p.unit_cells = (cells + kTile - 1) / kTile * kTile;
    p.n_units = int((range + p.unit_cells - 1) / p.unit_cells);
    if (p.n_units < 1) p.n_units = 1;
    p.slots = int64_t(n_kv) * p.n_units * p.parts;
    return p;
}
inline size_t plan_bytes(const attend_plan & p, int head_dim) { return size_t(p.slots) * p.m * (head_dim + 2) * 4; }

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
    float * ws_ml;   // [slots][m][2]: running maximum (in log2 units) and sum
    float * ws_acc;  // [slots][m][head_dim]
    uint32_t * err;
    int64_t cache_slots, range_begin, range_end, unit_cells;
    int rows, n_q, n_kv, n_rep, m, m_tiles, parts, n_units;
    float scale_log2;  // softmax scale x log2(e)
};

// ---- small PTX wrappers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s_addr(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// d += a (16 x 16, row) x b (16 x 8, col), FP16 operands, F32 accumulators
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 (or 8) bytes global -> shared; src_bytes = 0 writes zeros instead (cells past the end of a range)
__device__ __forceinline__ void cp_async16(void * dst, const void * src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s_addr(dst)), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async8(void * dst, const void * src, bool valid) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(s_addr(dst)), "l"(src), "r"(valid ? 8 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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

// operand tiles: rows of ROW_BYTES bytes (a power of two >= 128), 16-byte chunks XOR-swizzled by the row's low three bits
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return uint32_t(row) * ROW_BYTES + (uint32_t(chunk ^ (row & 7)) << 4);
}

// One pair of Q8_0 blocks of a cell (68 bytes = 17 aligned words x: d0 | 32 codes | d1 | 32 codes) widened into the
// operand tile(s): 64 values = eight 16-byte chunks.  The four threads of a cell (pair index pr = 0 .. 3) run the same
// instructions: a warp's raw loads fall on 32 different banks (word 68 cell + 17 pr + j), and its 16-byte stores, 512
// bytes an instruction, take the four wavefronts that much data needs whatever the order.
//   V = false: the codes as FP16 integers (the K operand).  V = true: hi = rn(d x code) and lo = fma(d, code, -hi).
template <bool V, int ROW_BYTES>
__device__ __forceinline__ void widen_pair(const uint32_t (&x)[17], int cell, int pr, uint8_t * t_hi, uint8_t * t_lo) {
    const __half d_first = __ushort_as_half(uint16_t(x[0] & 0xffffu)), d_second = __ushort_as_half(uint16_t(x[8] >> 16));
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
        uint32_t c0, c1;
        if (jj < 4) {
            c0 = __funnelshift_r(x[2 * jj], x[2 * jj + 1], 16), c1 = __funnelshift_r(x[2 * jj + 1], x[2 * jj + 2], 16);
        } else {
            c0 = x[2 * jj + 1], c1 = x[2 * jj + 2];
        }
        __half2 c[4];
        codes_to_h2(c0, c[0], c[1]);
        codes_to_h2(c1, c[2], c[3]);
        const uint32_t at = swz<ROW_BYTES>(cell, 8 * pr + jj);
        if (!V) {
            *reinterpret_cast<uint4 *>(t_hi + at) = make_uint4(h2_bits(c[0]), h2_bits(c[1]), h2_bits(c[2]), h2_bits(c[3]));
        } else {
            const __half2 d2 = __half2half2(jj < 4 ? d_first : d_second);
            __half2 h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                h[e] = __hmul2(d2, c[e]);
                l[e] = __hfma2(d2, c[e], __hneg2(h[e]));
            }
            *reinterpret_cast<uint4 *>(t_hi + at) = make_uint4(h2_bits(h[0]), h2_bits(h[1]), h2_bits(h[2]), h2_bits(h[3]));
            *reinterpret_cast<uint4 *>(t_lo + at) = make_uint4(h2_bits(l[0]), h2_bits(l[1]), h2_bits(l[2]), h2_bits(l[3]));
        }
    }
}
template <bool V, int ROW_BYTES>
__device__ __forceinline__ void widen_q8_0_tile(const uint8_t * raw, int cell_bytes, int pairs, uint8_t * t_hi, uint8_t * t_lo, int tid) {
    for (int i = tid; i < kTile * pairs; i += kThreads) {
        const int cell = i / pairs, pr = i - cell * pairs;
        const uint32_t * w = reinterpret_cast<const uint32_t *>(raw + cell * cell_bytes + 68 * pr);
        uint32_t x[17];
#pragma unroll
        for (int j = 0; j < 17; ++j) x[j] = w[j];
        widen_pair<V, ROW_BYTES>(x, cell, pr, t_hi, t_lo);
    }
}

// ---- shared memory layout -------------------------------------------------------------------------------------------
template <int HD, bool KV8>
struct smem_layout {
    static constexpr int kRow = HD * 2;                                 // bytes of an FP16 row
    static constexpr int kCell = KV8 ? HD : HD / 32 * 34;                // raw bytes of a cell
    static constexpr int kScale = KV8 ? HD / 64 * 2 : 0;                 // raw bytes of a cell's KV8 scales
    static constexpr int kRawTensor = kTile * kCell + kTile * (KV8 ? 8 : 0);  // one tensor's raw tile (scales in 8-byte slots)
    static constexpr int q_hi = 0;
    static constexpr int q_lo = q_hi + kMaxM * kRow;
    static constexpr int op = q_lo + kMaxM * kRow;                      // K codes as FP16 [64][HD], or V hi | V lo [64][HD] each
    static constexpr int raw = op + 2 * kTile * kRow;                   // [2 stages][K raw | V raw]
    static constexpr int ranges = raw + 2 * 2 * kRawTensor;             // int32 lo[kMaxM], hi[kMaxM]
    static constexpr int total = ranges + 2 * kMaxM * 4;
};

// ---- the attention kernel -------------------------------------------------------------------------------------------
template <int HD, bool KV8>
__global__ void __launch_bounds__(kThreads, 1) attend_kernel(const attend_params p) {
    using L = smem_layout<HD, KV8>;
    constexpr int NB = HD / 32;      // 32-dim blocks
    constexpr int NT = HD / 16;      // 8-dim output tiles of this warp's half of the columns
    constexpr int kHalfChunks = HD / 16;  // 16-byte chunks (8 FP16 values) in half a row
    constexpr int kRow = L::kRow;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * q_hi = smem + L::q_hi;
    uint8_t * q_lo = smem + L::q_lo;
    uint8_t * op = smem + L::op;
    int32_t * row_lo = reinterpret_cast<int32_t *>(smem + L::ranges);
    int32_t * row_hi = row_lo + kMaxM;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    // this warp's row tile and its steps of the CTA tile: one row tile -> a step each, two -> two each, more -> all four
    const int dh = wid & 1, pair = wid >> 1;  // which half of the output columns; which of the four warp pairs
    const int mt = p.parts == 4 ? 0 : p.parts == 2 ? (pair & 1) : pair;
    const int part = p.parts == 4 ? pair : p.parts == 2 ? (pair >> 1) : 0;
    const int n_steps = 4 / p.parts, step0 = part * n_steps;
    const bool mma_warp = mt < p.m_tiles;
    const int r0 = 16 * mt + g, r1 = r0 + 8;  // the two query rows this lane's accumulators belong to

    const int total_units = p.n_kv * p.n_units;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int head = unit / p.n_units, u = unit - head * p.n_units;
        const int64_t c_begin = p.range_begin + int64_t(u) * p.unit_cells;
        const int64_t c_end = c_begin + p.unit_cells < p.range_end ? c_begin + p.unit_cells : p.range_end;
        const int n_tiles = int((c_end - c_begin + kTile - 1) / kTile);

        __syncthreads();  // the previous unit's readers of q and the ranges are done
        // ---- the group's query rows: F32 -> hi + lo FP16 (rows past m are zero); each row's cell range ----
        for (int i = tid; i < kMaxM * (HD / 8); i += kThreads) {
            const int row = i / (HD / 8), chunk = i - row * (HD / 8);
            uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = hi4;
            if (row < p.m) {
                const int t = row / p.n_rep, r = row - t * p.n_rep;
                const float4 * src = reinterpret_cast<const float4 *>(p.q + (int64_t(t) * p.n_q + head * p.n_rep + r) * HD) + 2 * chunk;
                const float4 a = __ldg(src), b = __ldg(src + 1);
                const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                uint32_t h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __half2 hh = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                    const float2 back = __half22float2(hh);
                    h[e] = h2_bits(hh);
                    l[e] = h2_bits(__floats2half2_rn(v[2 * e] - back.x, v[2 * e + 1] - back.y));
                }
                hi4 = make_uint4(h[0], h[1], h[2], h[3]), lo4 = make_uint4(l[0], l[1], l[2], l[3]);
            }
            *reinterpret_cast<uint4 *>(q_hi + swz<kRow>(row, chunk)) = hi4;
            *reinterpret_cast<uint4 *>(q_lo + swz<kRow>(row, chunk)) = lo4;
        }
        for (int row = tid; row < kMaxM; row += kThreads) {
            int64_t lo = 0, hi = 0;  // rows past m: an empty range, so every cell is masked
            if (row < p.m) {
                const int t = row / p.n_rep;
                lo = p.first_cell != nullptr ? int64_t(__ldg(p.first_cell + t)) : p.range_begin;
                hi = p.n_cells != nullptr ? lo + int64_t(__ldg(p.n_cells + t)) : p.range_end;
                if (lo < 0 || hi > p.cache_slots || hi < lo) {
                    if (p.err != nullptr) atomicOr(p.err, FNB_ERR_SLOT);
                    lo = hi = 0;
                }
                lo = lo < p.range_begin ? p.range_begin : lo;
                hi = hi > p.range_end ? p.range_end : hi;
            }
            row_lo[row] = int32_t(lo), row_hi[row] = int32_t(hi);
        }

        // ---- raw tiles: cp.async of the tile's cells of this KV head into stage `st` ----
        auto issue = [&](int tile, int st) {
            uint8_t * base = smem + L::raw + st * 2 * L::kRawTensor;
            const int64_t c0 = c_begin + int64_t(tile) * kTile;
            // a thread copies one whole cell of one tensor (2 x 64 cells = the CTA's 128 threads): no index arithmetic
            // per piece.  A 256-wide Q8_0 cell is 272 bytes = 17 x 16; a 128-wide one 136 = 17 x 8, only 8-byte aligned.
            constexpr int kPiece = L::kCell % 16 == 0 ? 16 : 8;
            constexpr int kChunks = L::kCell / kPiece;
            static_assert(4 * kTile == kThreads, "two threads a (tensor, cell)");
            {
                const int item = tid >> 1, second = tid & 1;
                const int tensor = item / kTile, cell = item - tensor * kTile;
                const int64_t c = c0 + cell;
                const bool valid = c < c_end;
                const uint8_t * src = (tensor == 0 ? p.k_cache : p.v_cache) + ((valid ? c : c_begin) * p.n_kv + head) * L::kCell;
                uint8_t * dst = base + tensor * L::kRawTensor + cell * L::kCell;
                constexpr int kFirst = (kChunks + 1) / 2;  // pieces the first thread of the pair copies
#pragma unroll
                for (int j = 0; j < kFirst; ++j) {
                    const int ch = second ? kFirst + j : j;
                    if (ch < kChunks) {
                        if (kPiece == 16) {
                            cp_async16(dst + kPiece * ch, src + kPiece * ch, valid);
                        } else {
                            cp_async8(dst + kPiece * ch, src + kPiece * ch, valid);
                        }
                    }
                }
            }
            if (KV8) {
                for (int i = tid; i < 2 * kTile; i += kThreads) {
                    const int tensor = i / kTile, cell = i - tensor * kTile;
                    const int64_t c = c0 + cell;
                    const bool valid = c < c_end;
                    const uint16_t * src = (tensor == 0 ? p.k_scale : p.v_scale) + ((valid ? c : c_begin) * p.n_kv + head) * (HD / 64);
                    uint8_t * dst = base + tensor * L::kRawTensor + kTile * L::kCell + cell * 8;
                    if (HD == 256) {
                        cp_async8(dst, src, valid);
                    } else {  // two scales a cell: 4 bytes, plain loads
                        *reinterpret_cast<uint32_t *>(dst) = valid ? __ldg(reinterpret_cast<const uint32_t *>(src)) : 0u;
                    }
                }
            }
            cp_async_commit();
        };

        // running state of this lane's two rows
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
        float o[NT][4];
#pragma unroll
        for (int d = 0; d < NT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f;

        issue(0, 0);
        for (int tile = 0; tile < n_tiles; ++tile) {
            const int st = tile & 1;
            if (tile + 1 < n_tiles) {
                issue(tile + 1, st ^ 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();  // the raw tile has landed for every thread; the previous tile's operand readers are done
            const uint8_t * raw_k = smem + L::raw + st * 2 * L::kRawTensor;
            const uint8_t * raw_v = raw_k + L::kRawTensor;
            const int64_t tile_c0 = c_begin + int64_t(tile) * kTile;

            // ---- K: the codes as FP16 integers, [cell][dim] ----
            if (!KV8) {
                widen_q8_0_tile<false, kRow>(raw_k, L::kCell, NB / 2, op, nullptr, tid);
            } else {
                for (int i = tid; i < kTile * (HD / 8); i += kThreads) {
                    const int cell = i / (HD / 8), ch = i - cell * (HD / 8);
                    const uint2 w = *reinterpret_cast<const uint2 *>(raw_k + cell * L::kCell + 8 * ch);
                    __half2 a, b, c, d;
                    codes_to_h2(w.x, a, b);
                    codes_to_h2(w.y, c, d);
                    *reinterpret_cast<uint4 *>(op + swz<kRow>(cell, ch)) = make_uint4(h2_bits(a), h2_bits(b), h2_bits(c), h2_bits(d));
                }
            }
            __syncthreads();

            // ---- scores, softmax and the P operands, step by step ----
            uint32_t p_hi[4][4], p_lo[4][4];  // [step][A fragment]
            float alpha[4][2];
            const int lo0 = row_lo[r0], hi0 = row_hi[r0], lo1 = row_lo[r1], hi1 = row_hi[r1];
#pragma unroll
            for (int st4 = 0; st4 < 4; ++st4) {
                if (st4 >= n_steps) break;
                const int cell0 = (step0 + st4) * kStep;  // first cell of this step within the tile
                float s[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
                if (mma_warp) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        float blk[2][4];
#pragma unroll
                        for (int n = 0; n < 2; ++n) blk[n][0] = blk[n][1] = blk[n][2] = blk[n][3] = 0.0f;
#pragma unroll
                        for (int kk = 0; kk < 2; ++kk) {
                            const int ks = 2 * b + kk;
                            uint32_t ah[4], al[4], kb[4];
                            const int arow = 16 * mt + (lane & 15), achunk = 2 * ks + (lane >> 4);
                            ldsm4(ah, s_addr(q_hi + swz<kRow>(arow, achunk)));
                            ldsm4(al, s_addr(q_lo + swz<kRow>(arow, achunk)));
                            const int krow = cell0 + (lane & 7) + 8 * (lane >> 4), kchunk = 2 * ks + ((lane >> 3) & 1);
                            ldsm4(kb, s_addr(op + swz<kRow>(krow, kchunk)));
                            mma16816(blk[0], ah, kb[0], kb[1]);
                            mma16816(blk[0], al, kb[0], kb[1]);
                            mma16816(blk[1], ah, kb[2], kb[3]);
                            mma16816(blk[1], al, kb[2], kb[3]);
                        }
                        // the block's scale of this lane's two cells of each 8-cell tile
#pragma unroll
                        for (int n = 0; n < 2; ++n) {
                            const int c = cell0 + 8 * n + 2 * t4;
                            float d0, d1;
                            if (KV8) {
                                const uint16_t * sc = reinterpret_cast<const uint16_t *>(raw_k + kTile * L::kCell);
                                d0 = f16_bits_to_f32(sc[4 * c + b / 2]), d1 = f16_bits_to_f32(sc[4 * (c + 1) + b / 2]);
                            } else {
                                d0 = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(raw_k + c * L::kCell + 34 * b));
                                d1 = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(raw_k + (c + 1) * L::kCell + 34 * b));
                            }
                            s[n][0] = fmaf(blk[n][0], d0, s[n][0]), s[n][1] = fmaf(blk[n][1], d1, s[n][1]);
                            s[n][2] = fmaf(blk[n][2], d0, s[n][2]), s[n][3] = fmaf(blk[n][3], d1, s[n][3]);
                        }
                    }
                }
                // mask, running maximum, probabilities (rows r0 and r1; log2 units)
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int n = 0; n < 2; ++n) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int64_t c = tile_c0 + cell0 + 8 * n + 2 * t4 + j;
                        s[n][j] = c >= lo0 && c < hi0 ? s[n][j] * p.scale_log2 : -INFINITY;
                        s[n][2 + j] = c >= lo1 && c < hi1 ? s[n][2 + j] * p.scale_log2 : -INFINITY;
                        mx0 = fmaxf(mx0, s[n][j]), mx1 = fmaxf(mx1, s[n][2 + j]);
                    }
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 1)), mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 1)), mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 2));
                const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
                // a row with no live cell so far keeps reference 0 (exp2 of -inf is 0; -inf minus -inf is never formed)
                const float ref0 = mn0 == -INFINITY ? 0.0f : mn0, ref1 = mn1 == -INFINITY ? 0.0f : mn1;
                alpha[st4][0] = fast_exp2(m_run[0] - ref0), alpha[st4][1] = fast_exp2(m_run[1] - ref1);
                m_run[0] = mn0, m_run[1] = mn1;
                float pr[2][4];
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    pr[n][0] = fast_exp2(s[n][0] - ref0), pr[n][1] = fast_exp2(s[n][1] - ref0);
                    pr[n][2] = fast_exp2(s[n][2] - ref1), pr[n][3] = fast_exp2(s[n][3] - ref1);
                }
                l_run[0] = l_run[0] * alpha[st4][0] + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
                l_run[1] = l_run[1] * alpha[st4][1] + ((pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]));
                // P as the A fragment of the step: hi + lo of p x 2^12
#pragma unroll
                for (int f = 0; f < 4; ++f) {
                    const int n = f >> 1, jb = (f & 1) * 2;  // a0: (g, tile 0), a1: (g + 8, tile 0), a2: (g, tile 1), a3: (g + 8, tile 1)
                    const float x = pr[n][jb] * kPScale, y = pr[n][jb + 1] * kPScale;
                    const __half2 hv = __floats2half2_rn(x, y);
                    const float2 back = __half22float2(hv);
                    p_hi[st4][f] = h2_bits(hv);
                    p_lo[st4][f] = h2_bits(__floats2half2_rn(x - back.x, y - back.y));
                }
            }
            __syncthreads();  // every warp is done with the K operand tile

            // ---- V: hi = rn(d x code), lo = fma(d, code, -hi) exactly, [cell][dim] each ----
            uint8_t * v_hi = op;
            uint8_t * v_lo = op + kTile * kRow;
            if (!KV8) {
                widen_q8_0_tile<true, kRow>(raw_v, L::kCell, NB / 2, v_hi, v_lo, tid);
            } else {
                const uint16_t * sc = reinterpret_cast<const uint16_t *>(raw_v + kTile * L::kCell);
                for (int i = tid; i < kTile * (HD / 8); i += kThreads) {
                    const int cell = i / (HD / 8), ch = i - cell * (HD / 8);
                    const uint2 w = *reinterpret_cast<const uint2 *>(raw_v + cell * L::kCell + 8 * ch);
                    const __half2 d2 = __half2half2(__ushort_as_half(sc[4 * cell + ch / 8]));
                    __half2 c[4], h[4], l[4];
                    codes_to_h2(w.x, c[0], c[1]);
                    codes_to_h2(w.y, c[2], c[3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        h[e] = __hmul2(d2, c[e]);
                        l[e] = __hfma2(d2, c[e], __hneg2(h[e]));
                    }
                    *reinterpret_cast<uint4 *>(v_hi + swz<kRow>(cell, ch)) = make_uint4(h2_bits(h[0]), h2_bits(h[1]), h2_bits(h[2]), h2_bits(h[3]));
                    *reinterpret_cast<uint4 *>(v_lo + swz<kRow>(cell, ch)) = make_uint4(h2_bits(l[0]), h2_bits(l[1]), h2_bits(l[2]), h2_bits(l[3]));
                }
            }
            __syncthreads();

            // ---- outputs: o = o alpha + (p_hi + p_lo) (v_hi + v_lo) without the lo x lo term ----
            if (mma_warp) {
#pragma unroll
                for (int st4 = 0; st4 < 4; ++st4) {
                    if (st4 >= n_steps) break;
                    const int cell0 = (step0 + st4) * kStep;
                    // the maximum seldom moves once a few tiles are in: skip the rescaling when no row of the warp needs it
                    if (__any_sync(kFull, alpha[st4][0] != 1.0f || alpha[st4][1] != 1.0f)) {
#pragma unroll
                        for (int d = 0; d < NT; ++d) {
                            o[d][0] *= alpha[st4][0], o[d][1] *= alpha[st4][0];
                            o[d][2] *= alpha[st4][1], o[d][3] *= alpha[st4][1];
                        }
                    }
#pragma unroll
                    for (int dp = 0; dp < NT / 2; ++dp) {
                        uint32_t bh[4], bl[4];
                        const int vrow = cell0 + (lane & 7) + 8 * ((lane >> 3) & 1), vchunk = dh * kHalfChunks + 2 * dp + (lane >> 4);
                        ldsm4_t(bh, s_addr(v_hi + swz<kRow>(vrow, vchunk)));
                        ldsm4_t(bl, s_addr(v_lo + swz<kRow>(vrow, vchunk)));
                        mma16816(o[2 * dp], p_hi[st4], bh[0], bh[1]);
                        mma16816(o[2 * dp], p_lo[st4], bh[0], bh[1]);
                        mma16816(o[2 * dp], p_hi[st4], bl[0], bl[1]);
                        mma16816(o[2 * dp + 1], p_hi[st4], bh[2], bh[3]);
                        mma16816(o[2 * dp + 1], p_lo[st4], bh[2], bh[3]);
                        mma16816(o[2 * dp + 1], p_hi[st4], bl[2], bl[3]);
                    }
                }
            }
        }

        // ---- the unit's partial result of this warp: (max, sum, output / 2^12) of its rows ----
        if (mma_warp) {
            float l0 = l_run[0], l1 = l_run[1];
            l0 += __shfl_xor_sync(kFull, l0, 1), l0 += __shfl_xor_sync(kFull, l0, 2);
            l1 += __shfl_xor_sync(kFull, l1, 1), l1 += __shfl_xor_sync(kFull, l1, 2);
            const int64_t slot = (int64_t(head) * p.n_units + u) * p.parts + part;
            float * ml = p.ws_ml + slot * p.m * 2;
            float * acc = p.ws_acc + slot * p.m * HD;
            const int col0 = dh * (HD / 2);  // this warp's half of the output columns; the pair's first warp writes (max, sum)
            if (r0 < p.m) {
                if (t4 == 0 && dh == 0) ml[2 * r0] = m_run[0], ml[2 * r0 + 1] = l0;
#pragma unroll
                for (int d = 0; d < NT; ++d) {
                    *reinterpret_cast<float2 *>(acc + int64_t(r0) * HD + col0 + 8 * d + 2 * t4) = make_float2(o[d][0] * kPUnscale, o[d][1] * kPUnscale);
                }
            }
            if (r1 < p.m) {
                if (t4 == 0 && dh == 0) ml[2 * r1] = m_run[1], ml[2 * r1 + 1] = l1;
#pragma unroll
                for (int d = 0; d < NT; ++d) {
                    *reinterpret_cast<float2 *>(acc + int64_t(r1) * HD + col0 + 8 * d + 2 * t4) = make_float2(o[d][2] * kPUnscale, o[d][3] * kPUnscale);
                }
            }
        }
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

template <int HD, bool KV8>
bool configure() {
    static std::atomic<bool> done[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!done[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(attend_kernel<HD, KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_layout<HD, KV8>::total) != cudaSuccess) {
            return false;
        }
        done[dev].store(true, std::memory_order_release);
    }
    return true;
}

template <int HD, bool KV8>
int32_t launch_hd(const attend_params & p, cudaStream_t s) {
    if (!configure<HD, KV8>()) return FNB_LAUNCH_FAILED;
    const int units = p.n_kv * p.n_units;
    attend_kernel<HD, KV8><<<units < kSmCount ? units : kSmCount, kThreads, smem_layout<HD, KV8>::total, s>>>(p);
    if (cudaPeekAtLastError() != cudaSuccess) return FNB_LAUNCH_FAILED;
    attend_fold_kernel<HD><<<p.rows * p.n_q, HD * kFoldLanes, 0, s>>>(p);
    return launch_status();
}

bool shape_ok(const fnb_attend_args * a) {
    if (a == nullptr) return false;
    if (a->head_dim != 128 && a->head_dim != 256) return false;
    if (a->rows < 1 || a->n_q_heads < 1 || a->n_kv_heads < 1 || a->n_q_heads % a->n_kv_heads != 0) return false;
    if (int64_t(a->rows) * (a->n_q_heads / a->n_kv_heads) > kMaxM) return false;
    if (a->cache_slots < 1 || a->cache_slots > INT32_MAX) return false;
    if (a->range_begin < 0 || a->range_end <= a->range_begin || a->range_end > a->cache_slots) return false;
    return true;
}

}  // namespace

bool attend_prepare_device() {
    return configure<256, false>() && configure<256, true>() && configure<128, false>() && configure<128, true>();
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
    if (plan.n_units * plan.parts > kFoldMaxSlots) return FNB_REJECTED;  // cannot happen with the plan's two units an SM
    if (!ok_ptr(ws, 16) || ws_bytes < plan_bytes(plan, a->head_dim)) return FNB_REJECTED;

    attend_params p;
    p.q = a->q, p.gate = a->gate;
    p.k_cache = static_cast<const uint8_t *>(a->k_cache), p.v_cache = static_cast<const uint8_t *>(a->v_cache);
    p.k_scale = a->k_scale, p.v_scale = a->v_scale, p.first_cell = a->first_cell, p.n_cells = a->n_cells;
    p.out = a->out, p.err = a->err;
    p.ws_ml = static_cast<float *>(ws);
    p.ws_acc = p.ws_ml + plan.slots * plan.m * 2;
    p.cache_slots = a->cache_slots, p.range_begin = a->range_begin, p.range_end = a->range_end, p.unit_cells = plan.unit_cells;
    p.rows = a->rows, p.n_q = a->n_q_heads, p.n_kv = a->n_kv_heads, p.n_rep = a->n_q_heads / a->n_kv_heads;
    p.m = plan.m, p.m_tiles = plan.m_tiles, p.parts = plan.parts, p.n_units = plan.n_units;
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
