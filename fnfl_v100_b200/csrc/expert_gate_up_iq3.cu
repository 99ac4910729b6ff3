// The routed experts' gate / up mat-vec for a decode window with the GLU fused,
//     ff[t][r] = silu(g) u,   g = gate row r . act[t],  u = up row r . act[t],   t < nt,  r in [r0, r1)
// with ggml IQ3_XXS or IQ3_S weights against Q8_K activations (fnb_quantize_q8_k).  Replaces fn::experts::cpu::iq_gu_rows
// for fmt iq3_xxs and iq3_s (fn/kernels/experts/cpu_kernels.h:67; cpu_iq_avx2.cpp:256-271 and :273-290 decode, :305-337
// row_dot, :429-445 gu_rows; IQ3_S's differences are listed at `shape` below, the text here describes IQ3_XXS)
// and returns the SAME BITS: the AVX2 kernel keeps, per (row, t), eight int32 lanes a super-block - lane l collects,
// over the block's eight groups of 32 values, (2 s + 1) x the four codebook bytes of the group's index byte l times the
// sign-applied Q8_K codes 32 g + 4 l .. - adds them as floats by one fused multiply-add per super-block and lane with
// x.d y.d (x.d WITHOUT the format's 1/4), reduces in ggml's hsum_float_8 order, multiplies the sum by 1/4 and applies
// g / (1 + expf(-g)) * u (expf as the host C library evaluates it: exact_math.cuh).
//
// A warp takes four (gate, up) row pairs at a time: lanes 0..15 the gate rows, lanes 16..31 the up rows, FOUR GPU
// lanes a row, lane k standing for AVX2 lanes 2 k and 2 k + 1 (eight values of every group, which share one 7-bit
// sign index).  At three bits a weight the kernel is bound by instruction issue and shared-memory lookups, not by HBM:
// per eight weights one 16-bit index load, two codebook loads, one sign-mask load, about fifteen integer operations
// and, per window row, half a 16-byte activation load, two dp4a and two multiply-adds.
//
// The signs go onto the CODEBOOK bytes (once per weight, whatever the window), which equals the reference's negated
// codes unless a code is -128: _mm256_sign_epi8 leaves -128 as it is.  ggml's Q8_K quantiser cannot emit -128, but a
// CTA that finds one in its window takes the variant that negates the codes byte-wise in two's complement instead.
//
// The kernel is bound by instruction issue, so what can be a conflict-free shared-memory lookup is one: the codebook
// (256 entries of four magnitudes as bytes) is kept 32 times, copy j in bank j (one copy: about three wavefronts a
// lookup), and the 128 sign indices' eight byte masks (seven stored bits and their parity) 16 times, copy j in the
// bank pair 2 j, which replaces ten integer operations per eight weights.
//
// A row is 98-byte blocks; with an even number of them (n a multiple of 512) rows are 4-byte aligned.  A warp copies
// its eight rows (up to ten super-blocks of each at a time) with cp.async into its own shared-memory buffers, one unit
// ahead of the one it computes on: 16-byte copies between the 16-byte boundaries of the source, whose offset within 16
// bytes the shared-memory copy keeps, and up to three 4-byte copies at either end.
#include <atomic>

#include "common.cuh"
#include "exact_math.cuh"
#include "stage_span.cuh"

#ifndef FNB_GU_IQ3_GRID
#define FNB_GU_IQ3_GRID 1
#endif

namespace fnb {
namespace {

constexpr int kMaxWarps = 12;
constexpr int kMaxT = 8;
constexpr int kWholeRowBlocks = 10;                  // rows of up to ten super-blocks (2560 columns) are staged whole,
constexpr int kChunkBlocks = 8;                      // longer ones eight super-blocks (a multiple of 16 bytes) at a time
constexpr int kGridCopies = 32;                      // the codebook once per bank
constexpr int kSignCopies = 16;                      // 8-byte entries: a half-warp's lookups fill the 32 banks

// The five formats of fn::experts::cpu::iq_gu_rows (cpu_iq_avx2.cpp:551-565).  All share the row kernel's lane structure
// (eight int32 lanes a 32-value half, lane l the half's values 4 l .. 4 l + 3); they differ in how a half's codebook
// indices, signs and scale are packed, in the codebook, and in where the format's constant K enters:
//   IQ3_XXS  98 bytes: d, qs[64], eight words of 4 x 7-bit sign index + 4-bit scale; 256 entries of 4 magnitudes
//   IQ3_S   110 bytes: d, qs[64], qh[8] (ninth index bits), signs[32] (plain bits), scales[4] (a nibble per half); 512 entries
//   IQ2_XXS  66 bytes: d, eight x (4 index bytes, then 4 x 7-bit sign index + 4-bit scale); 256 entries of 8 magnitudes
//   IQ2_XS   74 bytes: d, 32 x u16 (9-bit index, 7-bit sign index), scales[8] (a nibble per 16 values); 512 entries of 8
//   IQ2_S    82 bytes: d, qs[32] (index low bytes), signs[32] (plain bits), qh[8] (index bits 8-9), scales[8]; 1024 of 8
// K: IQ3_XXS 1/4, IQ2_S 1/8 on the reduced sum with ggml's reduction order; IQ2_XXS, IQ2_XS 1/8 folded into d with the
// plain pairwise order; IQ3_S none (cpu_iq_avx2.cpp:203-206, :325-336).
enum { kIq3Xxs = 0, kIq3S = 1, kIq2Xxs = 2, kIq2Xs = 3, kIq2S = 4 };

template <int FMT>
struct shape {
    static constexpr bool kTwo = FMT >= kIq2Xxs;                      // 8-byte codebook entries (eight magnitudes)
    static constexpr bool kSignTable = FMT == kIq3Xxs || FMT == kIq2Xxs || FMT == kIq2Xs;  // 7-bit sign indices
    static constexpr int kBlock = FMT == kIq3Xxs ? 98 : FMT == kIq3S ? 110 : FMT == kIq2Xxs ? 66 : FMT == kIq2Xs ? 74 : 82;
    // a slot: ten blocks and 12 bytes of source offset, rounded up so that the eight slots start in different banks
    static constexpr int kSlot = FMT == kIq3Xxs ? 1008 : FMT == kIq3S ? 1136 : FMT == kIq2Xxs ? 688 : FMT == kIq2Xs ? 784 : 848;
    static constexpr int kUnit = 8 * kSlot;           // four gate rows, then four up rows
    static constexpr int kWarpStage = 2 * kUnit;      // two units: the one computed on and the one in flight
    static constexpr int kSpan = 4 * kWholeRowBlocks * kBlock + 16;  // four whole rows, back to back as in global memory
    static constexpr int kGridEntries = FMT == kIq3Xxs || FMT == kIq2Xxs ? 256 : FMT == kIq2S ? 1024 : 512;
    // copies of the codebook: 4-byte entries once per bank; 8-byte entries once per bank pair, fewer where the
    // codebook is large (IQ2_S: 1024 entries x 8 bytes x 8 copies = 64 KB)
    static constexpr int kCopies = !kTwo ? kGridCopies : FMT == kIq2S ? 8 : 16;
    static constexpr int kGridBytes = kGridEntries * kCopies * (kTwo ? 8 : 4);
    static constexpr int kSignBytes = kSignTable ? 128 * kSignCopies * 8 : 0;  // plain sign bits need no table
    static constexpr int kTableBytes = kGridBytes + kSignBytes;
    static constexpr bool kGgmlSum = FMT == kIq3Xxs || FMT == kIq3S || FMT == kIq2S;  // ggml's hsum_float_8 order, K at the end
    static constexpr float kEndK = FMT == kIq3Xxs ? 0.25f : FMT == kIq2S ? 0.125f : 1.0f;
    static constexpr float kBlockK = FMT == kIq2Xxs || FMT == kIq2Xs ? 0.125f : 1.0f;      // K folded into the block's d
    static_assert(2 * kSpan <= kUnit, "two spans fit a unit");
    static_assert(kSlot % 16 == 0 && kSlot >= kWholeRowBlocks * kBlock + 12, "a slot holds ten blocks and the source offset");
};
constexpr size_t kSmemLimit = 224 * 1024;            // one CTA an SM (227 KB less the static arrays)
constexpr int kGridPerSm = FNB_GU_IQ3_GRID;

__constant__ uint16_t c_grid_packed[256] = {
#include "iq3xxs_grid_packed.inc"
};
__constant__ uint16_t c_grid3s_packed[512] = {
#include "iq3s_grid_packed.inc"
};
// the IQ2 codebooks: eight 2-bit level indices an entry (magnitudes 8, 25, 43)
__constant__ uint16_t c_grid2xxs_packed[256] = {
#include "iq2xxs_grid_packed.inc"
};
__constant__ uint16_t c_grid2xs_packed[512] = {
#include "iq2xs_grid_packed.inc"
};
__constant__ uint16_t c_grid2s_packed[1024] = {
#include "iq2s_grid_packed.inc"
};

// 0xFF in byte j where bit j of a 4-bit sign field is set: the field times 0x10204080 puts bit j at the top of byte j,
// and a byte permute with the replicate-sign selectors spreads it over the byte
__device__ __forceinline__ uint32_t spread_msb(uint32_t v) {
    uint32_t r;  // prmt's selector bit 3 replicates the chosen byte's top bit (the __byte_perm intrinsic drops that bit)
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(v), "r"(0xba98u));
    return r;
}

// codebook bytes (4 .. 62) negated where the mask byte is 0xFF: 256 - g never carries out of its byte
__device__ __forceinline__ int signed_grid(uint32_t g, uint32_t mff) { return int((g ^ mff) + (mff & 0x01010101u)); }

// Q8_K codes negated in two's complement where the mask byte is 0xFF, -128 staying -128 (_mm256_sign_epi8)
__device__ __forceinline__ int signed_codes(uint32_t y, uint32_t mff) {
    const uint32_t a = y ^ mff;
    return int(((a & 0x7f7f7f7fu) + (mff & 0x01010101u)) ^ (a & 0x80808080u));
}

// where row r's chunk of a matrix starts; a ragged last quad re-reads the last row (its results are not stored)
template <int FMT>
__device__ __forceinline__ const uint8_t * chunk_src(const uint8_t * mat, int64_t row_bytes, int64_t r, int64_t r1, int chunk) {
    return mat + (r < r1 ? r : r1 - 1) * row_bytes + int64_t(chunk) * (kChunkBlocks * shape<FMT>::kBlock);
}

template <int FMT>
__device__ __forceinline__ void stage_unit(uint32_t buf_sm, const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up,
                                           int64_t row_bytes, int64_t r4, int64_t r1, int chunk, int bytes, int lane) {
#pragma unroll
    for (int slot = 0; slot < 8; ++slot) {
        stage_span(buf_sm + slot * shape<FMT>::kSlot, chunk_src<FMT>(slot < 4 ? gate : up, row_bytes, r4 + (slot & 3), r1, chunk), bytes,
                   lane);
    }
    cp_async_commit();
}

// rows of up to ten super-blocks: the quad's four gate rows are one contiguous span of the matrix, its up rows another
template <int FMT>
__device__ __forceinline__ void stage_unit_whole(uint32_t buf_sm, const uint8_t * __restrict__ gate,
                                                 const uint8_t * __restrict__ up, int64_t row_bytes, int64_t r4, int64_t r1,
                                                 int lane) {
    const int rows = r1 - r4 < 4 ? int(r1 - r4) : 4;  // a ragged last quad leaves its missing rows' bytes as they were
    stage_span(buf_sm, gate + r4 * row_bytes, rows * int(row_bytes), lane);
    stage_span(buf_sm + shape<FMT>::kSpan, up + r4 * row_bytes, rows * int(row_bytes), lane);
    cp_async_commit();
}

// one staged unit (n_blk super-blocks of the lane's row, x) against the window: acc[t][0 / 1] are AVX2 lanes 2 k, 2 k + 1
template <int NT, bool WRAP, int FMT>
__device__ __forceinline__ void dot_unit(const uint8_t * x, int n_blk, const uint8_t * codes_sm, const float * d_sm, int nb,
                                         int blk0, int k, const uint32_t * grid_lane, const uint2 * sign_lane, float (&acc)[NT][2]) {
    const int sh7 = 7 * k;
#pragma unroll 1
    for (int i = 0; i < n_blk; ++i, x += shape<FMT>::kBlock) {
        // d, times the format's K where the reference folds it into the block scale (an exact power of two)
        const float dx = __fmul_rn(f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(x)), shape<FMT>::kBlockK);
        int a0[NT], a1[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) a0[t] = 0, a1[t] = 0;
        const uint8_t * y0 = codes_sm + size_t(blk0 + i) * 256 + 16 * k;
        uint4 y4[NT];
#pragma unroll
        for (int grp = 0; grp < 8; ++grp) {
            // the lane's eight values of this 32-value half: their magnitudes as two words of four bytes (c0: AVX2 lane
            // 2 k, c1: lane 2 k + 1), their sign masks (0xFF where negative) and the half's scale for this lane
            uint32_t c0, c1, m0, m1;
            int sc;
            if (FMT == kIq3S) {
                const uint32_t h = *reinterpret_cast<const uint16_t *>(x + 2 + 8 * grp + 2 * k);  // index bytes 2 k, 2 k + 1
                uint32_t e0 = h & 0xffu, e1 = h >> 8;
                // ninth index bits 2 k, 2 k + 1 of the group's qh byte; sign byte k of the group's four (bit i: value
                // 8 k + i); the group's nibble of the scale byte it shares with its neighbour
                const uint32_t hb = uint32_t(x[66 + grp]) >> (2 * k);
                e0 |= (hb & 1u) << 8, e1 |= (hb & 2u) << 7;
                const uint32_t sb = x[74 + 4 * grp + k];
                m0 = spread_msb((sb & 15u) * 0x10204080u), m1 = spread_msb((sb >> 4) * 0x10204080u);
                const uint32_t sn = x[106 + (grp >> 1)];
                sc = int(2u * ((grp & 1) ? sn >> 4 : sn & 15u) + 1u);
                c0 = grid_lane[e0 * kGridCopies], c1 = grid_lane[e1 * kGridCopies];
            } else if (FMT == kIq3Xxs) {
                const uint32_t h = *reinterpret_cast<const uint16_t *>(x + 2 + 8 * grp + 2 * k);
                // the group's sign / scale word (2-byte aligned), read by each of the row's four lanes: handing it round
                // by shuffles from the lane that loaded it was slower (0.144 against 0.138 ms at a window of one row)
                const uint16_t * pg = reinterpret_cast<const uint16_t *>(x + 66 + 4 * grp);
                const uint32_t w = uint32_t(pg[0]) | (uint32_t(pg[1]) << 16);
                // the group's sign index k -> its eight byte masks; computing them here (mask, popc for the parity, two
                // multiplies, two permutes) instead of the lookup: 0.150 against 0.138 ms at a window of one row
                const uint2 sg = sign_lane[((w >> sh7) & 127u) * kSignCopies];
                m0 = sg.x, m1 = sg.y;
                sc = int(2u * (w >> 28) + 1u);
                c0 = grid_lane[(h & 0xffu) * kGridCopies], c1 = grid_lane[(h >> 8) * kGridCopies];
            } else {
                // the IQ2 formats: ONE codebook entry of eight magnitudes is the lane's whole share of the half
                const uint2 * grid2 = reinterpret_cast<const uint2 *>(grid_lane);  // this lane's copy (see run_warp)
                uint32_t e;
                if (FMT == kIq2Xxs) {
                    const uint16_t * pq = reinterpret_cast<const uint16_t *>(x + 2 + 8 * grp);  // 4 index bytes, then the sign / scale word
                    e = (uint32_t(pq[k >> 1]) >> (8 * (k & 1))) & 0xffu;
                    const uint32_t w = uint32_t(pq[2]) | (uint32_t(pq[3]) << 16);
                    const uint2 sg = sign_lane[((w >> sh7) & 127u) * kSignCopies];
                    m0 = sg.x, m1 = sg.y;
                    sc = int(2u * (w >> 28) + 1u);
                } else if (FMT == kIq2Xs) {
                    const uint32_t q = *reinterpret_cast<const uint16_t *>(x + 2 + 8 * grp + 2 * k);  // 9-bit index, 7-bit sign index
                    e = q & 511u;
                    const uint2 sg = sign_lane[(q >> 9) * kSignCopies];
                    m0 = sg.x, m1 = sg.y;
                    const uint32_t sn = x[66 + grp];  // low nibble: the half's first 16 values, high nibble: its last 16
                    sc = int(2u * (k < 2 ? sn & 15u : sn >> 4) + 1u);
                } else {
                    e = uint32_t(x[2 + 4 * grp + k]) | (((uint32_t(x[66 + grp]) >> (2 * k)) & 3u) << 8);
                    const uint32_t sb = x[34 + 4 * grp + k];
                    m0 = spread_msb((sb & 15u) * 0x10204080u), m1 = spread_msb((sb >> 4) * 0x10204080u);
                    const uint32_t sn = x[74 + grp];
                    sc = int(2u * (k < 2 ? sn & 15u : sn >> 4) + 1u);
                }
                const uint2 c = grid2[e * shape<FMT>::kCopies];
                c0 = c.x, c1 = c.y;
            }
            const int v0 = WRAP ? int(c0) : signed_grid(c0, m0), v1 = WRAP ? int(c1) : signed_grid(c1, m1);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                // one 16-byte load brings the lane's codes of two groups (the window's blocks are stored that way)
                if ((grp & 1) == 0) y4[t] = *reinterpret_cast<const uint4 *>(y0 + size_t(t) * nb * 256 + 32 * grp);
                const uint2 y = (grp & 1) == 0 ? make_uint2(y4[t].x, y4[t].y) : make_uint2(y4[t].z, y4[t].w);
                if (WRAP) {
                    a0[t] += sc * __dp4a(v0, signed_codes(y.x, m0), 0);
                    a1[t] += sc * __dp4a(v1, signed_codes(y.y, m1), 0);
                } else {
                    a0[t] += sc * __dp4a(v0, int(y.x), 0);
                    a1[t] += sc * __dp4a(v1, int(y.y), 0);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float dxy = __fmul_rn(dx, d_sm[t * nb + blk0 + i]);
            acc[t][0] = __fmaf_rn(dxy, float(a0[t]), acc[t][0]);
            acc[t][1] = __fmaf_rn(dxy, float(a1[t]), acc[t][1]);
        }
    }
}

template <int NT, bool WRAP, int FMT>
__device__ __forceinline__ void run_warp(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes,
                                         int nb, const uint8_t * codes_sm, const float * d_sm, uint8_t * stage,
                                         const uint32_t * grid_sm, const uint2 * sign_sm, float * __restrict__ ff,
                                         int64_t ff_stride, float * __restrict__ gu, int64_t r0, int64_t r1) {
    const int lane = threadIdx.x & 31, k = lane & 3, sub = (lane >> 2) & 3, mat = lane >> 4;
    const int warps = blockDim.x >> 5;
    const int64_t n_quads = (r1 - r0 + 3) / 4, stride = int64_t(gridDim.x) * warps;
    const bool whole = nb <= kWholeRowBlocks;
    const int chunk_blocks = whole ? nb : kChunkBlocks;
    const int n_chunks = (nb + chunk_blocks - 1) / chunk_blocks;
    const auto blocks_of = [&](int chunk) { return chunk == n_chunks - 1 ? nb - chunk * chunk_blocks : chunk_blocks; };
    int64_t q = int64_t(blockIdx.x) * warps + (threadIdx.x >> 5);
    if (q >= n_quads) return;
    const uint32_t stage_sm = uint32_t(__cvta_generic_to_shared(stage));
    const uint8_t * mine = mat == 0 ? gate : up;
    int c = 0, trip = 0;
    if (whole) {
        stage_unit_whole<FMT>(stage_sm, gate, up, row_bytes, r0 + 4 * q, r1, lane);
    } else {
        stage_unit<FMT>(stage_sm, gate, up, row_bytes, r0 + 4 * q, r1, 0, blocks_of(0) * shape<FMT>::kBlock, lane);
    }
    float acc[NT][2];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t][0] = 0.0f, acc[t][1] = 0.0f;
    for (;;) {
        int64_t qn = q;
        int cn = c + 1;
        if (cn == n_chunks) cn = 0, qn = q + stride;
        const bool more = qn < n_quads;
        if (more) {
            const uint32_t next_sm = stage_sm + uint32_t((trip + 1) & 1) * shape<FMT>::kUnit;
            if (whole) {
                stage_unit_whole<FMT>(next_sm, gate, up, row_bytes, r0 + 4 * qn, r1, lane);
            } else {
                stage_unit<FMT>(next_sm, gate, up, row_bytes, r0 + 4 * qn, r1, cn, blocks_of(cn) * shape<FMT>::kBlock, lane);
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const int64_t r = r0 + 4 * q + sub;
        {
            const uint8_t * x = stage + (trip & 1) * shape<FMT>::kUnit;
            if (whole) {
                const uintptr_t src = reinterpret_cast<uintptr_t>(mine + (r0 + 4 * q) * row_bytes);
                x += mat * shape<FMT>::kSpan + (src & 15) + sub * int(row_bytes);
            } else {
                const uintptr_t src = reinterpret_cast<uintptr_t>(chunk_src<FMT>(mine, row_bytes, r, r1, c));
                x += (4 * mat + sub) * shape<FMT>::kSlot + (src & 15);
            }
            dot_unit<NT, WRAP, FMT>(x, blocks_of(c), codes_sm, d_sm, nb, c * chunk_blocks, k,
                                    shape<FMT>::kTwo ? grid_sm + 2 * (lane & (shape<FMT>::kCopies - 1)) : grid_sm + lane,
                                    sign_sm + (lane & (kSignCopies - 1)), acc);
        }
        __syncwarp();  // every lane is done with the buffer the next trip's copies overwrite
        if (c == n_chunks - 1) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                // r_l on lane l / 2: first r_l + r_(l + 4) (two lanes up) in either order.  ggml's hsum_float_8 then adds
                // lanes 2, 3 onto 0, 1 (one lane up) and lane 1 onto lane 0 (the lane's own pair); the plain pairwise
                // order (hsum8, cpu_iq_avx2.cpp:187-193) adds the lane's own pair first and then the lane above.
                float a = acc[t][0], b = acc[t][1];
                a = __fadd_rn(__shfl_down_sync(kFull, a, 2, 4), a), b = __fadd_rn(__shfl_down_sync(kFull, b, 2, 4), b);
                float sum;
                if (shape<FMT>::kGgmlSum) {
                    a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 4)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 4));
                    sum = __fadd_rn(a, b);
                } else {
                    const float c = __fadd_rn(a, b);
                    sum = __fadd_rn(c, __shfl_down_sync(kFull, c, 1, 4));
                }
                const float dot = __fmul_rn(shape<FMT>::kEndK, sum);  // the format's K where it applies to the reduced sum
                const float us = __shfl_down_sync(kFull, dot, 16);  // the up row's sits 16 lanes above the gate row's
                if (mat == 0 && k == 0 && r < r1) {
                    ff[int64_t(t) * ff_stride + r] = __fmul_rn(__fdiv_rn(dot, __fadd_rn(1.0f, exact_expf(-dot))), us);
                    if (gu != nullptr) {
                        gu[int64_t(t) * ff_stride + r] = dot;
                        gu[(int64_t(NT) + t) * ff_stride + r] = us;
                    }
                }
                acc[t][0] = 0.0f, acc[t][1] = 0.0f;
            }
        }
        if (!more) break;
        q = qn, c = cn, ++trip;
    }
}

template <int NT, int FMT>
__global__ void __launch_bounds__(kMaxWarps * 32)
    gate_up_iq3_kernel(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes, int nb,
                           const uint8_t * __restrict__ act, int64_t act_stride, int act_bytes, float * __restrict__ ff,
                           int64_t ff_stride, float * __restrict__ gu, int64_t r0, int64_t r1) {
    // the codebook copies, the sign masks' copies, the window's codes [NT][nb][256] and scales [NT][nb], then each
    // warp's two units
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t * grid_sm = reinterpret_cast<uint32_t *>(smem);
    uint2 * sign_sm = reinterpret_cast<uint2 *>(smem + shape<FMT>::kGridBytes);
    uint8_t * codes_sm = smem + shape<FMT>::kTableBytes;
    float * d_sm = reinterpret_cast<float *>(codes_sm + size_t(NT) * nb * 256);
    load_exp2_table();
    int has_m128 = 0;
    for (int i = threadIdx.x; i < NT * nb * 65; i += blockDim.x) {  // the scale and the 64 code words of every block
        const int blk = i / 65, word = i - blk * 65;
        const int t = blk / nb, b = blk - t * nb;
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(act + int64_t(t) * act_stride) + b * 73 + word);
        if (word == 0) {
            d_sm[blk] = __uint_as_float(w);
        } else {
            // codes 32 g + 8 k .. + 7 of group g (two words) go to 64 (g / 2) + 16 k + 8 (g % 2): lane k's codes of a pair
            // of groups are 16 contiguous bytes
            const int j = word - 1, g = j >> 3, kk = (j & 7) >> 1;
            reinterpret_cast<uint32_t *>(codes_sm)[blk * 64 + (g >> 1) * 16 + kk * 4 + (g & 1) * 2 + (j & 1)] = w;
            const uint32_t v = w ^ 0x80808080u;  // a code byte equal to 0x80
            has_m128 |= ((v - 0x01010101u) & ~v & 0x80808080u) != 0u;
        }
    }
    __syncthreads();
    // the codebook's magnitudes as bytes, expanded from the packed level indices straight into the copies: one word an
    // entry (IQ3: entry e's copy j at word e kGridCopies + j), or two (IQ2: at uint2 index e kCopies + j)
    for (int i = threadIdx.x; i < shape<FMT>::kGridEntries * shape<FMT>::kCopies; i += blockDim.x) {
        const int e = i / shape<FMT>::kCopies;
        if (!shape<FMT>::kTwo) {
            const uint32_t c = FMT == kIq3S ? c_grid3s_packed[e] : c_grid_packed[e];  // four 3-bit levels
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lvl = (c >> (3 * j)) & 7u;
                // IQ3_S: 1, 3 .. 15; IQ3_XXS: 4, 12 .. 52, 62
                w |= (FMT == kIq3S ? 2u * lvl + 1u : (lvl == 7u ? 62u : 4u + 8u * lvl)) << (8 * j);
            }
            grid_sm[i] = w;
        } else {
            const uint32_t c = FMT == kIq2Xxs ? c_grid2xxs_packed[e] : FMT == kIq2Xs ? c_grid2xs_packed[e] : c_grid2s_packed[e];
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t lvl = (c >> (2 * j)) & 3u;  // 8, 25, 43
                w[j >> 2] |= (lvl == 0u ? 8u : lvl == 1u ? 25u : 43u) << (8 * (j & 3));
            }
            reinterpret_cast<uint2 *>(grid_sm)[i] = make_uint2(w[0], w[1]);
        }
    }
    for (int i = threadIdx.x; i < (shape<FMT>::kSignTable ? 128 * kSignCopies : 0); i += blockDim.x) {
        // sign index s7: values 0 .. 6 of its eight take bits 0 .. 6, value 7 their parity (ksigns_iq2xs)
        const uint32_t s7 = uint32_t(i) / kSignCopies;
        sign_sm[i] = make_uint2(spread_msb((s7 & 15u) * 0x10204080u),
                                spread_msb((s7 >> 4) * 0x10204080u + (uint32_t(__popc(s7)) << 31)));
    }
    const int wrap = __syncthreads_or(has_m128);
    uint8_t * stage = smem + shape<FMT>::kTableBytes + act_bytes + size_t(threadIdx.x >> 5) * shape<FMT>::kWarpStage;
    if (wrap) {
        run_warp<NT, true, FMT>(gate, up, row_bytes, nb, codes_sm, d_sm, stage, grid_sm, sign_sm, ff, ff_stride, gu, r0, r1);
    } else {
        run_warp<NT, false, FMT>(gate, up, row_bytes, nb, codes_sm, d_sm, stage, grid_sm, sign_sm, ff, ff_stride, gu, r0, r1);
    }
}

template <int NT, int FMT>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(gate_up_iq3_kernel<NT, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemLimit)) !=
            cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

// window rows one launch can hold for nb super-blocks a row (their codes and scales and at least two warps' buffers)
template <int FMT>
int window_rows(int nb) {
    const size_t per_t = size_t(nb) * 260, room = kSmemLimit - shape<FMT>::kTableBytes - 2 * size_t(shape<FMT>::kWarpStage) - 16;
    const size_t m = room / per_t;
    return int(m > size_t(kMaxT) ? size_t(kMaxT) : m);
}

template <int NT, int FMT>
int32_t launch_nt(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride,
                  float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t act_bytes = (size_t(NT) * nb * 260 + 15) & ~size_t(15);
    constexpr size_t tables = shape<FMT>::kTableBytes, per_warp = shape<FMT>::kWarpStage;
    if (tables + act_bytes + per_warp > kSmemLimit) return FNB_REJECTED;
    int warps = int((kSmemLimit - tables - act_bytes) / per_warp);  // one CTA an SM, as many warps as fit
    warps = warps > kMaxWarps ? kMaxWarps : warps;
    if (!ensure_configured<NT, FMT>()) return FNB_LAUNCH_FAILED;
    const size_t smem = tables + act_bytes + size_t(warps) * per_warp;
    const int64_t quads = (r1 - r0 + 3) / 4;
    const int grid = grid_for((quads + warps - 1) / warps, kGridPerSm);
    gate_up_iq3_kernel<NT, FMT><<<grid, warps * 32, smem, s>>>(gate, up, row_bytes, nb, act, act_stride, int(act_bytes), ff,
                                                                ff_stride, gu, r0, r1);
    return launch_status();
}

template <int FMT>
bool prepare_fmt() {
    return ensure_configured<1, FMT>() && ensure_configured<2, FMT>() && ensure_configured<3, FMT>() && ensure_configured<4, FMT>() &&
           ensure_configured<5, FMT>() && ensure_configured<6, FMT>() && ensure_configured<7, FMT>() && ensure_configured<8, FMT>();
}

template <int FMT>
int32_t gate_up_rows(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                     int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    if (!ok_ptr(gate, 16) || !ok_ptr(up, 16) || !ok_ptr(act, 4) || !ok_ptr(ff, 4) || !ok_opt(gu, 4)) return FNB_REJECTED;
    // an even number of super-blocks a row: rows on 4-byte boundaries, which the copies into shared memory need
    if (n < 512 || n > 16384 || n % 512 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 256;
    if (row_bytes != int64_t(nb) * shape<FMT>::kBlock || act_stride < int64_t(nb) * 292 || act_stride % 4 != 0 || ff_stride < r1) {
        return FNB_REJECTED;
    }
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * gp = static_cast<const uint8_t *>(gate);
    const uint8_t * upp = static_cast<const uint8_t *>(up);
    const uint8_t * a = static_cast<const uint8_t *>(act);
    const int max_t = window_rows<FMT>(nb);
    if (max_t < 1) return FNB_REJECTED;
    // g and u of a later pass would need their own [2][m] planes: the debug output is for windows of one pass
    if (gu != nullptr && nt > max_t) return FNB_REJECTED;
    for (int t0 = 0; t0 < nt; t0 += max_t) {  // longer windows take further passes, as the reference's do above eight rows
        const int m = nt - t0 < max_t ? nt - t0 : max_t;
        const uint8_t * at = a + int64_t(t0) * act_stride;
        float * ft = ff + int64_t(t0) * ff_stride;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 2: st = launch_nt<2, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 3: st = launch_nt<3, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 4: st = launch_nt<4, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 5: st = launch_nt<5, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 6: st = launch_nt<6, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 7: st = launch_nt<7, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            default: st = launch_nt<8, FMT>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}

}  // namespace

bool expert_gate_up_prepare_device() {
    return prepare_fmt<kIq3Xxs>() && prepare_fmt<kIq3S>() && prepare_fmt<kIq2Xxs>() && prepare_fmt<kIq2Xs>() && prepare_fmt<kIq2S>();
}

}  // namespace fnb

extern "C" int32_t fnb_expert_gate_up_rows_iq3_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                   const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                   int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<fnb::kIq3Xxs>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_iq3_s(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                 const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                 int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<fnb::kIq3S>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_iq2_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                   const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                   int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<fnb::kIq2Xxs>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_iq2_xs(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                  const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                  int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<fnb::kIq2Xs>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_iq2_s(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                 const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                 int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<fnb::kIq2S>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}
