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

// S: ggml IQ3_S rows (110-byte super-blocks: d, qs[64], qh[8], signs[32], scales[4]; 512-entry codebook, plain sign
// bits, one 4-bit scale per 32 values) instead of IQ3_XXS (98 bytes: d, qs[64], eight words of 4 x 7-bit sign index +
// 4-bit scale; 256-entry codebook)
template <bool S>
struct shape {
    static constexpr int kBlock = S ? 110 : 98;
    // a slot: ten blocks and 12 bytes of source offset, rounded up so that the eight slots start in different banks
    static constexpr int kSlot = S ? 1136 : 1008;
    static constexpr int kUnit = 8 * kSlot;           // four gate rows, then four up rows
    static constexpr int kWarpStage = 2 * kUnit;      // two units: the one computed on and the one in flight
    static constexpr int kSpan = 4 * kWholeRowBlocks * kBlock + 16;  // four whole rows, back to back as in global memory
    static constexpr int kGridEntries = S ? 512 : 256;
    static constexpr int kGridBytes = kGridEntries * kGridCopies * 4;
    static constexpr int kSignBytes = S ? 0 : 128 * kSignCopies * 8;  // IQ3_S's sign bits need no table
    static constexpr int kTableBytes = kGridBytes + kSignBytes;
    static_assert(2 * kSpan <= kUnit, "two spans fit a unit");
};
constexpr size_t kSmemLimit = 224 * 1024;            // one CTA an SM (227 KB less the static arrays)
constexpr int kGridPerSm = FNB_GU_IQ3_GRID;

__constant__ uint16_t c_grid_packed[256] = {
#include "iq3xxs_grid_packed.inc"
};
__constant__ uint16_t c_grid3s_packed[512] = {
#include "iq3s_grid_packed.inc"
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
template <bool S>
__device__ __forceinline__ const uint8_t * chunk_src(const uint8_t * mat, int64_t row_bytes, int64_t r, int64_t r1, int chunk) {
    return mat + (r < r1 ? r : r1 - 1) * row_bytes + int64_t(chunk) * (kChunkBlocks * shape<S>::kBlock);
}

template <bool S>
__device__ __forceinline__ void stage_unit(uint32_t buf_sm, const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up,
                                           int64_t row_bytes, int64_t r4, int64_t r1, int chunk, int bytes, int lane) {
#pragma unroll
    for (int slot = 0; slot < 8; ++slot) {
        stage_span(buf_sm + slot * shape<S>::kSlot, chunk_src<S>(slot < 4 ? gate : up, row_bytes, r4 + (slot & 3), r1, chunk), bytes,
                   lane);
    }
    cp_async_commit();
}

// rows of up to ten super-blocks: the quad's four gate rows are one contiguous span of the matrix, its up rows another
template <bool S>
__device__ __forceinline__ void stage_unit_whole(uint32_t buf_sm, const uint8_t * __restrict__ gate,
                                                 const uint8_t * __restrict__ up, int64_t row_bytes, int64_t r4, int64_t r1,
                                                 int lane) {
    const int rows = r1 - r4 < 4 ? int(r1 - r4) : 4;  // a ragged last quad leaves its missing rows' bytes as they were
    stage_span(buf_sm, gate + r4 * row_bytes, rows * int(row_bytes), lane);
    stage_span(buf_sm + shape<S>::kSpan, up + r4 * row_bytes, rows * int(row_bytes), lane);
    cp_async_commit();
}

// one staged unit (n_blk super-blocks of the lane's row, x) against the window: acc[t][0 / 1] are AVX2 lanes 2 k, 2 k + 1
template <int NT, bool WRAP, bool S>
__device__ __forceinline__ void dot_unit(const uint8_t * x, int n_blk, const uint8_t * codes_sm, const float * d_sm, int nb,
                                         int blk0, int k, const uint32_t * grid_lane, const uint2 * sign_lane, float (&acc)[NT][2]) {
    const int sh7 = 7 * k;
#pragma unroll 1
    for (int i = 0; i < n_blk; ++i, x += shape<S>::kBlock) {
        const float dx = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(x));
        int a0[NT], a1[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) a0[t] = 0, a1[t] = 0;
        const uint8_t * y0 = codes_sm + size_t(blk0 + i) * 256 + 16 * k;
        uint4 y4[NT];
#pragma unroll
        for (int grp = 0; grp < 8; ++grp) {
            const uint32_t h = *reinterpret_cast<const uint16_t *>(x + 2 + 8 * grp + 2 * k);  // index bytes 2 k, 2 k + 1
            uint32_t e0 = h & 0xffu, e1 = h >> 8, m0, m1;
            int sc;
            if (S) {
                // ninth index bits 2 k, 2 k + 1 of the group's qh byte; sign byte k of the group's four (bit i: value
                // 8 k + i); the group's nibble of the scale byte it shares with its neighbour
                const uint32_t hb = uint32_t(x[66 + grp]) >> (2 * k);
                e0 |= (hb & 1u) << 8, e1 |= (hb & 2u) << 7;
                const uint32_t sb = x[74 + 4 * grp + k];
                m0 = spread_msb((sb & 15u) * 0x10204080u), m1 = spread_msb((sb >> 4) * 0x10204080u);
                const uint32_t s = x[106 + (grp >> 1)];
                sc = int(2u * ((grp & 1) ? s >> 4 : s & 15u) + 1u);
            } else {
                // the group's sign / scale word (2-byte aligned), read by each of the row's four lanes: handing it round
                // by shuffles from the lane that loaded it was slower (0.144 against 0.138 ms at a window of one row)
                const uint16_t * pg = reinterpret_cast<const uint16_t *>(x + 66 + 4 * grp);
                const uint32_t w = uint32_t(pg[0]) | (uint32_t(pg[1]) << 16);
                // the group's sign index k -> its eight byte masks; computing them here (mask, popc for the parity, two
                // multiplies, two permutes) instead of the lookup: 0.150 against 0.138 ms at a window of one row
                const uint2 sg = sign_lane[((w >> sh7) & 127u) * kSignCopies];
                m0 = sg.x, m1 = sg.y;
                sc = int(2u * (w >> 28) + 1u);
            }
            const uint32_t c0 = grid_lane[e0 * kGridCopies], c1 = grid_lane[e1 * kGridCopies];
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

template <int NT, bool WRAP, bool S>
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
        stage_unit_whole<S>(stage_sm, gate, up, row_bytes, r0 + 4 * q, r1, lane);
    } else {
        stage_unit<S>(stage_sm, gate, up, row_bytes, r0 + 4 * q, r1, 0, blocks_of(0) * shape<S>::kBlock, lane);
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
            const uint32_t next_sm = stage_sm + uint32_t((trip + 1) & 1) * shape<S>::kUnit;
            if (whole) {
                stage_unit_whole<S>(next_sm, gate, up, row_bytes, r0 + 4 * qn, r1, lane);
            } else {
                stage_unit<S>(next_sm, gate, up, row_bytes, r0 + 4 * qn, r1, cn, blocks_of(cn) * shape<S>::kBlock, lane);
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        const int64_t r = r0 + 4 * q + sub;
        {
            const uint8_t * x = stage + (trip & 1) * shape<S>::kUnit;
            if (whole) {
                const uintptr_t src = reinterpret_cast<uintptr_t>(mine + (r0 + 4 * q) * row_bytes);
                x += mat * shape<S>::kSpan + (src & 15) + sub * int(row_bytes);
            } else {
                const uintptr_t src = reinterpret_cast<uintptr_t>(chunk_src<S>(mine, row_bytes, r, r1, c));
                x += (4 * mat + sub) * shape<S>::kSlot + (src & 15);
            }
            dot_unit<NT, WRAP, S>(x, blocks_of(c), codes_sm, d_sm, nb, c * chunk_blocks, k, grid_sm + lane,
                               sign_sm + (lane & (kSignCopies - 1)), acc);
        }
        __syncwarp();  // every lane is done with the buffer the next trip's copies overwrite
        if (c == n_chunks - 1) {
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                // ggml's hsum_float_8, r_l on lane l / 2: r_l + r_(l + 4) (two lanes up), then lanes 2, 3 onto 0, 1 (one
                // lane up), then lane 1 onto lane 0 (the lane's own pair)
                float a = acc[t][0], b = acc[t][1];
                a = __fadd_rn(__shfl_down_sync(kFull, a, 2, 4), a), b = __fadd_rn(__shfl_down_sync(kFull, b, 2, 4), b);
                a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 4)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 4));
                const float dot = __fmul_rn(S ? 1.0f : 0.25f, __fadd_rn(a, b));  // the format's K, applied to the reduced sum
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

template <int NT, bool S>
__global__ void __launch_bounds__(kMaxWarps * 32)
    gate_up_iq3_kernel(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes, int nb,
                           const uint8_t * __restrict__ act, int64_t act_stride, int act_bytes, float * __restrict__ ff,
                           int64_t ff_stride, float * __restrict__ gu, int64_t r0, int64_t r1) {
    // the codebook copies, the sign masks' copies, the window's codes [NT][nb][256] and scales [NT][nb], then each
    // warp's two units
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ uint32_t s_grid[shape<S>::kGridEntries];  // the codebook's four magnitudes per entry as bytes
    uint32_t * grid_sm = reinterpret_cast<uint32_t *>(smem);
    uint2 * sign_sm = reinterpret_cast<uint2 *>(smem + shape<S>::kGridBytes);
    uint8_t * codes_sm = smem + shape<S>::kTableBytes;
    float * d_sm = reinterpret_cast<float *>(codes_sm + size_t(NT) * nb * 256);
    load_exp2_table();
    for (int i = threadIdx.x; i < shape<S>::kGridEntries; i += blockDim.x) {
        const uint32_t c = S ? c_grid3s_packed[i] : c_grid_packed[i];  // four 3-bit levels
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            // IQ3_S: 1, 3 .. 15; IQ3_XXS: 4, 12 .. 52, 62
            w |= (S ? 2u * lvl + 1u : (lvl == 7u ? 62u : 4u + 8u * lvl)) << (8 * j);
        }
        s_grid[i] = w;
    }
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
    for (int i = threadIdx.x; i < shape<S>::kGridEntries * kGridCopies; i += blockDim.x) grid_sm[i] = s_grid[i / kGridCopies];
    for (int i = threadIdx.x; i < (S ? 0 : 128 * kSignCopies); i += blockDim.x) {
        // sign index s7: values 0 .. 6 of its eight take bits 0 .. 6, value 7 their parity (ksigns_iq2xs)
        const uint32_t s7 = uint32_t(i) / kSignCopies;
        sign_sm[i] = make_uint2(spread_msb((s7 & 15u) * 0x10204080u),
                                spread_msb((s7 >> 4) * 0x10204080u + (uint32_t(__popc(s7)) << 31)));
    }
    const int wrap = __syncthreads_or(has_m128);
    uint8_t * stage = smem + shape<S>::kTableBytes + act_bytes + size_t(threadIdx.x >> 5) * shape<S>::kWarpStage;
    if (wrap) {
        run_warp<NT, true, S>(gate, up, row_bytes, nb, codes_sm, d_sm, stage, grid_sm, sign_sm, ff, ff_stride, gu, r0, r1);
    } else {
        run_warp<NT, false, S>(gate, up, row_bytes, nb, codes_sm, d_sm, stage, grid_sm, sign_sm, ff, ff_stride, gu, r0, r1);
    }
}

template <int NT, bool S>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(gate_up_iq3_kernel<NT, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemLimit)) !=
            cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

// window rows one launch can hold for nb super-blocks a row (their codes and scales and at least two warps' buffers)
template <bool S>
int window_rows(int nb) {
    const size_t per_t = size_t(nb) * 260, room = kSmemLimit - shape<S>::kTableBytes - 2 * size_t(shape<S>::kWarpStage) - 16;
    const size_t m = room / per_t;
    return int(m > size_t(kMaxT) ? size_t(kMaxT) : m);
}

template <int NT, bool S>
int32_t launch_nt(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride,
                  float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t act_bytes = (size_t(NT) * nb * 260 + 15) & ~size_t(15);
    constexpr size_t tables = shape<S>::kTableBytes, per_warp = shape<S>::kWarpStage;
    if (tables + act_bytes + per_warp > kSmemLimit) return FNB_REJECTED;
    int warps = int((kSmemLimit - tables - act_bytes) / per_warp);  // one CTA an SM, as many warps as fit
    warps = warps > kMaxWarps ? kMaxWarps : warps;
    if (!ensure_configured<NT, S>()) return FNB_LAUNCH_FAILED;
    const size_t smem = tables + act_bytes + size_t(warps) * per_warp;
    const int64_t quads = (r1 - r0 + 3) / 4;
    const int grid = grid_for((quads + warps - 1) / warps, kGridPerSm);
    gate_up_iq3_kernel<NT, S><<<grid, warps * 32, smem, s>>>(gate, up, row_bytes, nb, act, act_stride, int(act_bytes), ff,
                                                                ff_stride, gu, r0, r1);
    return launch_status();
}

template <bool S>
bool prepare_fmt() {
    return ensure_configured<1, S>() && ensure_configured<2, S>() && ensure_configured<3, S>() && ensure_configured<4, S>() &&
           ensure_configured<5, S>() && ensure_configured<6, S>() && ensure_configured<7, S>() && ensure_configured<8, S>();
}

template <bool S>
int32_t gate_up_rows(const void * gate, const void * up, int64_t row_bytes, int32_t n, const void * act, int64_t act_stride,
                     int32_t nt, float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    if (!ok_ptr(gate, 16) || !ok_ptr(up, 16) || !ok_ptr(act, 4) || !ok_ptr(ff, 4) || !ok_opt(gu, 4)) return FNB_REJECTED;
    // an even number of super-blocks a row: rows on 4-byte boundaries, which the copies into shared memory need
    if (n < 512 || n > 16384 || n % 512 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 256;
    if (row_bytes != int64_t(nb) * shape<S>::kBlock || act_stride < int64_t(nb) * 292 || act_stride % 4 != 0 || ff_stride < r1) {
        return FNB_REJECTED;
    }
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * gp = static_cast<const uint8_t *>(gate);
    const uint8_t * upp = static_cast<const uint8_t *>(up);
    const uint8_t * a = static_cast<const uint8_t *>(act);
    const int max_t = window_rows<S>(nb);
    if (max_t < 1) return FNB_REJECTED;
    // g and u of a later pass would need their own [2][m] planes: the debug output is for windows of one pass
    if (gu != nullptr && nt > max_t) return FNB_REJECTED;
    for (int t0 = 0; t0 < nt; t0 += max_t) {  // longer windows take further passes, as the reference's do above eight rows
        const int m = nt - t0 < max_t ? nt - t0 : max_t;
        const uint8_t * at = a + int64_t(t0) * act_stride;
        float * ft = ff + int64_t(t0) * ff_stride;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 2: st = launch_nt<2, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 3: st = launch_nt<3, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 4: st = launch_nt<4, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 5: st = launch_nt<5, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 6: st = launch_nt<6, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 7: st = launch_nt<7, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            default: st = launch_nt<8, S>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}

}  // namespace

bool expert_gate_up_prepare_device() { return prepare_fmt<false>() && prepare_fmt<true>(); }

}  // namespace fnb

extern "C" int32_t fnb_expert_gate_up_rows_iq3_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                   const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                   int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<false>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}

extern "C" int32_t fnb_expert_gate_up_rows_iq3_s(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                 const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                 int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    return fnb::gate_up_rows<true>(gate, up, row_bytes, n, act, act_stride, nt, ff, ff_stride, gu, r0, r1, stream);
}
