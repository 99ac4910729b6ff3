// Token-embedding get_rows: out[t] = dequantised row ids[t] of a quantised table, F32.
//
// HBM-bound and write-dominated: per token 1152 (Q4_K) / 784 (IQ3_XXS) / 2176 (Q8_0) bytes of table are read
// at a random row and 8192 bytes written (cols = 2048).  The decode is a few integer ops and one or two
// separately rounded F32 products per value, so results are bit-exact with the CPU row decoders.
//
// Layout in HBM: table [n_vocab][cols / block_values] blocks, rows contiguous (ggml's layout); ids I32 [rows];
// out F32 [rows][cols].
//
// Work decomposition: a warp owns a token.  All of the row's table bytes are requested before the first
// value is decoded (Q4_K: per super-block one broadcast 16-byte header load and one coalesced 128-byte load
// of the nibbles, 8 super-blocks in flight per lane; IQ3_XXS: the 784-byte row is staged into the warp's
// shared-memory slot by cp.async because its 98-byte super-blocks are only 2-byte aligned).  Every
// store instruction of the warp writes whole 128-byte lines with the streaming hint, so the 126 MB L2 keeps
// the table rather than the output.  The IQ3_XXS codebook (256 x 4 magnitudes, as floats) and its sign table are
// expanded into shared memory once per CTA; the CTAs are persistent (grid = SM count x resident CTAs) so that cost and
// the id fetch are amortised over many rows.
#include "common.cuh"
#include "norm_math.cuh"

namespace fnb {
namespace {

constexpr int kWarpsPerCta = 8;

__constant__ uint16_t c_iq3xxs_grid_packed[256] = {
#include "iq3xxs_grid_packed.inc"
};

// returns the row's table offset, or -1 after recording a bad id
__device__ __forceinline__ int64_t row_of(const int32_t * __restrict__ ids, int64_t t, int64_t n_vocab,
                                          uint32_t * err, int lane) {
    const int32_t id = __ldg(ids + t);
    if (id < 0 || id >= n_vocab) {
        if (lane == 0 && err != nullptr) atomicOr(err, FNB_ERR_TOKEN);
        return -1;
    }
    return id;
}

// ---- Q4_K ------------------------------------------------------------------------------------------------
// super-block: fp16 d, fp16 dmin, 12 bytes of 6-bit scales/mins, 128 bytes of nibbles; value = d*sc*q - dmin*m.
// Lane i takes nibble word i: bytes 4(i%8)..+3 of 64-value group i/8, whose low nibbles are outputs
// 64(i/8) + 4(i%8) .. +3 and whose high nibbles are the same positions 32 further on.
__device__ __forceinline__ void scale_min_k4(int is, uint32_t s0, uint32_t s1, uint32_t s2, float * sc, float * mn) {
    const int sh = 8 * (is & 3);
    const uint32_t a = (s0 >> sh) & 0xffu, b = (s1 >> sh) & 0xffu, c = (s2 >> sh) & 0xffu;
    uint32_t sv, mv;
    if (is < 4) {
        sv = a & 63u;
        mv = b & 63u;
    } else {
        sv = (c & 0x0fu) | ((a >> 6) << 4);
        mv = (c >> 4) | ((b >> 6) << 4);
    }
    *sc = float(sv);
    *mn = float(mv);
}

// one super-block: hdr its first 16 bytes (d, dmin, scales), w this lane's nibble word; lo: outputs 64 grp + 4 pos ..
// + 3 of the super-block, hi: the same positions 32 further on
__device__ __forceinline__ void q4_k_values(uint4 hdr, uint32_t w, int grp, float4 & lo, float4 & hi) {
    const float d = f16_bits_to_f32(uint16_t(hdr.x & 0xffffu));
    const float dmin = f16_bits_to_f32(uint16_t(hdr.x >> 16));
    float sc, mn;
    scale_min_k4(2 * grp, hdr.y, hdr.z, hdr.w, &sc, &mn);
    const float d1 = __fmul_rn(d, sc), m1 = __fmul_rn(dmin, mn);
    scale_min_k4(2 * grp + 1, hdr.y, hdr.z, hdr.w, &sc, &mn);
    const float d2 = __fmul_rn(d, sc), m2 = __fmul_rn(dmin, mn);
    lo.x = __fsub_rn(__fmul_rn(d1, float(w & 15u)), m1);
    lo.y = __fsub_rn(__fmul_rn(d1, float((w >> 8) & 15u)), m1);
    lo.z = __fsub_rn(__fmul_rn(d1, float((w >> 16) & 15u)), m1);
    lo.w = __fsub_rn(__fmul_rn(d1, float((w >> 24) & 15u)), m1);
    hi.x = __fsub_rn(__fmul_rn(d2, float((w >> 4) & 15u)), m2);
    hi.y = __fsub_rn(__fmul_rn(d2, float((w >> 12) & 15u)), m2);
    hi.z = __fsub_rn(__fmul_rn(d2, float((w >> 20) & 15u)), m2);
    hi.w = __fsub_rn(__fmul_rn(d2, float(w >> 28)), m2);
}
__device__ __forceinline__ void q4_k_finish(uint4 hdr, uint32_t w, float * dst256, int grp, int pos) {
    float4 lo, hi;
    q4_k_values(hdr, w, grp, lo, hi);
    float4 * o = reinterpret_cast<float4 *>(dst256 + grp * 64) + pos;
    st_stream(o, lo);
    st_stream(o + 8, hi);
}

// Rows of 8 super-blocks (2048 columns, 1152 bytes): the whole row is fetched with three 128-bit loads per lane one
// row ahead of its decode and parked in the warp's shared-memory slot (ids run two rows ahead), so no lane ever
// waits on a global load it has just issued.
constexpr int kQ4kRowBytes = 8 * 144;
// CTAs of a staged kernel resident per SM (the launch bound holds registers to that) and CTAs LAUNCHED per SM.
// Measured at 65536 rows: a grid of exactly one resident wave (6 per SM, 11 rows per warp) ran at 83 % of the HBM
// roofline, 8 per SM at 87 %, 24 at 91-93 %, 32 and more at 93-95 %: SMs do not drain their share of rows at the
// same rate, and only the hardware's CTA dispatch evens that out.  At 32 per SM a warp still decodes two rows or
// more, so the row fetched ahead keeps paying.
constexpr int kStagedCtasPerSm = 6;
constexpr int kStagedGridPerSm = 32;
__device__ __forceinline__ void q4_k_fetch_row(const uint8_t * __restrict__ table, int32_t id, int lane, uint4 (&r)[3]) {
    const uint4 * p = reinterpret_cast<const uint4 *>(table + int64_t(id) * kQ4kRowBytes);
    r[0] = __ldg(p + lane);
    r[1] = __ldg(p + 32 + lane);
    r[2] = lane < kQ4kRowBytes / 16 - 64 ? __ldg(p + 64 + lane) : make_uint4(0u, 0u, 0u, 0u);
}
__global__ void __launch_bounds__(kWarpsPerCta * 32, kStagedCtasPerSm)
    get_rows_q4_k_staged_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                                float * __restrict__ out, uint32_t * err, int64_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) uint8_t s_rows[kWarpsPerCta][kQ4kRowBytes];
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int grp = lane >> 3, pos = lane & 7;
    uint8_t * buf = s_rows[threadIdx.x >> 5];
    auto valid = [&](int32_t id) { return id >= 0 && id < n_vocab; };

    int32_t id = warp < rows ? __ldg(ids + warp) : -1;
    int32_t id_next = warp + n_warps < rows ? __ldg(ids + warp + n_warps) : -1;
    uint4 r[3] = {};
    if (valid(id)) q4_k_fetch_row(table, id, lane, r);
    for (int64_t t = warp; t < rows; t += n_warps) {
        const bool ok = valid(id);
        if (ok) {
            reinterpret_cast<uint4 *>(buf)[lane] = r[0];
            reinterpret_cast<uint4 *>(buf)[32 + lane] = r[1];
            if (lane < kQ4kRowBytes / 16 - 64) reinterpret_cast<uint4 *>(buf)[64 + lane] = r[2];
        } else if (lane == 0 && err != nullptr) {
            atomicOr(err, FNB_ERR_TOKEN);
        }
        __syncwarp();
        const int64_t t2 = t + 2 * n_warps;
        const int32_t id_after = t2 < rows ? __ldg(ids + t2) : -1;
        if (valid(id_next)) q4_k_fetch_row(table, id_next, lane, r);
        if (ok) {
            float * dst = out + t * 2048;
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const uint8_t * blk = buf + 144 * sb;
                q4_k_finish(*reinterpret_cast<const uint4 *>(blk), reinterpret_cast<const uint32_t *>(blk + 16)[lane],
                            dst + 256 * sb, grp, pos);
            }
        }
        __syncwarp();  // every lane is done with the slot before the next row overwrites it
        id = id_next;
        id_next = id_after;
    }
}

// get_rows and the RMSNorm that follows it in one pass: the decoded row stays in the warp's registers (64 values a
// lane), is written out, summed (F32 squares in double, as rms_norm.cu), scaled, weighted and written again.  Against
// the two kernels it saves the second kernel's read of the row: 17.5 KB a token instead of 25.7 KB.  The row is the
// same bytes as fnb_get_rows_q4_k writes; the normalised row is fnb_rms_norm_f32's up to the order of the double sum.
constexpr int kFusedCtasPerSm = 2;  // 16 warps an SM at up to 128 registers
constexpr int kFusedGridPerSm = 16;
__global__ void __launch_bounds__(kWarpsPerCta * 32, kFusedCtasPerSm)
    get_rows_norm_q4_k_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                              const float * __restrict__ w, float eps, float * __restrict__ out, float * __restrict__ normed,
                              uint32_t * err, int64_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) uint8_t s_rows[kWarpsPerCta][kQ4kRowBytes];
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int grp = lane >> 3, pos = lane & 7;
    uint8_t * buf = s_rows[threadIdx.x >> 5];
    const float4 * w4 = reinterpret_cast<const float4 *>(w);
    auto valid = [&](int32_t id) { return id >= 0 && id < n_vocab; };

    int32_t id = warp < rows ? __ldg(ids + warp) : -1;
    int32_t id_next = warp + n_warps < rows ? __ldg(ids + warp + n_warps) : -1;
    uint4 r[3] = {};
    if (valid(id)) q4_k_fetch_row(table, id, lane, r);
    for (int64_t t = warp; t < rows; t += n_warps) {
        const bool ok = valid(id);
        if (ok) {
            reinterpret_cast<uint4 *>(buf)[lane] = r[0];
            reinterpret_cast<uint4 *>(buf)[32 + lane] = r[1];
            if (lane < kQ4kRowBytes / 16 - 64) reinterpret_cast<uint4 *>(buf)[64 + lane] = r[2];
        } else if (lane == 0 && err != nullptr) {
            atomicOr(err, FNB_ERR_TOKEN);
        }
        __syncwarp();
        const int64_t t2 = t + 2 * n_warps;
        const int32_t id_after = t2 < rows ? __ldg(ids + t2) : -1;
        if (valid(id_next)) q4_k_fetch_row(table, id_next, lane, r);
        if (ok) {
            float4 lo[8], hi[8];
            double acc = 0.0;
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const uint8_t * blk = buf + 144 * sb;
                q4_k_values(*reinterpret_cast<const uint4 *>(blk), reinterpret_cast<const uint32_t *>(blk + 16)[lane], grp, lo[sb], hi[sb]);
                float4 * o = reinterpret_cast<float4 *>(out + t * 2048 + 256 * sb + grp * 64) + pos;
                st_stream(o, lo[sb]);
                st_stream(o + 8, hi[sb]);
                acc = sq_acc(sq_acc(sq_acc(sq_acc(acc, lo[sb].x), lo[sb].y), lo[sb].z), lo[sb].w);
                acc = sq_acc(sq_acc(sq_acc(sq_acc(acc, hi[sb].x), hi[sb].y), hi[sb].z), hi[sb].w);
            }
            const float scale = norm_scale(warp_sum_f64(acc), 2048, eps);
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const int at = (256 * sb + grp * 64) / 4 + pos;  // float4 index of lo in the row; hi is 8 further on
                float4 a = lo[sb], b = hi[sb];
                a.x = __fmul_rn(a.x, scale), a.y = __fmul_rn(a.y, scale), a.z = __fmul_rn(a.z, scale), a.w = __fmul_rn(a.w, scale);
                b.x = __fmul_rn(b.x, scale), b.y = __fmul_rn(b.y, scale), b.z = __fmul_rn(b.z, scale), b.w = __fmul_rn(b.w, scale);
                if (w != nullptr) {
                    const float4 ga = __ldg(w4 + at), gb = __ldg(w4 + at + 8);
                    a.x = __fmul_rn(a.x, ga.x), a.y = __fmul_rn(a.y, ga.y), a.z = __fmul_rn(a.z, ga.z), a.w = __fmul_rn(a.w, ga.w);
                    b.x = __fmul_rn(b.x, gb.x), b.y = __fmul_rn(b.y, gb.y), b.z = __fmul_rn(b.z, gb.z), b.w = __fmul_rn(b.w, gb.w);
                }
                float4 * o = reinterpret_cast<float4 *>(normed + t * 2048) + at;
                st_stream(o, a);
                st_stream(o + 8, b);
            }
        }
        __syncwarp();  // every lane is done with the slot before the next row overwrites it
        id = id_next;
        id_next = id_after;
    }
}

template <int NSB>  // super-blocks per row held in flight at once
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_q4_k_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                         float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nsb = cols / 256;
    const int64_t row_bytes = int64_t(nsb) * 144;
    const int grp = lane >> 3, pos = lane & 7;

    for (int64_t t = warp; t < rows; t += n_warps) {
        const int64_t id = row_of(ids, t, n_vocab, err, lane);
        if (id < 0) continue;
        const uint8_t * row = table + id * row_bytes;
        float * dst = out + t * cols;
        for (int sb0 = 0; sb0 < nsb; sb0 += NSB) {
            uint4 hdr[NSB];
            uint32_t qw[NSB];
#pragma unroll
            for (int j = 0; j < NSB; ++j) {
                if (sb0 + j < nsb) {
                    const uint8_t * blk = row + (sb0 + j) * 144;
                    hdr[j] = __ldg(reinterpret_cast<const uint4 *>(blk));
                    qw[j] = __ldg(reinterpret_cast<const uint32_t *>(blk + 16) + lane);
                }
            }
#pragma unroll
            for (int j = 0; j < NSB; ++j) {
                if (sb0 + j < nsb) q4_k_finish(hdr[j], qw[j], dst + (sb0 + j) * 256, grp, pos);
            }
        }
    }
}

// ---- IQ3_XXS ---------------------------------------------------------------------------------------------
// super-block: fp16 d, 64 codebook indices, 8 words of {4-bit scale, 4 x 7 sign bits}; index n decodes to the four
// outputs 4n .. 4n + 3.  Lane L takes indices L and L + 32 of each super-block, so the warp's two store instructions
// per super-block each write 512 contiguous bytes (whole 32-byte sectors).
//
// What ncu showed on earlier versions shaped this one:
//   * first version (row staged in shared memory, byte codebook, lane = indices 2L and 2L + 1): 30 % issue rate at
//     65 % occupancy, stalls per issue long scoreboard 10, MIO throttle 9, short scoreboard 7; 800 warp instructions
//     per row.  Three different load structures (staged, cp.async double buffer, direct) all ran at the same 0.16 ms
//     because the limit was the STORE shape: with adjacent indices per lane every store instruction wrote half of 32
//     sectors.  Hence indices L and L + 32;
//   * no staging: the 98-byte super-blocks are 2-byte aligned, so each lane fetches exactly the pieces it needs (d,
//     its two index bytes, its two scale/sign words as halves) straight from global memory through L1, four
//     super-blocks issued before the first use, as the Q4_K kernel does;
//   * the codebook sits in shared memory as one 32-bit word of four magnitude bytes per entry; a byte becomes a
//     float with one byte permute and one exact subtraction (an earlier build kept FLOAT magnitudes, 256 x float4:
//     no conversion, but the random 128-bit lookups cost ~11 shared-memory wavefronts each and, with the stores'
//     own wavefronts, kept the load/store pipe ~70 % busy at 77 % of the HBM roofline);
//   * a sign is applied by choosing +db or -db as the multiplier ((-db) g and -(db g) are the same bits); the
//     eighth sign bit is the parity of the seven stored ones (a population count, no table).
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t * p) { return __ldg(reinterpret_cast<const uint16_t *>(p)); }
__device__ __forceinline__ uint32_t ldg_u8(const uint8_t * p) { return __ldg(p); }

// magnitude byte J of a codebook word as a float: 0x4B0000bb is 2^23 + bb exactly, so one byte permute and one
// exact subtraction convert it
template <int J>
__device__ __forceinline__ float grid_byte_f32(uint32_t g) {
    return __fadd_rn(__uint_as_float(__byte_perm(g, 0x4B000000u, 0x7540u + J)), -8388608.0f);
}
// one index: aux is its 32-value group's scale/sign word, n the index within the super-block
__device__ __forceinline__ float4 iq3_decode(float d, uint32_t q, uint32_t aux, int n, const uint32_t * s_grid) {
    const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, float(aux >> 28))), 0.5f);
    const float nb = -db;
    const uint32_t s7 = (aux >> (7 * ((n >> 1) & 3))) & 127u;            // seven stored sign bits,
    const uint32_t sg = (s7 | ((__popc(s7) & 1u) << 7)) >> (4 * (n & 1));  // the eighth is their parity
    const uint32_t g = s_grid[q];
    return make_float4(__fmul_rn((sg & 1u) ? nb : db, grid_byte_f32<0>(g)), __fmul_rn((sg & 2u) ? nb : db, grid_byte_f32<1>(g)),
                       __fmul_rn((sg & 4u) ? nb : db, grid_byte_f32<2>(g)), __fmul_rn((sg & 8u) ? nb : db, grid_byte_f32<3>(g)));
}

struct iq3_sb_regs {
    uint32_t dq, q0, q1, a0lo, a0hi, a1lo, a1hi;
};
__device__ __forceinline__ void iq3_load(iq3_sb_regs & r, const uint8_t * blk, int lane) {
    const int o_aux = 66 + 4 * (lane >> 3);
    r.dq = ldg_u16(blk);
    r.q0 = ldg_u8(blk + 2 + lane);
    r.q1 = ldg_u8(blk + 34 + lane);
    r.a0lo = ldg_u16(blk + o_aux);
    r.a0hi = ldg_u16(blk + o_aux + 2);
    r.a1lo = ldg_u16(blk + o_aux + 16);
    r.a1hi = ldg_u16(blk + o_aux + 18);
}
__device__ __forceinline__ void iq3_finish(const iq3_sb_regs & r, float * dst256, int lane, const uint32_t * s_grid) {
    const float d = f16_bits_to_f32(uint16_t(r.dq));
    float4 * o = reinterpret_cast<float4 *>(dst256) + lane;
    st_stream(o, iq3_decode(d, r.q0, r.a0lo | (r.a0hi << 16), lane, s_grid));
    st_stream(o + 32, iq3_decode(d, r.q1, r.a1lo | (r.a1hi << 16), lane, s_grid));  // n = lane + 32: same parity bits
}

// any column count that is a multiple of 256 (2048 columns take the staged kernel after this one)
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_iq3_xxs_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                            float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    // The codebook's four magnitudes per entry as BYTES (one 32-bit word per entry): a lookup is a 32-bit shared
    // load, where 32 random entries collide on a bank about three deep.  As float4 entries (one 128-bit load, no
    // conversion) the same lookup took about eleven wavefronts and the kernel ran against the shared-memory pipe.
    __shared__ uint32_t s_grid[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint32_t c = c_iq3xxs_grid_packed[i];
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            w |= (lvl == 7u ? 62u : 4u + 8u * lvl) << (8 * j);
        }
        s_grid[i] = w;
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nsb = cols / 256;
    const int64_t row_bytes = int64_t(nsb) * 98;

    int32_t id_next = warp < rows ? __ldg(ids + warp) : 0;  // ids run one row ahead of the decode
    for (int64_t t = warp; t < rows; t += n_warps) {
        const int32_t id = id_next;
        if (t + n_warps < rows) id_next = __ldg(ids + t + n_warps);
        if (id < 0 || id >= n_vocab) {
            if (lane == 0 && err != nullptr) atomicOr(err, FNB_ERR_TOKEN);
            continue;
        }
        const uint8_t * row = table + int64_t(id) * row_bytes;
        float * dst = out + t * cols;
        for (int sb = 0; sb < nsb; ++sb) {
            iq3_sb_regs r;
            iq3_load(r, row + sb * 98, lane);
            iq3_finish(r, dst + sb * 256, lane, s_grid);
        }
    }
}

// Rows of 8 super-blocks (2048 columns) are 784 bytes, a multiple of 16, and start 16-byte aligned: the whole row is
// fetched with two 128-bit loads per lane ONE ROW AHEAD of its decode (held in eight registers), then parked in the
// warp's own shared-memory slot, from which every lane picks its pieces.  With per-lane 1- and 2-byte global loads
// issued just before their use the kernel sat on global-load latency (ncu: 20 long-scoreboard stall cycles per issue,
// 45 % issue rate at 85 % occupancy).
constexpr int kIq3RowBytes = 8 * 98;
__device__ __forceinline__ void iq3_fetch_row(const uint8_t * __restrict__ table, int32_t id, int lane, uint4 & a, uint4 & b) {
    const uint4 * p = reinterpret_cast<const uint4 *>(table + int64_t(id) * kIq3RowBytes);
    a = __ldg(p + lane);
    b = lane < kIq3RowBytes / 16 - 32 ? __ldg(p + 32 + lane) : make_uint4(0u, 0u, 0u, 0u);
}
// super-block SB of the staged row: this lane's outputs 4 lane .. + 3 (lo) and 128 further on (hi)
template <int SB>
__device__ __forceinline__ void iq3_values_staged(const uint8_t * buf, int lane, const uint32_t * s_grid, float4 & lo, float4 & hi) {
    const uint8_t * blk = buf + 98 * SB;
    const int o_aux = 66 + 4 * (lane >> 3);
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk));
    const uint32_t q0 = blk[2 + lane], q1 = blk[34 + lane];
    uint32_t a0, a1;
    if constexpr ((SB & 1) != 0) {  // 98 SB + 66 is a multiple of 4: the scale/sign words are aligned
        a0 = *reinterpret_cast<const uint32_t *>(blk + o_aux);
        a1 = *reinterpret_cast<const uint32_t *>(blk + o_aux + 16);
    } else {
        const uint16_t * h = reinterpret_cast<const uint16_t *>(blk + o_aux);
        a0 = uint32_t(h[0]) | (uint32_t(h[1]) << 16);
        a1 = uint32_t(h[8]) | (uint32_t(h[9]) << 16);
    }
    lo = iq3_decode(d, q0, a0, lane, s_grid);
    hi = iq3_decode(d, q1, a1, lane, s_grid);  // n = lane + 32: same parity bits
}
template <int SB>
__device__ __forceinline__ void iq3_finish_staged(const uint8_t * buf, float * dst, int lane, const uint32_t * s_grid) {
    float4 lo, hi;
    iq3_values_staged<SB>(buf, lane, s_grid, lo, hi);
    float4 * o = reinterpret_cast<float4 *>(dst + 256 * SB) + lane;
    st_stream(o, lo);
    st_stream(o + 32, hi);
}
// the fused form's share of a super-block: the values kept, written out and their squares added
template <int SB>
__device__ __forceinline__ void iq3_keep_staged(const uint8_t * buf, float * dst, int lane, const uint32_t * s_grid, float4 (&lo)[8],
                                                float4 (&hi)[8], double & acc) {
    iq3_values_staged<SB>(buf, lane, s_grid, lo[SB], hi[SB]);
    float4 * o = reinterpret_cast<float4 *>(dst + 256 * SB) + lane;
    st_stream(o, lo[SB]);
    st_stream(o + 32, hi[SB]);
    acc = sq_acc(sq_acc(sq_acc(sq_acc(acc, lo[SB].x), lo[SB].y), lo[SB].z), lo[SB].w);
    acc = sq_acc(sq_acc(sq_acc(sq_acc(acc, hi[SB].x), hi[SB].y), hi[SB].z), hi[SB].w);
}
__global__ void __launch_bounds__(kWarpsPerCta * 32, kStagedCtasPerSm)
    get_rows_iq3_xxs_staged_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                                   float * __restrict__ out, uint32_t * err, int64_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t s_grid[256];
    __shared__ __align__(16) uint8_t s_rows[kWarpsPerCta][kIq3RowBytes];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint32_t c = c_iq3xxs_grid_packed[i];
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            w |= (lvl == 7u ? 62u : 4u + 8u * lvl) << (8 * j);
        }
        s_grid[i] = w;
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    uint8_t * buf = s_rows[threadIdx.x >> 5];
    auto valid = [&](int32_t id) { return id >= 0 && id < n_vocab; };

    // ids run two rows ahead of the decode, row bytes one
    int32_t id = warp < rows ? __ldg(ids + warp) : -1;
    int32_t id_next = warp + n_warps < rows ? __ldg(ids + warp + n_warps) : -1;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (valid(id)) iq3_fetch_row(table, id, lane, a, b);
    for (int64_t t = warp; t < rows; t += n_warps) {
        const bool ok = valid(id);
        if (ok) {
            reinterpret_cast<uint4 *>(buf)[lane] = a;
            if (lane < kIq3RowBytes / 16 - 32) reinterpret_cast<uint4 *>(buf)[32 + lane] = b;
        } else if (lane == 0 && err != nullptr) {
            atomicOr(err, FNB_ERR_TOKEN);
        }
        __syncwarp();
        const int64_t t2 = t + 2 * n_warps;
        const int32_t id_after = t2 < rows ? __ldg(ids + t2) : -1;
        if (valid(id_next)) iq3_fetch_row(table, id_next, lane, a, b);  // (an id past the end is -1: nothing fetched)
        if (ok) {
            float * dst = out + t * 2048;
            iq3_finish_staged<0>(buf, dst, lane, s_grid);
            iq3_finish_staged<1>(buf, dst, lane, s_grid);
            iq3_finish_staged<2>(buf, dst, lane, s_grid);
            iq3_finish_staged<3>(buf, dst, lane, s_grid);
            iq3_finish_staged<4>(buf, dst, lane, s_grid);
            iq3_finish_staged<5>(buf, dst, lane, s_grid);
            iq3_finish_staged<6>(buf, dst, lane, s_grid);
            iq3_finish_staged<7>(buf, dst, lane, s_grid);
        }
        __syncwarp();  // every lane is done with the slot before the next row overwrites it
        id = id_next;
        id_next = id_after;
    }
}

// the IQ3_XXS form of get_rows_norm_q4_k_kernel
__global__ void __launch_bounds__(kWarpsPerCta * 32, kFusedCtasPerSm)
    get_rows_norm_iq3_xxs_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                                 const float * __restrict__ w, float eps, float * __restrict__ out, float * __restrict__ normed,
                                 uint32_t * err, int64_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t s_grid[256];
    __shared__ __align__(16) uint8_t s_rows[kWarpsPerCta][kIq3RowBytes];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint32_t c = c_iq3xxs_grid_packed[i];
        uint32_t g = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            g |= (lvl == 7u ? 62u : 4u + 8u * lvl) << (8 * j);
        }
        s_grid[i] = g;
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    uint8_t * buf = s_rows[threadIdx.x >> 5];
    const float4 * w4 = reinterpret_cast<const float4 *>(w);
    auto valid = [&](int32_t id) { return id >= 0 && id < n_vocab; };

    int32_t id = warp < rows ? __ldg(ids + warp) : -1;
    int32_t id_next = warp + n_warps < rows ? __ldg(ids + warp + n_warps) : -1;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (valid(id)) iq3_fetch_row(table, id, lane, a, b);
    for (int64_t t = warp; t < rows; t += n_warps) {
        const bool ok = valid(id);
        if (ok) {
            reinterpret_cast<uint4 *>(buf)[lane] = a;
            if (lane < kIq3RowBytes / 16 - 32) reinterpret_cast<uint4 *>(buf)[32 + lane] = b;
        } else if (lane == 0 && err != nullptr) {
            atomicOr(err, FNB_ERR_TOKEN);
        }
        __syncwarp();
        const int64_t t2 = t + 2 * n_warps;
        const int32_t id_after = t2 < rows ? __ldg(ids + t2) : -1;
        if (valid(id_next)) iq3_fetch_row(table, id_next, lane, a, b);
        if (ok) {
            float * dst = out + t * 2048;
            float4 lo[8], hi[8];
            double acc = 0.0;
            iq3_keep_staged<0>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<1>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<2>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<3>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<4>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<5>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<6>(buf, dst, lane, s_grid, lo, hi, acc);
            iq3_keep_staged<7>(buf, dst, lane, s_grid, lo, hi, acc);
            const float scale = norm_scale(warp_sum_f64(acc), 2048, eps);
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const int at = 64 * sb + lane;  // float4 index of lo in the row; hi is 32 further on
                float4 x = lo[sb], y = hi[sb];
                x.x = __fmul_rn(x.x, scale), x.y = __fmul_rn(x.y, scale), x.z = __fmul_rn(x.z, scale), x.w = __fmul_rn(x.w, scale);
                y.x = __fmul_rn(y.x, scale), y.y = __fmul_rn(y.y, scale), y.z = __fmul_rn(y.z, scale), y.w = __fmul_rn(y.w, scale);
                if (w != nullptr) {
                    const float4 gx = __ldg(w4 + at), gy = __ldg(w4 + at + 32);
                    x.x = __fmul_rn(x.x, gx.x), x.y = __fmul_rn(x.y, gx.y), x.z = __fmul_rn(x.z, gx.z), x.w = __fmul_rn(x.w, gx.w);
                    y.x = __fmul_rn(y.x, gy.x), y.y = __fmul_rn(y.y, gy.y), y.z = __fmul_rn(y.z, gy.z), y.w = __fmul_rn(y.w, gy.w);
                }
                float4 * o = reinterpret_cast<float4 *>(normed + t * 2048) + at;
                st_stream(o, x);
                st_stream(o + 32, y);
            }
        }
        __syncwarp();  // every lane is done with the slot before the next row overwrites it
        id = id_next;
        id_next = id_after;
    }
}

// ---- Q8_0 ------------------------------------------------------------------------------------------------
// block: fp16 d, 32 int8; value = q * d.  A lane decodes 4 codes of each of the row's blocks it visits; blocks
// are 34 bytes (2-byte aligned), so codes are fetched as two 16-bit loads from L1/L2.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_q8_0_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                         float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nb = cols / 32;
    const int64_t row_bytes = int64_t(nb) * 34;
    for (int64_t t = warp; t < rows; t += n_warps) {
        const int64_t id = row_of(ids, t, n_vocab, err, lane);
        if (id < 0) continue;
        const uint8_t * row = table + id * row_bytes;
        float * dst = out + t * cols;
        // 8 lanes per block, 4 blocks per warp trip
        for (int b0 = 0; b0 < nb; b0 += 4) {
            const int b = b0 + (lane >> 3);
            if (b < nb) {
                const uint16_t * blk = reinterpret_cast<const uint16_t *>(row + b * 34);
                const float d = f16_bits_to_f32(__ldg(blk));
                const uint32_t w = uint32_t(__ldg(blk + 1 + 2 * (lane & 7))) | (uint32_t(__ldg(blk + 2 + 2 * (lane & 7))) << 16);
                float4 o;
                o.x = __fmul_rn(float(int8_t(w & 0xffu)), d);
                o.y = __fmul_rn(float(int8_t((w >> 8) & 0xffu)), d);
                o.z = __fmul_rn(float(int8_t((w >> 16) & 0xffu)), d);
                o.w = __fmul_rn(float(int8_t(w >> 24)), d);
                st_stream(reinterpret_cast<float4 *>(dst + b * 32) + (lane & 7), o);
            }
        }
    }
}

bool common_ok(const void * table, int64_t n_vocab, const int32_t * ids, float * out, uint32_t * err, int64_t rows,
               int32_t cols, int block_values, int block_bytes, int row_align) {
    if (!ok_ptr(table, 16) || !ok_ptr(ids, 4) || !ok_ptr(out, 16) || !ok_opt(err, 4)) return false;
    if (rows < 1 || rows > INT32_MAX || n_vocab < 1 || n_vocab > INT32_MAX) return false;
    if (cols < block_values || cols > 16384 || cols % block_values != 0) return false;
    return (int64_t(cols / block_values) * block_bytes) % row_align == 0;
}

int persistent_grid(int64_t rows, int ctas_per_sm) {
    return grid_for((rows + kWarpsPerCta - 1) / kWarpsPerCta, ctas_per_sm);
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_get_rows_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                                     uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 256, 144, 16)) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(table);
    if (cols == 2048) {
        launch_pdl(get_rows_q4_k_staged_kernel, persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s, tb, n_vocab, ids, out, err, rows);
    } else {
        get_rows_q4_k_kernel<8><<<persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    }
    return launch_status();
}

extern "C" int32_t fnb_get_rows_rms_norm_q4_k(const void * table, int64_t n_vocab, const int32_t * ids, const float * w, float eps,
                                              float * out, float * normed, uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 256, 144, 16)) return FNB_REJECTED;
    if (!ok_ptr(normed, 16) || !ok_opt(w, 16) || !(eps >= 0.0f) || normed == out) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(table);
    if (cols == 2048) {
        launch_pdl(get_rows_norm_q4_k_kernel, persistent_grid(rows, kFusedGridPerSm), kWarpsPerCta * 32, 0, s, tb, n_vocab, ids, w, eps,
                   out, normed, err, rows);
        return launch_status();
    }
    // other widths: the two kernels one after the other.  A row whose id is refused is left unwritten by the first
    // and normalised from whatever `out` held by the second, as with the two entry points called in turn.
    get_rows_q4_k_kernel<8><<<persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    if (cudaPeekAtLastError() != cudaSuccess) return FNB_LAUNCH_FAILED;
    return rms_norm_launch(out, w, eps, normed, rows, cols, s);
}

extern "C" int32_t fnb_get_rows_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                                        uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 256, 98, 2)) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(table);
    if (cols == 2048) {
        launch_pdl(get_rows_iq3_xxs_staged_kernel, persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s, tb, n_vocab, ids, out, err, rows);
    } else {
        get_rows_iq3_xxs_kernel<<<persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    }
    return launch_status();
}

extern "C" int32_t fnb_get_rows_rms_norm_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, const float * w, float eps,
                                                 float * out, float * normed, uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 256, 98, 2)) return FNB_REJECTED;
    if (!ok_ptr(normed, 16) || !ok_opt(w, 16) || !(eps >= 0.0f) || normed == out) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(table);
    if (cols == 2048) {
        launch_pdl(get_rows_norm_iq3_xxs_kernel, persistent_grid(rows, kFusedGridPerSm), kWarpsPerCta * 32, 0, s, tb, n_vocab, ids, w,
                   eps, out, normed, err, rows);
        return launch_status();
    }
    get_rows_iq3_xxs_kernel<<<persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    if (cudaPeekAtLastError() != cudaSuccess) return FNB_LAUNCH_FAILED;
    return rms_norm_launch(out, w, eps, normed, rows, cols, s);
}

extern "C" int32_t fnb_get_rows_q8_0(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                                     uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 32, 34, 2)) return FNB_REJECTED;
    get_rows_q8_0_kernel<<<persistent_grid(rows, kStagedGridPerSm), kWarpsPerCta * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(table), n_vocab, ids, out, err, rows, cols);
    return launch_status();
}

extern "C" int64_t fnb_check_tokens(const int32_t * ids_host, int64_t rows, int64_t n_vocab) {
    if (ids_host == nullptr || rows < 0) return -1;
    for (int64_t t = 0; t < rows; ++t) {
        if (ids_host[t] < 0 || ids_host[t] >= n_vocab) return t + 1;
    }
    return 0;
}
