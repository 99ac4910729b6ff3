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

template <int NSB>  // super-blocks per row held in flight at once
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_q4_k_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                         float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
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
                if (sb0 + j < nsb) {
                    const float d = f16_bits_to_f32(uint16_t(hdr[j].x & 0xffffu));
                    const float dmin = f16_bits_to_f32(uint16_t(hdr[j].x >> 16));
                    float sc, mn;
                    scale_min_k4(2 * grp, hdr[j].y, hdr[j].z, hdr[j].w, &sc, &mn);
                    const float d1 = __fmul_rn(d, sc), m1 = __fmul_rn(dmin, mn);
                    scale_min_k4(2 * grp + 1, hdr[j].y, hdr[j].z, hdr[j].w, &sc, &mn);
                    const float d2 = __fmul_rn(d, sc), m2 = __fmul_rn(dmin, mn);
                    const uint32_t w = qw[j];
                    float4 lo, hi;
                    lo.x = __fsub_rn(__fmul_rn(d1, float(w & 15u)), m1);
                    lo.y = __fsub_rn(__fmul_rn(d1, float((w >> 8) & 15u)), m1);
                    lo.z = __fsub_rn(__fmul_rn(d1, float((w >> 16) & 15u)), m1);
                    lo.w = __fsub_rn(__fmul_rn(d1, float((w >> 24) & 15u)), m1);
                    hi.x = __fsub_rn(__fmul_rn(d2, float((w >> 4) & 15u)), m2);
                    hi.y = __fsub_rn(__fmul_rn(d2, float((w >> 12) & 15u)), m2);
                    hi.z = __fsub_rn(__fmul_rn(d2, float((w >> 20) & 15u)), m2);
                    hi.w = __fsub_rn(__fmul_rn(d2, float(w >> 28)), m2);
                    float4 * o = reinterpret_cast<float4 *>(dst + (sb0 + j) * 256 + grp * 64) + pos;
                    st_stream(o, lo);
                    st_stream(o + 8, hi);
                }
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
//   * the codebook is expanded to FLOAT magnitudes in shared memory (256 x float4 = 4 KiB), so an index costs one
//     128-bit shared load and no byte extraction or integer-to-float conversion;
//   * a sign is applied by choosing +db or -db as the multiplier ((-db) g and -(db g) are the same bits); the sign
//     byte comes from the 128-entry sign table in shared memory.
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t * p) { return __ldg(reinterpret_cast<const uint16_t *>(p)); }
__device__ __forceinline__ uint32_t ldg_u8(const uint8_t * p) { return __ldg(p); }

// one index: aux is its 32-value group's scale/sign word, n the index within the super-block
__device__ __forceinline__ float4 iq3_decode(float d, uint32_t q, uint32_t aux, int n, const float4 * s_grid,
                                             const uint8_t * s_signs) {
    const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, float(aux >> 28))), 0.5f);
    const float nb = -db;
    const uint32_t sg = uint32_t(s_signs[(aux >> (7 * ((n >> 1) & 3))) & 127u]) >> (4 * (n & 1));
    const float4 g = s_grid[q];
    return make_float4(__fmul_rn((sg & 1u) ? nb : db, g.x), __fmul_rn((sg & 2u) ? nb : db, g.y),
                       __fmul_rn((sg & 4u) ? nb : db, g.z), __fmul_rn((sg & 8u) ? nb : db, g.w));
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
__device__ __forceinline__ void iq3_finish(const iq3_sb_regs & r, float * dst256, int lane, const float4 * s_grid,
                                           const uint8_t * s_signs) {
    const float d = f16_bits_to_f32(uint16_t(r.dq));
    float4 * o = reinterpret_cast<float4 *>(dst256) + lane;
    st_stream(o, iq3_decode(d, r.q0, r.a0lo | (r.a0hi << 16), lane, s_grid, s_signs));
    st_stream(o + 32, iq3_decode(d, r.q1, r.a1lo | (r.a1hi << 16), lane, s_grid, s_signs));  // n = lane + 32: same parity bits
}

template <int NSB>  // super-blocks per row when known at compile time (a multiple of 4), 0 = read cols at run time
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_iq3_xxs_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                            float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
    __shared__ float4 s_grid[256];    // the codebook's four magnitudes per entry, as floats
    __shared__ uint8_t s_signs[128];  // 7 stored sign bits -> 8 sign bits (the eighth is their parity)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint32_t c = c_iq3xxs_grid_packed[i];
        float m[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            m[j] = lvl == 7u ? 62.0f : float(4u + 8u * lvl);
        }
        s_grid[i] = make_float4(m[0], m[1], m[2], m[3]);
    }
    for (int i = threadIdx.x; i < 128; i += blockDim.x) s_signs[i] = uint8_t(i | ((__popc(i) & 1) << 7));
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nsb = NSB > 0 ? NSB : cols / 256;
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
        if constexpr (NSB > 0) {
#pragma unroll
            for (int sb0 = 0; sb0 < NSB; sb0 += 4) {
                iq3_sb_regs r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) iq3_load(r[j], row + (sb0 + j) * 98, lane);
#pragma unroll
                for (int j = 0; j < 4; ++j) iq3_finish(r[j], dst + (sb0 + j) * 256, lane, s_grid, s_signs);
            }
        } else {
            for (int sb = 0; sb < nsb; ++sb) {
                iq3_sb_regs r;
                iq3_load(r, row + sb * 98, lane);
                iq3_finish(r, dst + sb * 256, lane, s_grid, s_signs);
            }
        }
    }
}

// ---- Q8_0 ------------------------------------------------------------------------------------------------
// block: fp16 d, 32 int8; value = q * d.  A lane decodes 4 codes of each of the row's blocks it visits; blocks
// are 34 bytes (2-byte aligned), so codes are fetched as two 16-bit loads from L1/L2.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    get_rows_q8_0_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ ids,
                         float * __restrict__ out, uint32_t * err, int64_t rows, int cols) {
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
    get_rows_q4_k_kernel<8><<<persistent_grid(rows, 8), kWarpsPerCta * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(table), n_vocab, ids, out, err, rows, cols);
    return launch_status();
}

extern "C" int32_t fnb_get_rows_iq3_xxs(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                                        uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 256, 98, 2)) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(table);
    if (cols == 2048) {
        get_rows_iq3_xxs_kernel<8><<<persistent_grid(rows, 8), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    } else {
        get_rows_iq3_xxs_kernel<0><<<persistent_grid(rows, 8), kWarpsPerCta * 32, 0, s>>>(tb, n_vocab, ids, out, err, rows, cols);
    }
    return launch_status();
}

extern "C" int32_t fnb_get_rows_q8_0(const void * table, int64_t n_vocab, const int32_t * ids, float * out,
                                     uint32_t * err, int64_t rows, int32_t cols, void * stream) {
    using namespace fnb;
    if (!common_ok(table, n_vocab, ids, out, err, rows, cols, 32, 34, 2)) return FNB_REJECTED;
    get_rows_q8_0_kernel<<<persistent_grid(rows, 8), kWarpsPerCta * 32, 0, static_cast<cudaStream_t>(stream)>>>(
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
