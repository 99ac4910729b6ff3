// The reference engine's own embedding layouts: an IQ3_S or Q8_0 table that holds one card's `n_own` features of
// every token, decoded to F32 and fanned out to up to three destinations - own [rows][n_own], the card's columns of
// full [rows][n_full], and the same columns of every one of n_streams residual streams [rows][n_streams][n_full] -
// plus the two copy kernels that go with it: join (the peer card's half into the other columns) and supply (rows
// produced elsewhere, e.g. by a vision encoder, written over the decoded ones).  Semantics and argument rules follow
// fn::embed::embed_rows / embed_join / embed_supply (fn/kernels/embed/embed.h:70-105, embed_prompt.cu:26-146); the
// widths the reference hard-codes (1280 / 2560 / 4 streams, two cards) are arguments here, so one GPU can also hold
// whole rows (n_own = n_full, col0 = 0).
//
// Write-bound: every decoded value is stored 1 + 1 + n_streams times.  A warp owns a token; lane L decodes codebook
// indices L and L + 32 of each 256-value super-block so that each store instruction writes 512 contiguous bytes; the
// IQ3_S codebook (512 x 4 magnitudes, expanded to floats) lives in shared memory.
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarpsPerCta = 8;

__constant__ uint16_t c_iq3s_grid_packed[512] = {
#include "iq3s_grid_packed.inc"
};

struct row_sink {
    float * own;
    float * full;
    float * streams;
    int n_own, n_full, col0, n_streams;
    // four values of token t starting at column `col` of the card's own features
    __device__ __forceinline__ void put(int64_t t, int col, float4 v) const {
        if (own != nullptr) st_stream(reinterpret_cast<float4 *>(own + t * n_own + col), v);
        if (full != nullptr) st_stream(reinterpret_cast<float4 *>(full + t * n_full + col0 + col), v);
        if (streams != nullptr) {
            for (int s = 0; s < n_streams; ++s) {
                st_stream(reinterpret_cast<float4 *>(streams + (t * n_streams + s) * n_full + col0 + col), v);
            }
        }
    }
};

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t * p) { return __ldg(reinterpret_cast<const uint16_t *>(p)); }
__device__ __forceinline__ uint32_t ldg_u8(const uint8_t * p) { return __ldg(p); }

// index n of an IQ3_S super-block -> its four values (ggml/src/ggml-quants.c:2605-2644 restated per index)
// magnitude byte J of a codebook word as a float: 0x4B0000bb is 2^23 + bb exactly
template <int J>
__device__ __forceinline__ float grid_byte_f32(uint32_t g) {
    return __fadd_rn(__uint_as_float(__byte_perm(g, 0x4B000000u, 0x7540u + J)), -8388608.0f);
}
__device__ __forceinline__ float4 iq3s_decode(float d, uint32_t q, uint32_t qh, uint32_t sg, uint32_t sc, int n,
                                              const uint32_t * s_grid) {
    const int m = n & 7, ib = n >> 3;
    const uint32_t nib = (ib & 1) ? sc >> 4 : sc & 0x0fu;
    const float db = __fmul_rn(d, float(1 + 2 * int(nib)));
    const float nb = -db;
    const uint32_t g = s_grid[q | (((qh >> m) & 1u) << 8)];
    const uint32_t s4 = sg >> (4 * (n & 1));
    return make_float4(__fmul_rn((s4 & 1u) ? nb : db, grid_byte_f32<0>(g)), __fmul_rn((s4 & 2u) ? nb : db, grid_byte_f32<1>(g)),
                       __fmul_rn((s4 & 4u) ? nb : db, grid_byte_f32<2>(g)), __fmul_rn((s4 & 8u) ? nb : db, grid_byte_f32<3>(g)));
}

__global__ void __launch_bounds__(kWarpsPerCta * 32)
    embed_iq3s_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ tok, int64_t rows,
                      const row_sink sink, uint32_t * err) {
    // four magnitude bytes per entry: a random 32-bit lookup collides on a bank about three deep, where a float4
    // entry (no conversion) cost about eleven shared-memory wavefronts
    __shared__ uint32_t s_grid[512];
    for (int i = threadIdx.x; i < 512; i += blockDim.x) {
        const uint32_t c = c_iq3s_grid_packed[i];
        s_grid[i] = (2 * (c & 7u) + 1) | ((2 * ((c >> 3) & 7u) + 1) << 8) | ((2 * ((c >> 6) & 7u) + 1) << 16) |
                    ((2 * ((c >> 9) & 7u) + 1) << 24);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nsb = sink.n_own / 256;
    const int64_t row_bytes = int64_t(nsb) * 110;
    int32_t id_next = warp < rows ? __ldg(tok + warp) : 0;
    for (int64_t t = warp; t < rows; t += n_warps) {
        const int32_t id = id_next;
        if (t + n_warps < rows) id_next = __ldg(tok + t + n_warps);
        if (id < 0 || id >= n_vocab) {
            if (lane == 0 && err != nullptr) atomicOr(err, FNB_ERR_TOKEN);
            continue;
        }
        const uint8_t * row = table + int64_t(id) * row_bytes;
        for (int sb = 0; sb < nsb; ++sb) {
            const uint8_t * blk = row + sb * 110;
            const float d = f16_bits_to_f32(uint16_t(ldg_u16(blk)));
            const uint32_t q0 = ldg_u8(blk + 2 + lane), q1 = ldg_u8(blk + 34 + lane);
            const uint32_t h0 = ldg_u8(blk + 66 + (lane >> 3)), h1 = ldg_u8(blk + 70 + (lane >> 3));
            const uint32_t g0 = ldg_u8(blk + 74 + (lane >> 1)), g1 = ldg_u8(blk + 90 + (lane >> 1));
            const uint32_t c0 = ldg_u8(blk + 106 + (lane >> 4)), c1 = ldg_u8(blk + 108 + (lane >> 4));
            sink.put(t, sb * 256 + 4 * lane, iq3s_decode(d, q0, h0, g0, c0, lane, s_grid));
            sink.put(t, sb * 256 + 128 + 4 * lane, iq3s_decode(d, q1, h1, g1, c1, lane, s_grid));  // index lane + 32
        }
    }
}

__global__ void __launch_bounds__(kWarpsPerCta * 32)
    embed_q8_0_kernel(const uint8_t * __restrict__ table, int64_t n_vocab, const int32_t * __restrict__ tok, int64_t rows,
                      const row_sink sink, uint32_t * err) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int nb = sink.n_own / 32;
    const int64_t row_bytes = int64_t(nb) * 34;
    for (int64_t t = warp; t < rows; t += n_warps) {
        const int32_t id = __ldg(tok + t);
        if (id < 0 || id >= n_vocab) {
            if (lane == 0 && err != nullptr) atomicOr(err, FNB_ERR_TOKEN);
            continue;
        }
        const uint8_t * row = table + int64_t(id) * row_bytes;
        for (int b0 = 0; b0 < nb; b0 += 4) {  // 8 lanes per block, 4 blocks per trip
            const int b = b0 + (lane >> 3);
            if (b < nb) {
                const uint8_t * blk = row + b * 34;
                const float d = f16_bits_to_f32(uint16_t(ldg_u16(blk)));
                const uint32_t w = ldg_u16(blk + 2 + 4 * (lane & 7)) | (ldg_u16(blk + 4 + 4 * (lane & 7)) << 16);
                sink.put(t, b * 32 + 4 * (lane & 7),
                         make_float4(__fmul_rn(float(int8_t(w & 0xffu)), d), __fmul_rn(float(int8_t((w >> 8) & 0xffu)), d),
                                     __fmul_rn(float(int8_t((w >> 16) & 0xffu)), d), __fmul_rn(float(int8_t(w >> 24)), d)));
            }
        }
    }
}

// a thread a float4: src rows [n][n_own] into destination rows row0 .. row0 + n - 1 at column col0;
// check_tok: skip rows whose token is outside the table (embed_rows flagged them and wrote nothing)
__global__ void embed_copy_kernel(const float * __restrict__ src, int64_t n, int64_t row0, const row_sink sink,
                                  const int32_t * __restrict__ tok, int64_t n_vocab) {
    const int q4 = sink.n_own / 4;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n * q4; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / q4;
        const int c4 = int(i - r * q4);
        const int64_t t = row0 + r;
        if (tok != nullptr) {
            const int32_t id = __ldg(tok + t);
            if (id < 0 || id >= n_vocab) continue;
        }
        sink.put(t, 4 * c4, __ldg(reinterpret_cast<const float4 *>(src + r * sink.n_own) + c4));
    }
}

bool sink_of(const fnb_embed_args * a, row_sink & s) {
    if (a == nullptr) return false;
    if (a->n_own < 4 || a->n_own > 16384 || a->n_own % 4 != 0) return false;
    if (!ok_opt(a->own, 16) || !ok_opt(a->full, 16) || !ok_opt(a->streams, 16)) return false;
    if (a->own == nullptr && a->full == nullptr && a->streams == nullptr) return false;
    if (a->full != nullptr || a->streams != nullptr) {
        if (a->n_full < a->n_own || a->n_full % 4 != 0 || a->col0 < 0 || a->col0 % 4 != 0 || a->col0 + a->n_own > a->n_full) {
            return false;
        }
    }
    if (a->streams != nullptr && (a->n_streams < 1 || a->n_streams > 64)) return false;
    if (a->rows < 1 || a->rows > INT32_MAX) return false;
    s.own = a->own, s.full = a->full, s.streams = a->streams;
    s.n_own = a->n_own, s.n_full = a->n_full, s.col0 = a->col0, s.n_streams = a->n_streams;
    return true;
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_embed_rows(const fnb_embed_args * a, void * stream) {
    using namespace fnb;
    row_sink s;
    if (!sink_of(a, s)) return FNB_REJECTED;
    if (!ok_ptr(a->table, 2) || !ok_ptr(a->tok, 4) || !ok_opt(a->err, 4) || a->n_vocab < 1 || a->n_vocab > INT32_MAX) {
        return FNB_REJECTED;
    }
    // many more CTAs than are resident: the CTA dispatcher evens out SMs that drain their rows at different rates
    const int grid = grid_for((a->rows + kWarpsPerCta - 1) / kWarpsPerCta, 32);
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t * tb = static_cast<const uint8_t *>(a->table);
    if (a->fmt == FNB_TABLE_IQ3_S) {
        if (a->n_own % 256 != 0) return FNB_REJECTED;
        embed_iq3s_kernel<<<grid, kWarpsPerCta * 32, 0, st>>>(tb, a->n_vocab, a->tok, a->rows, s, a->err);
    } else if (a->fmt == FNB_TABLE_Q8_0) {
        if (a->n_own % 32 != 0) return FNB_REJECTED;
        embed_q8_0_kernel<<<grid, kWarpsPerCta * 32, 0, st>>>(tb, a->n_vocab, a->tok, a->rows, s, a->err);
    } else {
        return FNB_REJECTED;
    }
    return launch_status();
}

extern "C" int32_t fnb_embed_join(const fnb_embed_args * a, const float * peer, int32_t peer_col0, void * stream) {
    using namespace fnb;
    row_sink s;
    if (!sink_of(a, s) || !ok_ptr(peer, 16) || !ok_ptr(a->tok, 4) || a->n_vocab < 1) return FNB_REJECTED;
    if (a->full == nullptr && a->streams == nullptr) return FNB_REJECTED;
    if (peer_col0 < 0 || peer_col0 % 4 != 0 || peer_col0 + a->n_own > a->n_full) return FNB_REJECTED;
    s.own = nullptr;        // the peer's half goes into full and the streams only
    s.col0 = peer_col0;
    const int64_t n4 = a->rows * (a->n_own / 4);
    embed_copy_kernel<<<grid_for((n4 + 255) / 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(peer, a->rows, 0, s, a->tok,
                                                                                                  a->n_vocab);
    return launch_status();
}

extern "C" int32_t fnb_embed_supply(const fnb_embed_args * a, const float * src, int64_t row0, int64_t n, void * stream) {
    using namespace fnb;
    row_sink s;
    if (!sink_of(a, s) || !ok_ptr(src, 16)) return FNB_REJECTED;
    if (n < 1 || row0 < 0 || row0 + n > a->rows) return FNB_REJECTED;
    const int64_t n4 = n * (a->n_own / 4);
    embed_copy_kernel<<<grid_for((n4 + 255) / 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, n, row0, s, nullptr, 0);
    return launch_status();
}
