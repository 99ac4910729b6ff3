// The routed experts' gate / up mat-vec for a decode window with the GLU fused,
//     ff[t][r] = silu(g) u,   g = gate row r . act[t],  u = up row r . act[t],   t < nt,  r in [r0, r1)
// with ggml IQ3_XXS weights against Q8_K activations (fnb_quantize_q8_k).  Replaces fn::experts::cpu::iq_gu_rows for
// fmt iq3_xxs (fn/kernels/experts/cpu_kernels.h:67; cpu_iq_avx2.cpp:256-271 decode, :305-337 row_dot, :429-445 gu_rows)
// and returns the SAME BITS: the AVX2 kernel keeps, per (row, t), eight int32 lanes a super-block - lane l collects,
// over the block's eight groups of 32 values, (2 s + 1) x the four codebook bytes of the group's index byte l times the
// sign-applied Q8_K codes 32 g + 4 l .. - adds them as floats by one fused multiply-add per super-block and lane with
// x.d y.d (x.d WITHOUT the format's 1/4), reduces in ggml's hsum_float_8 order, multiplies the sum by 1/4 and applies
// g / (1 + expf(-g)) * u (expf as the host C library evaluates it: exact_math.cuh).  Here EIGHT GPU LANES stand for the
// eight AVX2 lanes of one weight row and a warp takes four (gate, up) row pairs at a time.
//
// The signs go onto the CODEBOOK bytes (once per weight, whatever the window), which equals the reference's negated
// codes unless a code is -128: _mm256_sign_epi8 leaves -128 as it is.  ggml's Q8_K quantiser cannot emit -128, but a
// CTA that finds one in its window takes the variant that negates the codes byte-wise in two's complement instead.
//
// A row is 98-byte blocks; with an even number of them (n a multiple of 512) rows are 4-byte aligned.  A warp copies
// its eight rows (up to ten super-blocks of each at a time) with cp.async into its own shared-memory buffers, one unit
// ahead of the one it computes on: 16-byte copies between the 16-byte boundaries of the source, whose offset within 16
// bytes the shared-memory copy keeps, and up to three 4-byte copies at either end.
// At three bits a weight the kernel is as much arithmetic as HBM traffic: per four weights one index-byte load, one
// codebook load, about six integer operations for the signs and, per window row, one dp4a and one multiply-add.
#include <atomic>

#include "common.cuh"
#include "exact_math.cuh"

#ifndef FNB_GU_IQ3_GRID
#define FNB_GU_IQ3_GRID 8
#endif

namespace fnb {
namespace {

constexpr int kMaxWarps = 8;
constexpr int kMaxT = 8;
constexpr int kWholeRowBlocks = 10;                  // rows of up to ten super-blocks (2560 columns) are staged whole,
constexpr int kChunkBlocks = 8;                      // longer ones eight super-blocks (784 = 49 x 16 bytes) at a time
constexpr int kSlotBytes = 1008;                     // ten blocks, 12 bytes of source offset, rounded up to 16
constexpr int kUnitBytes = 8 * kSlotBytes;           // four gate rows, then four up rows
constexpr int kWarpStage = 2 * kUnitBytes;           // two units: the one computed on and the one in flight
constexpr size_t kSmemLimit = 200 * 1024;            // one CTA per SM
constexpr size_t kSmemTwo = 113 * 1024;              // two CTAs per SM (228 KB an SM, 1 KB reserved and ~1.3 KB static a CTA)
constexpr int kGridPerSm = FNB_GU_IQ3_GRID;

__constant__ uint16_t c_grid_packed[256] = {
#include "iq3xxs_grid_packed.inc"
};

// the four sign bits of values 4 l .. 4 l + 3 of a group, one per byte (0x01 where the value is negated): seven stored
// bits per eight values, the eighth their parity (ksigns_iq2xs)
__device__ __forceinline__ uint32_t sign_bytes(uint32_t w, int sh7, int sh4) {
    const uint32_t s7 = (w >> sh7) & 127u;
    const uint32_t s8 = s7 | ((__popc(s7) & 1u) << 7);
    return (((s8 >> sh4) & 15u) * 0x00204081u) & 0x01010101u;
}

// codebook bytes (4 .. 62) negated where m1 has the byte's bit: 256 - g never carries out of its byte
__device__ __forceinline__ int signed_grid(uint32_t g, uint32_t m1) { return int((g ^ (m1 * 0xffu)) + m1); }

// Q8_K codes negated in two's complement where m1 has the byte's bit, -128 staying -128 (_mm256_sign_epi8)
__device__ __forceinline__ int signed_codes(uint32_t y, uint32_t m1) {
    const uint32_t a = y ^ (m1 * 0xffu);
    return int(((a & 0x7f7f7f7fu) + m1) ^ (a & 0x80808080u));
}

// where row r's chunk of a matrix starts; a ragged last quad re-reads the last row (its results are not stored)
__device__ __forceinline__ const uint8_t * chunk_src(const uint8_t * mat, int64_t row_bytes, int64_t r, int64_t r1, int chunk) {
    return mat + (r < r1 ? r : r1 - 1) * row_bytes + int64_t(chunk) * (kChunkBlocks * 98);
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const uint8_t * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const uint8_t * src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// `bytes` (a multiple of 4) from src (4-byte aligned) into a slot, at src's own offset within 16 bytes
__device__ __forceinline__ void stage_slot(uint32_t slot_sm, const uint8_t * src, int bytes, int lane) {
    const int phase = int(reinterpret_cast<uintptr_t>(src) & 15);
    const uint32_t dst = slot_sm + phase;
    const int head = (16 - phase) & 15;  // bytes is at least 196, so the head is whole
    const int body = (bytes - head) >> 4, tail = (bytes - head) & 15;
    for (int c = lane; c < body; c += 32) cp_async_16(dst + head + 16 * c, src + head + 16 * c);
    if (lane < (head >> 2)) {
        cp_async_4(dst + 4 * lane, src + 4 * lane);
    } else if (lane >= 8 && lane - 8 < (tail >> 2)) {
        const int o = head + 16 * body + 4 * (lane - 8);
        cp_async_4(dst + o, src + o);
    }
}

__device__ __forceinline__ void stage_unit(uint32_t buf_sm, const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up,
                                           int64_t row_bytes, int64_t r4, int64_t r1, int chunk, int bytes, int lane) {
#pragma unroll
    for (int slot = 0; slot < 8; ++slot) {
        stage_slot(buf_sm + slot * kSlotBytes, chunk_src(slot < 4 ? gate : up, row_bytes, r4 + (slot & 3), r1, chunk), bytes, lane);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// one staged unit (n_blk super-blocks of four row pairs; xg, xu: this lane's gate and up row in it) against the window
template <int NT, bool WRAP>
__device__ __forceinline__ void dot_unit(const uint8_t * xg, const uint8_t * xu, int n_blk, const uint8_t * act_sm, int nb,
                                         int blk0, int l, const uint32_t * s_grid, float (&g)[NT], float (&u)[NT]) {
    const int sh7 = 7 * (l >> 1), sh4 = 4 * (l & 1);
#pragma unroll 1
    for (int i = 0; i < n_blk; ++i, xg += 98, xu += 98) {
        // lane l holds the sign / scale word of group l (2-byte aligned), every lane gets each group's by a shuffle
        const uint16_t * pg = reinterpret_cast<const uint16_t *>(xg + 66 + 4 * l);
        const uint16_t * pu = reinterpret_cast<const uint16_t *>(xu + 66 + 4 * l);
        const uint32_t own_g = uint32_t(pg[0]) | (uint32_t(pg[1]) << 16), own_u = uint32_t(pu[0]) | (uint32_t(pu[1]) << 16);
        const float dg = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(xg));
        const float du = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(xu));
        int ag[NT], au[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) ag[t] = 0, au[t] = 0;
        const uint8_t * y0 = act_sm + size_t(blk0 + i) * 292 + 4 + 4 * l;
#pragma unroll
        for (int grp = 0; grp < 8; ++grp) {
            const uint32_t wg = __shfl_sync(kFull, own_g, grp, 8), wu = __shfl_sync(kFull, own_u, grp, 8);
            const uint32_t cg = s_grid[xg[2 + 8 * grp + l]], cu = s_grid[xu[2 + 8 * grp + l]];
            const uint32_t mg = sign_bytes(wg, sh7, sh4), mu = sign_bytes(wu, sh7, sh4);
            const int scg = int(2u * (wg >> 28) + 1u), scu = int(2u * (wu >> 28) + 1u);
            const int vg = WRAP ? int(cg) : signed_grid(cg, mg), vu = WRAP ? int(cu) : signed_grid(cu, mu);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const uint32_t y = *reinterpret_cast<const uint32_t *>(y0 + size_t(t) * nb * 292 + 32 * grp);
                if (WRAP) {
                    ag[t] += scg * __dp4a(vg, signed_codes(y, mg), 0);
                    au[t] += scu * __dp4a(vu, signed_codes(y, mu), 0);
                } else {
                    ag[t] += scg * __dp4a(vg, int(y), 0);
                    au[t] += scu * __dp4a(vu, int(y), 0);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float yd = *reinterpret_cast<const float *>(act_sm + (size_t(t) * nb + blk0 + i) * 292);
            g[t] = __fmaf_rn(__fmul_rn(dg, yd), float(ag[t]), g[t]);
            u[t] = __fmaf_rn(__fmul_rn(du, yd), float(au[t]), u[t]);
        }
    }
}

template <int NT, bool WRAP>
__device__ __forceinline__ void run_warp(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes,
                                         int nb, const uint8_t * act_sm, uint8_t * stage, const uint32_t * s_grid,
                                         float * __restrict__ ff, int64_t ff_stride, float * __restrict__ gu, int64_t r0,
                                         int64_t r1) {
    const int lane = threadIdx.x & 31, l = lane & 7, sub = lane >> 3;
    const int warps = blockDim.x >> 5;
    const int64_t n_quads = (r1 - r0 + 3) / 4, stride = int64_t(gridDim.x) * warps;
    const int chunk_blocks = nb <= kWholeRowBlocks ? nb : kChunkBlocks;
    const int n_chunks = (nb + chunk_blocks - 1) / chunk_blocks;
    const auto blocks_of = [&](int chunk) { return chunk == n_chunks - 1 ? nb - chunk * chunk_blocks : chunk_blocks; };
    int64_t q = int64_t(blockIdx.x) * warps + (threadIdx.x >> 5);
    if (q >= n_quads) return;
    const uint32_t stage_sm = uint32_t(__cvta_generic_to_shared(stage));
    int c = 0, k = 0;
    stage_unit(stage_sm, gate, up, row_bytes, r0 + 4 * q, r1, 0, blocks_of(0) * 98, lane);
    float g[NT], u[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) g[t] = 0.0f, u[t] = 0.0f;
    for (;;) {
        int64_t qn = q;
        int cn = c + 1;
        if (cn == n_chunks) cn = 0, qn = q + stride;
        const bool more = qn < n_quads;
        if (more) {
            stage_unit(stage_sm + uint32_t((k + 1) & 1) * kUnitBytes, gate, up, row_bytes, r0 + 4 * qn, r1, cn,
                       blocks_of(cn) * 98, lane);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();
        {
            const uint8_t * buf = stage + (k & 1) * kUnitBytes;
            const int64_t r = r0 + 4 * q + sub;
            const uintptr_t pg = reinterpret_cast<uintptr_t>(chunk_src(gate, row_bytes, r, r1, c));
            const uintptr_t pu = reinterpret_cast<uintptr_t>(chunk_src(up, row_bytes, r, r1, c));
            dot_unit<NT, WRAP>(buf + sub * kSlotBytes + (pg & 15), buf + (4 + sub) * kSlotBytes + (pu & 15), blocks_of(c), act_sm,
                               nb, c * chunk_blocks, l, s_grid, g, u);
        }
        __syncwarp();  // every lane is done with the buffer the next trip's copies overwrite
        if (c == n_chunks - 1) {
            const int64_t r = r0 + 4 * q + sub;
            const bool live = r < r1;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                // ggml's hsum_float_8: lane i + 4 onto lane i, lanes 2, 3 onto 0, 1, lane 1 onto lane 0
                float a = g[t], b = u[t];
                a = __fadd_rn(__shfl_down_sync(kFull, a, 4, 8), a), b = __fadd_rn(__shfl_down_sync(kFull, b, 4, 8), b);
                a = __fadd_rn(a, __shfl_down_sync(kFull, a, 2, 8)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 2, 8));
                a = __fadd_rn(a, __shfl_down_sync(kFull, a, 1, 8)), b = __fadd_rn(b, __shfl_down_sync(kFull, b, 1, 8));
                if (l == 0 && live) {
                    const float gs = __fmul_rn(0.25f, a), us = __fmul_rn(0.25f, b);
                    ff[int64_t(t) * ff_stride + r] = __fmul_rn(__fdiv_rn(gs, __fadd_rn(1.0f, exact_expf(-gs))), us);
                    if (gu != nullptr) {
                        gu[int64_t(t) * ff_stride + r] = gs;
                        gu[(int64_t(NT) + t) * ff_stride + r] = us;
                    }
                }
                g[t] = 0.0f, u[t] = 0.0f;
            }
        }
        if (!more) break;
        q = qn, c = cn, ++k;
    }
}

template <int NT>
__global__ void __launch_bounds__(kMaxWarps * 32)
    gate_up_iq3_xxs_kernel(const uint8_t * __restrict__ gate, const uint8_t * __restrict__ up, int64_t row_bytes, int nb,
                           const uint8_t * __restrict__ act, int64_t act_stride, int act_bytes, float * __restrict__ ff,
                           int64_t ff_stride, float * __restrict__ gu, int64_t r0, int64_t r1) {
    extern __shared__ __align__(16) uint8_t smem[];  // the window's Q8_K blocks [NT][nb][292], then each warp's two units
    __shared__ uint32_t s_grid[256];                 // the codebook's four magnitudes per entry as bytes
    load_exp2_table();
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        const uint32_t c = c_grid_packed[i];
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lvl = (c >> (3 * j)) & 7u;
            w |= (lvl == 7u ? 62u : 4u + 8u * lvl) << (8 * j);
        }
        s_grid[i] = w;
    }
    int has_m128 = 0;
    for (int i = threadIdx.x; i < NT * nb * 73; i += blockDim.x) {
        const int t = i / (nb * 73), k = i - t * nb * 73;
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(act + int64_t(t) * act_stride) + k);
        reinterpret_cast<uint32_t *>(smem)[i] = w;
        const int word = k % 73;
        if (word >= 1 && word <= 64) {  // a code byte equal to 0x80
            const uint32_t v = w ^ 0x80808080u;
            has_m128 |= ((v - 0x01010101u) & ~v & 0x80808080u) != 0u;
        }
    }
    const int wrap = __syncthreads_or(has_m128);
    uint8_t * stage = smem + act_bytes + size_t(threadIdx.x >> 5) * kWarpStage;
    if (wrap) {
        run_warp<NT, true>(gate, up, row_bytes, nb, smem, stage, s_grid, ff, ff_stride, gu, r0, r1);
    } else {
        run_warp<NT, false>(gate, up, row_bytes, nb, smem, stage, s_grid, ff, ff_stride, gu, r0, r1);
    }
}

template <int NT>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(gate_up_iq3_xxs_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemLimit)) !=
            cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

// window rows one launch can hold for nb super-blocks a row (their Q8_K blocks and at least four warps' buffers)
inline int window_rows(int nb) {
    const size_t per_t = size_t(nb) * 292, room = kSmemLimit - 4 * size_t(kWarpStage) - 16;
    const size_t m = room / per_t;
    return int(m > size_t(kMaxT) ? size_t(kMaxT) : m);
}

template <int NT>
int32_t launch_nt(const uint8_t * gate, const uint8_t * up, int64_t row_bytes, int nb, const uint8_t * act, int64_t act_stride,
                  float * ff, int64_t ff_stride, float * gu, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t act_bytes = (size_t(NT) * nb * 292 + 15) & ~size_t(15);
    // as many warps as leave room for two CTAs on an SM, else one CTA of up to eight
    int warps = act_bytes < kSmemTwo ? int((kSmemTwo - act_bytes) / kWarpStage) : 0;
    if (warps < 4) warps = int((kSmemLimit - act_bytes) / kWarpStage);
    warps = warps > kMaxWarps ? kMaxWarps : warps;
    if (warps < 1) return FNB_REJECTED;
    if (!ensure_configured<NT>()) return FNB_LAUNCH_FAILED;
    const size_t smem = act_bytes + size_t(warps) * kWarpStage;
    const int64_t quads = (r1 - r0 + 3) / 4;
    const int grid = grid_for((quads + warps - 1) / warps, kGridPerSm);
    gate_up_iq3_xxs_kernel<NT><<<grid, warps * 32, smem, s>>>(gate, up, row_bytes, nb, act, act_stride, int(act_bytes), ff,
                                                                ff_stride, gu, r0, r1);
    return launch_status();
}

}  // namespace

bool expert_gate_up_prepare_device() {
    return ensure_configured<1>() && ensure_configured<2>() && ensure_configured<3>() && ensure_configured<4>() &&
           ensure_configured<5>() && ensure_configured<6>() && ensure_configured<7>() && ensure_configured<8>();
}

}  // namespace fnb

extern "C" int32_t fnb_expert_gate_up_rows_iq3_xxs(const void * gate, const void * up, int64_t row_bytes, int32_t n,
                                                   const void * act, int64_t act_stride, int32_t nt, float * ff,
                                                   int64_t ff_stride, float * gu, int64_t r0, int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(gate, 16) || !ok_ptr(up, 16) || !ok_ptr(act, 4) || !ok_ptr(ff, 4) || !ok_opt(gu, 4)) return FNB_REJECTED;
    // an even number of 98-byte super-blocks a row: rows on 4-byte boundaries, which the copies into shared memory need
    if (n < 512 || n > 16384 || n % 512 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 256;
    if (row_bytes != int64_t(nb) * 98 || act_stride < int64_t(nb) * 292 || act_stride % 4 != 0 || ff_stride < r1) return FNB_REJECTED;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t * gp = static_cast<const uint8_t *>(gate);
    const uint8_t * upp = static_cast<const uint8_t *>(up);
    const uint8_t * a = static_cast<const uint8_t *>(act);
    const int max_t = window_rows(nb);
    if (max_t < 1) return FNB_REJECTED;
    // g and u of a later pass would need their own [2][m] planes: the debug output is for windows of one pass
    if (gu != nullptr && nt > max_t) return FNB_REJECTED;
    for (int t0 = 0; t0 < nt; t0 += max_t) {  // longer windows take further passes, as the reference's do above eight rows
        const int m = nt - t0 < max_t ? nt - t0 : max_t;
        const uint8_t * at = a + int64_t(t0) * act_stride;
        float * ft = ff + int64_t(t0) * ff_stride;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 2: st = launch_nt<2>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 3: st = launch_nt<3>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 4: st = launch_nt<4>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 5: st = launch_nt<5>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 6: st = launch_nt<6>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            case 7: st = launch_nt<7>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
            default: st = launch_nt<8>(gp, upp, row_bytes, nb, at, act_stride, ft, ff_stride, gu, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}
