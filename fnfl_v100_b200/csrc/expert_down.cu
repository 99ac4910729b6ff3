// The consumer of the Q8_1 activations SwiGLU leaves: the routed experts' down mat-vec for a decode window,
//     out[t][r] = weight row r . act[t],   t < nt (a few rows share one pass over the weights), r in [r0, r1)
// with ggml's Q5_1 weights (24-byte blocks: fp16 d, fp16 m, 32 high bits, 16 bytes of nibbles; value = d q + m)
// against Q8_1 activations.  Replaces fn::experts::cpu::kq_down_rows (fn/kernels/experts/cpu_kernels.h,
// cpu_kq_avx2.cpp:293-320, :382-394) and is BIT-IDENTICAL to it: the AVX2 kernel keeps eight F32 lanes per (row, t),
// lane j taking bytes 4 j .. 4 j + 3 of every block by one fused multiply-add per block with the block's scale
// product, a fused scalar side sum of m x s, and one horizontal sum at the end in a fixed order; a GPU lane owns a
// weight row and keeps the same eight accumulators per t in registers, so every float operation happens in the
// reference's order.
//
// HBM-bound on the weights for the window sizes decode uses (nt <= 3); for larger nt the per-(block, t) arithmetic
// the bit-exact order needs (8 dp4a + 8 conversions + 9 fused multiply-adds per lane) takes over.  A warp stages 32
// consecutive weight rows into shared memory with coalesced loads (padded so that lane = row reads are conflict-free),
// the window's activation blocks sit in shared memory once per CTA (their fp16 d and s widened once).
#include <atomic>

#include "common.cuh"

namespace fnb {
namespace {

constexpr int kMaxWarps = 4;  // warps per CTA (fewer when 32 staged rows per warp would not fit in shared memory)
constexpr int kMaxT = 8;      // rows of a window per pass over the weights (the reference's maxt)
constexpr size_t kSmemLimit = 200 * 1024;

__device__ __forceinline__ uint32_t smem_addr(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ float hsum8(const float (&a)[8]) {  // hsum_float_8's order
    const float r0 = __fadd_rn(a[4], a[0]), r1 = __fadd_rn(a[5], a[1]), r2 = __fadd_rn(a[6], a[2]), r3 = __fadd_rn(a[7], a[3]);
    return __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
}

// NT: activation rows of this pass (1..8), compile time so the accumulators stay in registers.
// Q8: Q8_0 weights against Q8_0 activations (cpu_kq_avx2.cpp:322-344: no side sum) instead of Q5_1 against Q8_1.
template <int NT, bool Q8>
__global__ void __launch_bounds__(kMaxWarps * 32)
    down_rows_kernel(const uint32_t * __restrict__ w, int row_words, int nb, const uint8_t * __restrict__ act,
                          int64_t act_stride, float * __restrict__ out, int64_t out_stride, int64_t r0, int64_t r1) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int kWarps = blockDim.x >> 5;
    // row stride in shared memory: even (8-byte copies land aligned) and 2 mod 4, so lane = row reads of one word are
    // at most two deep on a bank
    const int pad_words = row_words + (row_words % 4 == 0 ? 2 : 0);
    // activations first (16-byte aligned vectors), then the warps' staged rows
    // (block-major, so that within a block the window rows sit at compile-time offsets)
    uint32_t * qy_sm = reinterpret_cast<uint32_t *>(smem);                     // [nb][NT][8] the activations' code words
    float2 * ds_sm = reinterpret_cast<float2 *>(qy_sm + size_t(NT) * nb * 8);  // [nb][NT] {d, s} as F32
    uint32_t * rows_sm = reinterpret_cast<uint32_t *>(ds_sm + size_t(NT) * nb);  // [kWarps][32][pad_words]

    for (int i = threadIdx.x; i < NT * nb; i += blockDim.x) {
        const int t = i / nb, ib = i - t * nb;
        const int o = ib * NT + t;
        if (Q8) {  // 34-byte blocks, 2-byte aligned: {fp16 d, 32 codes}
            const uint16_t * y = reinterpret_cast<const uint16_t *>(act + int64_t(t) * act_stride + size_t(ib) * 34);
            ds_sm[o] = make_float2(f16_bits_to_f32(__ldg(y)), 0.0f);
#pragma unroll
            for (int k = 0; k < 8; ++k) qy_sm[size_t(o) * 8 + k] = uint32_t(__ldg(y + 1 + 2 * k)) | (uint32_t(__ldg(y + 2 + 2 * k)) << 16);
        } else {   // 36-byte blocks, 4-byte aligned: {fp16 d, fp16 s, 32 codes}
            const uint8_t * y = act + int64_t(t) * act_stride + size_t(ib) * 36;
            const uint32_t hdr = __ldg(reinterpret_cast<const uint32_t *>(y));
            ds_sm[o] = make_float2(f16_bits_to_f32(uint16_t(hdr & 0xffffu)), f16_bits_to_f32(uint16_t(hdr >> 16)));
#pragma unroll
            for (int k = 0; k < 8; ++k) qy_sm[size_t(o) * 8 + k] = __ldg(reinterpret_cast<const uint32_t *>(y + 4) + k);
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    uint32_t * mine = rows_sm + size_t(wid) * 32 * pad_words;
    const int64_t n_tiles = (r1 - r0 + 31) / 32;
    for (int64_t tile = int64_t(blockIdx.x) * kWarps + wid; tile < n_tiles; tile += int64_t(gridDim.x) * kWarps) {
        const int64_t row0 = r0 + tile * 32;
        const int live = int(r1 - row0 < 32 ? r1 - row0 : 32);
        // stage `live` consecutive rows with 8-byte asynchronous copies straight into shared memory (a row is a whole
        // number of 8-byte pairs: 24-byte blocks): every copy of the tile is in flight at once, none through registers.
        // Staging through registers, six loads at a time, cost ten memory round trips per tile and held the kernel at
        // 35 % of the roofline.
        {
            const uint2 * src = reinterpret_cast<const uint2 *>(w + row0 * row_words);
            const uint32_t rp = uint32_t(row_words) >> 1;
            const uint32_t total = uint32_t(live) * rp;
            const uint32_t inv = uint32_t((0x100000000ull + rp - 1) / rp);  // g / rp by multiply-high (g < 2^20)
            const uint32_t base_sm = smem_addr(mine);
            for (uint32_t g = lane; g < total; g += 32) {
                const uint32_t row = __umulhi(g, inv), col = 2 * (g - row * rp);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(base_sm + 4 * (row * pad_words + col)), "l"(src + g)
                             : "memory");
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
        __syncwarp();
        if (lane < live) {
            const uint32_t * my_row = mine + lane * pad_words;
            float acc[NT][8];
            float summs[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                summs[t] = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[t][j] = 0.0f;
            }
            // one block's eight code words against every window row (the arithmetic both formats share)
            auto block = [&](const uint32_t (&qx)[8], float xd, float xm, int ib) {
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float2 ds = ds_sm[ib * NT + t];
                    const uint4 y0 = *reinterpret_cast<const uint4 *>(qy_sm + size_t(ib * NT + t) * 8);
                    const uint4 y1 = *reinterpret_cast<const uint4 *>(qy_sm + size_t(ib * NT + t) * 8 + 4);
                    if (!Q8) summs[t] = __fmaf_rn(xm, ds.y, summs[t]);
                    const float scale = __fmul_rn(xd, ds.x);
                    const uint32_t qy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
                    // The integer sums become floats without a conversion instruction: the dot product accumulates onto
                    // the bits of 1.5 x 2^23, which makes the word the float 12582912 + sum (|sum| < 2^22), and one exact
                    // subtraction leaves float(sum); the subtraction and the fused multiply-add run two accumulators per
                    // instruction.
                    const f32x2 scale2 = pk(scale, scale), magic2 = pk(-12582912.0f, -12582912.0f);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const f32x2 biased = pk(__int_as_float(__dp4a(int(qx[j]), int(qy[j]), 0x4B400000)),
                                                __int_as_float(__dp4a(int(qx[j + 1]), int(qy[j + 1]), 0x4B400000)));
                        unpk(fma2(add2(biased, magic2), scale2, pk(acc[t][j], acc[t][j + 1])), acc[t][j], acc[t][j + 1]);
                    }
                }
            };
            if (Q8) {
                // 34-byte blocks in a word-aligned row: an even block starts on a word (d in its low half, the codes
                // straddle words), the odd block after it starts half a word in (d in the high half, codes aligned)
                for (int ib = 0; ib < nb; ib += 2) {
                    const uint32_t * b = my_row + 17 * (ib >> 1);
                    uint32_t wv[17];
#pragma unroll
                    for (int k = 0; k < 17; ++k) wv[k] = b[k];
                    uint32_t qe[8], qo[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        qe[j] = __funnelshift_r(wv[j], wv[j + 1], 16);
                        qo[j] = wv[9 + j];
                    }
                    block(qe, f16_bits_to_f32(uint16_t(wv[0] & 0xffffu)), 0.0f, ib);
                    block(qo, f16_bits_to_f32(uint16_t(wv[8] >> 16)), 0.0f, ib + 1);
                }
            } else {
#pragma unroll 2
                for (int ib = 0; ib < nb; ++ib) {
                    const uint32_t * b = my_row + 6 * ib;
                    const uint32_t dm = b[0], qh = b[1];
                    // bytes 4 j .. 4 j + 3 of the block's 32 five-bit values: low nibbles of qs[0..15], then the high
                    // ones, each with its bit of qh as bit 4
                    uint32_t qx[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t q = b[2 + k];
                        // four bits of qh to bit 4 of four bytes: bit i of the nibble times 0x02040810 lands on bit
                        // 4 + 7 i + i = 4 + 8 i (no two partial products share a bit below 2^32), the mask keeps those
                        const uint32_t sl = (((qh >> (4 * k)) & 15u) * 0x02040810u) & 0x10101010u;
                        const uint32_t sh = (((qh >> (16 + 4 * k)) & 15u) * 0x02040810u) & 0x10101010u;
                        qx[k] = (q & 0x0f0f0f0fu) | sl;
                        qx[k + 4] = ((q >> 4) & 0x0f0f0f0fu) | sh;
                    }
                    block(qx, f16_bits_to_f32(uint16_t(dm & 0xffffu)), f16_bits_to_f32(uint16_t(dm >> 16)), ib);
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                out[int64_t(t) * out_stride + row0 + lane] = Q8 ? hsum8(acc[t]) : __fadd_rn(hsum8(acc[t]), summs[t]);
            }
        }
        __syncwarp();
    }
}

// raises the kernel's dynamic shared-memory limit once per device
template <int NT, bool Q8>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(down_rows_kernel<NT, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemLimit)) !=
            cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

template <int NT, bool Q8>
int32_t launch_nt(const uint32_t * w, int row_words, int nb, const uint8_t * act, int64_t act_stride, float * out,
                  int64_t out_stride, int64_t r0, int64_t r1, cudaStream_t s) {
    const size_t per_warp = size_t(32) * (row_words + (row_words % 4 == 0 ? 2 : 0)) * 4, fixed = size_t(NT) * nb * 40;
    if (fixed + per_warp > kSmemLimit) return FNB_REJECTED;  // n beyond ~11 000 columns
    int warps = int((kSmemLimit - fixed) / per_warp);
    warps = warps > kMaxWarps ? kMaxWarps : warps;
    const size_t smem = fixed + size_t(warps) * per_warp;
    if (!ensure_configured<NT, Q8>()) return FNB_LAUNCH_FAILED;
    const int64_t n_tiles = (r1 - r0 + 31) / 32;
    const int grid = grid_for((n_tiles + warps - 1) / warps, 16);
    down_rows_kernel<NT, Q8><<<grid, warps * 32, smem, s>>>(w, row_words, nb, act, act_stride, out, out_stride, r0, r1);
    return launch_status();
}

}  // namespace

template <bool Q8>
bool prepare_fmt() {
    return ensure_configured<1, Q8>() && ensure_configured<2, Q8>() && ensure_configured<3, Q8>() &&
           ensure_configured<4, Q8>() && ensure_configured<5, Q8>() && ensure_configured<6, Q8>() &&
           ensure_configured<7, Q8>() && ensure_configured<8, Q8>();
}

// the window in passes of at most eight rows, as the reference's
template <bool Q8>
int32_t launch_window(const uint32_t * w, int row_words, int nb, const uint8_t * act, int64_t act_stride, int32_t nt,
                      float * out, int64_t out_stride, int64_t r0, int64_t r1, cudaStream_t s) {
    for (int t0 = 0; t0 < nt; t0 += kMaxT) {
        const int m = nt - t0 < kMaxT ? nt - t0 : kMaxT;
        const uint8_t * at = act + int64_t(t0) * act_stride;
        float * ot = out + int64_t(t0) * out_stride;
        int32_t st;
        switch (m) {
            case 1: st = launch_nt<1, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 2: st = launch_nt<2, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 3: st = launch_nt<3, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 4: st = launch_nt<4, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 5: st = launch_nt<5, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 6: st = launch_nt<6, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            case 7: st = launch_nt<7, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
            default: st = launch_nt<8, Q8>(w, row_words, nb, at, act_stride, ot, out_stride, r0, r1, s); break;
        }
        if (st != FNB_OK) return st;
    }
    return FNB_OK;
}

bool expert_down_prepare_device() { return prepare_fmt<false>() && prepare_fmt<true>(); }

}  // namespace fnb

extern "C" int32_t fnb_expert_down_rows_q5_1(const void * w, int64_t row_bytes, int32_t n, const void * act,
                                             int64_t act_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0,
                                             int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(w, 8) || !ok_ptr(act, 4) || !ok_ptr(out, 4)) return FNB_REJECTED;
    if (n < 32 || n > 16384 || n % 32 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 32;
    if (row_bytes < int64_t(nb) * 24 || row_bytes % 4 != 0 || row_bytes != int64_t(nb) * 24) return FNB_REJECTED;  // rows back to back
    if (act_stride < int64_t(nb) * 36 || act_stride % 4 != 0 || out_stride < r1) return FNB_REJECTED;
    return launch_window<false>(static_cast<const uint32_t *>(w), nb * 6, nb, static_cast<const uint8_t *>(act), act_stride, nt,
                                out, out_stride, r0, r1, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_expert_down_rows_q8_0(const void * w, int64_t row_bytes, int32_t n, const void * act,
                                             int64_t act_stride, int32_t nt, float * out, int64_t out_stride, int64_t r0,
                                             int64_t r1, void * stream) {
    using namespace fnb;
    if (!ok_ptr(w, 8) || !ok_ptr(act, 2) || !ok_ptr(out, 4)) return FNB_REJECTED;
    // rows of whole 8-byte pairs: n a multiple of 128 (34-byte blocks, four to 136 bytes)
    if (n < 128 || n > 16384 || n % 128 != 0 || nt < 1 || nt > 64 || r0 < 0 || r1 <= r0 || r1 - r0 > INT32_MAX) return FNB_REJECTED;
    const int nb = n / 32;
    if (row_bytes != int64_t(nb) * 34 || act_stride < int64_t(nb) * 34 || act_stride % 2 != 0 || out_stride < r1) return FNB_REJECTED;
    return launch_window<true>(static_cast<const uint32_t *>(w), nb * 17 / 2, nb, static_cast<const uint8_t *>(act), act_stride,
                               nt, out, out_stride, r0, r1, static_cast<cudaStream_t>(stream));
}

