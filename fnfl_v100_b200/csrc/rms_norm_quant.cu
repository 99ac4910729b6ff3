// Hidden RMSNorm fused with requantisation of its output: the activation a quantised mat-vec consumes next is
// written once, as 8-bit blocks, instead of being written as F32 and read back by a separate quantise launch.
// The reference fuses the same pair (its split hidden norm writes the activation format directly:
// fn/kernels/draft/draft_in.cu:124-130).
//
//   y = (x * scale) * w, scale = 1 / sqrtf(mean(x^2) + eps)     (as fnb_rms_norm_f32, sum of squares in double)
//   every 32 values of y -> one Q8_1 / Q8_0 block, or the reference's activation format
//
// HBM-bound: 4 bytes read and 1.06 - 1.25 written per value.  Same pipeline shape as the SwiGLU kernel: one producer
// lane streams tiles of four rows (one bulk copy per tile) into a ring of shared-memory stages; consumer warps take a
// row each.  A lane owns whole blocks (block b = lane, lane + 32, ...), reads them in rotated 16-byte chunks
// (conflict-free), and RELEASES THE STAGE AS SOON AS THE ROW IS IN REGISTERS (the release is made to depend on every
// loaded value), so nearly the whole ring is in flight.
// amax, code sums and block headers are in-lane; only the row's sum of squares crosses lanes (one 5-step butterfly).
//
// Tiles go to the consumer groups in turn (tile i of a CTA to group i mod groups) and stage i mod stages holds it.
// A group's parity waits on a stage are only sound while the ring is at least as deep as the number of groups
// taking tiles (then the fill a group waits for is at most one phase past the last one the producer's own order
// guarantees consumed); wide rows leave room for fewer stages than there are groups, so the launcher then runs
// only `stages` groups and the other warps idle.
// All barrier waits are bounded; a wait that gives up sets FNB_ERR_TIMEOUT in the caller's error word (when one is
// given), consumers return and the producer stays until every copy it issued has landed.
#include <atomic>

#include "bulk_pipe.cuh"

namespace fnb {
namespace {

enum class out_fmt { q8_1, q8_0, act };
template <out_fmt F>
__host__ __device__ constexpr int block_bytes() {
    return F == out_fmt::q8_1 ? 36 : F == out_fmt::q8_0 ? 34 : 32;
}

constexpr int kGroups = 5;      // 15 consumer warps + the producer = 16 warps, four per scheduler: 128 registers each, a row of 2048 fits
constexpr int kGroupWarps = 3;  // rows per tile
constexpr int kConsumerWarps = kGroups * kGroupWarps;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr size_t kSmemBudget = 220 * 1024;

__device__ __forceinline__ float amax4(float4 v) { return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))); }
__device__ __forceinline__ double sq4(double acc, float4 v) {
    acc = __dadd_rn(acc, double(__fmul_rn(v.x, v.x)));
    acc = __dadd_rn(acc, double(__fmul_rn(v.y, v.y)));
    acc = __dadd_rn(acc, double(__fmul_rn(v.z, v.z)));
    return __dadd_rn(acc, double(__fmul_rn(v.w, v.w)));
}

// BPL: blocks per lane (cols <= 1024 BPL); F32OUT: also store the normalised row
template <out_fmt F, int BPL, bool F32OUT>
__global__ void __launch_bounds__(kThreads, 1)
    rms_norm_quant_kernel(const float * __restrict__ x, const float * __restrict__ w, float eps, uint8_t * __restrict__ out,
                          float * __restrict__ scales, float * __restrict__ out_f32, int64_t rows, int cols, int stages,
                          int groups, uint32_t * err) {
    constexpr int BB = block_bytes<F>();
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const int nb = cols / 32;                            // blocks per row
    const uint32_t row_bytes = uint32_t(cols) * 4;
    const uint32_t tile_bytes = row_bytes * kGroupWarps;
    const int row_out = nb * BB;                         // output bytes per row
    const int row_out_pad = (row_out + 15) & ~15;
    uint8_t * data = smem;                                                      // [stages][4][row_bytes]
    float * wsm = reinterpret_cast<float *>(data + size_t(stages) * tile_bytes);  // [cols]
    uint8_t * outs = reinterpret_cast<uint8_t *>(wsm + cols);                     // [warps][row_out_pad]
    uint64_t * full = reinterpret_cast<uint64_t *>(outs + size_t(kConsumerWarps) * row_out_pad);
    uint64_t * empty = full + stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGroupWarps);
        }
        mbar_init_fence();
    }
    __syncthreads();  // nothing slow before this point: the producer starts streaming at once
    pdl_wait();       // the predecessor's writes are visible from here on; no global memory was touched before

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t n_tiles = (rows + kGroupWarps - 1) / kGroupWarps;

    if (wid == kConsumerWarps) {
        if (lane != 0) return;
        const uint64_t policy = l2_evict_first_policy();
        int it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            const int s = it % stages;
            if (it >= stages && !mbar_wait(&empty[s], (uint32_t(it / stages) & 1u) ^ 1u, err)) {
                ok = false;
                break;
            }
            const int64_t r0 = tile * kGroupWarps;
            const uint32_t bytes = uint32_t(rows - r0 < kGroupWarps ? rows - r0 : kGroupWarps) * row_bytes;
            mbar_expect_tx(&full[s], bytes);
            bulk_g2s(data + size_t(s) * tile_bytes, x + r0 * cols, bytes, &full[s], policy);
            mbar_arrive(&full[s]);
        }
        // the producer leaves last: every copy it issued has landed before the CTA's shared memory is released
        (void) ok;
        for (int j = 1; j <= stages && j <= it; ++j) {
            const int its = it - j;
            mbar_wait_landed(&full[its % stages], uint32_t(its / stages) & 1u);
        }
        return;
    }

    // the weights reach shared memory while the first tiles are in flight (every consumer warp helps, then the idle
    // groups leave)
    for (int i = threadIdx.x; i < cols; i += kConsumerWarps * 32) wsm[i] = w != nullptr ? __ldg(w + i) : 1.0f;
    named_barrier<1>(kConsumerWarps * 32);
    const int grp = wid / kGroupWarps, gw = wid - grp * kGroupWarps;
    if (grp >= groups) return;  // a ring shallower than kGroups is shared by `groups` groups only
    uint8_t * my_out = outs + size_t(wid) * row_out_pad;

    int it = 0;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
        if (it % groups != grp) continue;
        const int s = it % stages;
        const uint32_t fill = uint32_t(it / stages);
        // successive fills of a stage go to different groups: wait for the previous fill to have been consumed before
        // trusting the parity of this one (a parity wait is only meaningful at most one phase ahead; stages >= groups
        // keeps the empty barrier itself within one phase of this group's view)
        if (fill > 0 && !mbar_wait(&empty[s], (fill - 1u) & 1u, err)) return;
        if (!mbar_wait(&full[s], fill & 1u, err)) return;
        const int64_t row = tile * kGroupWarps + gw;
        const bool live = row < rows;
        const uint8_t * src = data + size_t(s) * tile_bytes + size_t(live ? gw : 0) * row_bytes;

        float4 v[BPL][8];
#pragma unroll
        for (int k = 0; k < BPL; ++k) {
            const int b = lane + 32 * k;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = (j + lane) & 7;
                v[k][j] = b < nb ? *reinterpret_cast<const float4 *>(src + 128 * b + 16 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // The stage is handed back as soon as the row is in registers - and no sooner: the arrive is predicated on a
        // cheap value computed from EVERY loaded register (a packed F32 sum; no addition yields the all-ones pattern,
        // so the predicate is always true), which keeps it behind the completion of all the loads above in any
        // schedule, instead of resting on the ordering of a release that follows loads nothing has consumed yet.
        f32x2 touch[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int k = 0; k < BPL; ++k) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                touch[j & 3] = add2(touch[j & 3], pk(v[k][j].x, v[k][j].y));
                touch[j & 3] = add2(touch[j & 3], pk(v[k][j].z, v[k][j].w));
            }
        }
        float t_lo, t_hi;
        unpk(add2(add2(touch[0], touch[1]), add2(touch[2], touch[3])), t_lo, t_hi);
        const bool landed = __float_as_uint(__fadd_rn(t_lo, t_hi)) != 0xffffffffu;
        __syncwarp();
        if (lane == 0 && landed) mbar_arrive(&empty[s]);  // the row is in registers: the stage can be refilled
        if (!live) continue;                              // uniform over the warp

        // four independent chains (a double tree sum differs from the sequential one far below the F32 narrowing)
        double a4[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int k = 0; k < BPL; ++k) {
#pragma unroll
            for (int j = 0; j < 8; ++j) a4[j & 3] = sq4(a4[j & 3], v[k][j]);
        }
        double acc = warp_sum_f64(__dadd_rn(__dadd_rn(a4[0], a4[1]), __dadd_rn(a4[2], a4[3])));
        const double m = (cols & (cols - 1)) == 0 ? __dmul_rn(acc, 1.0 / double(cols)) : __ddiv_rn(acc, double(cols));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__double2float_rn(m), eps)));

#pragma unroll
        for (int k = 0; k < BPL; ++k) {
            const int b = lane + 32 * k;
            if (b >= nb) continue;  // (not `break`: the loop must stay fully unrolled so v[][] lives in registers)
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c = (j + lane) & 7;
                const float4 g = *reinterpret_cast<const float4 *>(wsm + 32 * b + 4 * c);
                float4 y = v[k][j];
                y.x = __fmul_rn(__fmul_rn(y.x, scale), g.x);
                y.y = __fmul_rn(__fmul_rn(y.y, scale), g.y);
                y.z = __fmul_rn(__fmul_rn(y.z, scale), g.z);
                y.w = __fmul_rn(__fmul_rn(y.w, scale), g.w);
                v[k][j] = y;
                amax = fmaxf(amax, amax4(y));
                if (F32OUT) st_stream(reinterpret_cast<float4 *>(out_f32 + row * cols + 32 * b) + c, y);
            }
            int qsum = 0;
            if (F == out_fmt::q8_1) {
                const ggml_q8_rule rule(amax);
                uint32_t * o = reinterpret_cast<uint32_t *>(my_out) + 9 * b;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t wd = rule.code4(v[k][j]);
                    qsum += sum4_i8(wd);
                    o[1 + ((j + lane) & 7)] = wd;
                }
                o[0] = uint32_t(f32_to_f16_bits(rule.d)) | (uint32_t(f32_to_f16_bits(__fmul_rn(float(qsum), rule.d))) << 16);
            } else if (F == out_fmt::q8_0) {
                const ggml_q8_rule rule(amax);
                uint16_t * o = reinterpret_cast<uint16_t *>(my_out) + 17 * b;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t wd = rule.code4(v[k][j]);
                    const int c = (j + lane) & 7;
                    o[1 + 2 * c] = uint16_t(wd);
                    o[2 + 2 * c] = uint16_t(wd >> 16);
                }
                o[0] = f32_to_f16_bits(rule.d);
            } else {
                const act_rule rule(amax);
                uint32_t * o = reinterpret_cast<uint32_t *>(my_out) + 8 * b;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t wd = rule.code4(v[k][j]);
                    qsum += sum4_i8(wd);
                    o[(j + lane) & 7] = wd;
                }
                st_stream(reinterpret_cast<uint2 *>(scales) + row * nb + b,
                          make_uint2(__float_as_uint(rule.d), __float_as_uint(__fmul_rn(rule.d, float(qsum)))));
            }
        }
        __syncwarp();
        uint8_t * dst = out + row * int64_t(row_out);
        if ((row_out & 15) == 0) {  // every row of the output starts 16-byte aligned
            for (int i = lane; i < row_out / 16; i += 32) {
                st_stream(reinterpret_cast<uint4 *>(dst) + i, reinterpret_cast<const uint4 *>(my_out)[i]);
            }
        } else {
            for (int i = lane * 2; i < row_out; i += 64) {
                *reinterpret_cast<uint16_t *>(dst + i) = *reinterpret_cast<const uint16_t *>(my_out + i);
            }
        }
        __syncwarp();
    }
}

// raises the kernel's dynamic shared-memory limit once per device
template <out_fmt F, int BPL, bool F32OUT>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(rms_norm_quant_kernel<F, BPL, F32OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kSmemBudget)) != cudaSuccess) {
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}
template <out_fmt F>
bool prepare_fmt() {
    return ensure_configured<F, 1, false>() && ensure_configured<F, 1, true>() && ensure_configured<F, 2, false>() &&
           ensure_configured<F, 2, true>() && ensure_configured<F, 3, false>() && ensure_configured<F, 3, true>() &&
           ensure_configured<F, 4, false>() && ensure_configured<F, 4, true>();
}

template <out_fmt F, int BPL, bool F32OUT>
int32_t launch_one(const float * x, const float * w, float eps, uint8_t * out, float * scales, float * out_f32, int64_t rows,
                   int32_t cols, uint32_t * err, cudaStream_t s) {
    constexpr int BB = block_bytes<F>();
    const size_t tile = size_t(cols) * 4 * kGroupWarps;
    const size_t row_out_pad = (size_t(cols / 32) * BB + 15) & ~size_t(15);
    const size_t fixed = size_t(cols) * 4 + size_t(kConsumerWarps) * row_out_pad + 256;
    int stages = int((kSmemBudget - fixed) / tile);
    stages = stages > 8 ? 8 : stages;
    if (stages < 2) return FNB_REJECTED;
    const size_t smem = size_t(stages) * tile + fixed;

    if (!ensure_configured<F, BPL, F32OUT>()) return FNB_LAUNCH_FAILED;
    const int64_t n_tiles = (rows + kGroupWarps - 1) / kGroupWarps;
    const int grid = int(n_tiles < kSmCount ? n_tiles : kSmCount);
    const int groups = stages < kGroups ? stages : kGroups;
    launch_pdl(rms_norm_quant_kernel<F, BPL, F32OUT>, grid, kThreads, smem, s, x, w, eps, out, scales, out_f32, rows, cols, stages,
               groups, err);
    return launch_status();
}

template <out_fmt F>
int32_t launch(const float * x, const float * w, float eps, void * out, float * scales, float * out_f32, int64_t rows,
               int32_t cols, uint32_t * err, cudaStream_t s) {
    if (!ok_ptr(x, 16) || !ok_opt(w, 16) || !ok_ptr(out, 16) || !ok_opt(out_f32, 16) || !ok_opt(err, 4)) return FNB_REJECTED;
    if (F == out_fmt::act && !ok_ptr(scales, 8)) return FNB_REJECTED;
    if (rows < 1 || rows > INT32_MAX || cols < 32 || cols > 4096 || cols % 32 != 0 || !(eps >= 0.0f)) return FNB_REJECTED;
    uint8_t * o = static_cast<uint8_t *>(out);
    const int bpl = (cols / 32 + 31) / 32;
    const bool f = out_f32 != nullptr;
#define FNB_CASE(B)                                                                                   \
    case B:                                                                                           \
        return f ? launch_one<F, B, true>(x, w, eps, o, scales, out_f32, rows, cols, err, s)          \
                 : launch_one<F, B, false>(x, w, eps, o, scales, nullptr, rows, cols, err, s);
    switch (bpl) {
        FNB_CASE(1)
        FNB_CASE(2)
        FNB_CASE(3)
        FNB_CASE(4)
        default: return FNB_REJECTED;
    }
#undef FNB_CASE
}

}  // namespace

bool rms_norm_quant_prepare_device() {
    return prepare_fmt<out_fmt::q8_1>() && prepare_fmt<out_fmt::q8_0>() && prepare_fmt<out_fmt::act>();
}

}  // namespace fnb

extern "C" int32_t fnb_rms_norm_q8_1(const float * x, const float * w, float eps, void * out_q8_1, float * out_f32,
                                     int64_t rows, int32_t cols, uint32_t * err, void * stream) {
    return fnb::launch<fnb::out_fmt::q8_1>(x, w, eps, out_q8_1, nullptr, out_f32, rows, cols, err,
                                          static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_rms_norm_q8_0(const float * x, const float * w, float eps, void * out_q8_0, float * out_f32,
                                     int64_t rows, int32_t cols, uint32_t * err, void * stream) {
    return fnb::launch<fnb::out_fmt::q8_0>(x, w, eps, out_q8_0, nullptr, out_f32, rows, cols, err,
                                          static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_rms_norm_act(const float * x, const float * w, float eps, int8_t * codes, float * scales,
                                    float * out_f32, int64_t rows, int32_t cols, uint32_t * err, void * stream) {
    return fnb::launch<fnb::out_fmt::act>(x, w, eps, codes, scales, out_f32, rows, cols, err,
                                          static_cast<cudaStream_t>(stream));
}
