// Reading the 8-bit KV cache back as F32: the read format of whatever consumes the cache the rope / append kernel
// writes (attention widens cells exactly like this before its dot products).  One cache row is a (cell, kv head) pair
// of head_dim values:
//   Q8_0 cells:  value = fp16 d x code           (ggml dequantize_row_q8_0, ggml/src/ggml-quants.c:551-565)
//   KV8:         value = float(code) x f32(scale of the value's group of 64), exact in F32
//                (fn::qsa::kv8::decode4, fn/kernels/qsa/kv_q8.cuh:61-67; CPU: fn::quant::kv_q8_value)
// HBM-bound and write-dominated (272 or 264 bytes read, 1024 written per 256-value row): a warp takes a row, every
// lane two groups of four values half a row apart, two 128-bit streaming stores per lane; many more CTAs than are resident, as in
// get_rows, so that SMs which drain slower get fewer rows.
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kUnroll = 4;  // cache rows a warp has in flight

struct kv_read_params {
    const uint8_t * cache;
    const uint16_t * scale;  // KV8 scale plane, or null: Q8_0 cells
    const int32_t * cells;   // [rows] or null: cell0 + row
    float * out;
    uint32_t * err;
    int64_t rows, cache_slots, cell0;
    int n_kv, head_dim;
};

// 0x4B0000bb - 2^23 = bb for a byte; codes are signed, so the byte is biased by 128 first (the reference's decode4)
__device__ __forceinline__ float4 widen4(uint32_t w, float s) {
    const uint32_t b = w ^ 0x80808080u;
    float4 r;
    r.x = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(b, 0x4b000000u, 0x7650u)), -8388736.0f), s);
    r.y = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(b, 0x4b000000u, 0x7651u)), -8388736.0f), s);
    r.z = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(b, 0x4b000000u, 0x7652u)), -8388736.0f), s);
    r.w = __fmul_rn(__fadd_rn(__uint_as_float(__byte_perm(b, 0x4b000000u, 0x7653u)), -8388736.0f), s);
    return r;
}

template <bool KV8>
__global__ void __launch_bounds__(kWarpsPerCta * 32) kv_read_kernel(const kv_read_params p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int HD = p.head_dim;
    const int64_t n_rows = p.rows * p.n_kv;  // (row, head) pairs
    const int per_row = HD / 8;              // lanes that hold values (32 for 256, 16 for 128, 8 for 64)
    const int rows_per_warp = 32 / per_row;
    const int sub = lane % per_row, rw = lane / per_row;
    // kUnroll rows' loads are issued before the first is widened and stored: one row per trip left the kernel waiting
    // on its own loads (79 % of the HBM roofline at 262144 cells)
    for (int64_t base = warp * kUnroll * rows_per_warp; base < n_rows; base += n_warps * kUnroll * rows_per_warp) {
        uint32_t w0[kUnroll], w1[kUnroll];
        float s0[kUnroll], s1[kUnroll];
        int64_t row[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int64_t r = base + int64_t(j) * rows_per_warp + rw;
            row[j] = -1;
            if (r >= n_rows) continue;
            const int64_t t = r / p.n_kv;
            const int h = int(r - t * p.n_kv);
            const int64_t cell = p.cells != nullptr ? int64_t(__ldg(p.cells + t)) : p.cell0 + t;
            if (cell < 0 || cell >= p.cache_slots) {
                if (sub == 0 && p.err != nullptr) atomicOr(p.err, FNB_ERR_SLOT);
                continue;
            }
            row[j] = r;
            const int64_t c = cell * p.n_kv + h;
            // the lane takes code words `sub` and `sub + per_row` of the row (four codes each), so that each of its two
            // store instructions writes per_row x 16 contiguous bytes; with eight adjacent codes per lane every store
            // instruction wrote half of each 32-byte sector it touched
            const int k0 = sub, k1 = sub + per_row;
            if (KV8) {
                const uint32_t * w = reinterpret_cast<const uint32_t *>(p.cache + c * HD);
                w0[j] = __ldg(w + k0), w1[j] = __ldg(w + k1);
                const uint16_t * sc = p.scale + c * (HD / 64);
                s0[j] = f16_bits_to_f32(__ldg(sc + k0 / 16)), s1[j] = f16_bits_to_f32(__ldg(sc + k1 / 16));
            } else {
                // 34-byte blocks: fp16 d, 32 codes; code word k is bytes 2 + 4 (k % 8) .. of block k / 8 (2-byte aligned)
                const uint16_t * b0 = reinterpret_cast<const uint16_t *>(p.cache + (c * (HD / 32) + k0 / 8) * 34);
                const uint16_t * b1 = reinterpret_cast<const uint16_t *>(p.cache + (c * (HD / 32) + k1 / 8) * 34);
                s0[j] = f16_bits_to_f32(__ldg(b0)), s1[j] = f16_bits_to_f32(__ldg(b1));
                const uint16_t * q0 = b0 + 1 + 2 * (k0 % 8);
                const uint16_t * q1 = b1 + 1 + 2 * (k1 % 8);
                w0[j] = uint32_t(__ldg(q0)) | (uint32_t(__ldg(q0 + 1)) << 16);
                w1[j] = uint32_t(__ldg(q1)) | (uint32_t(__ldg(q1 + 1)) << 16);
            }
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            if (row[j] < 0) continue;
            float4 * dst = reinterpret_cast<float4 *>(p.out + row[j] * HD) + sub;
            st_stream(dst, widen4(w0[j], s0[j]));
            st_stream(dst + per_row, widen4(w1[j], s1[j]));
        }
    }
}

// Q8_0 cells of 256 values are 272 bytes = 17 x 16, 16-byte aligned: 17 lanes fetch a row with one 128-bit load each
// and park it in the warp's shared-memory slot, from which every lane picks its two code words and their d (the
// blocks are only 2-byte aligned, and six 2-byte GLOBAL loads per lane and row held this format at 71 % of the
// roofline where KV8 ran at 93 %).
__global__ void __launch_bounds__(kWarpsPerCta * 32) kv_read_q8_0_256_kernel(const kv_read_params p) {
    __shared__ __align__(16) uint8_t s_rows[kWarpsPerCta][kUnroll][272];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp = int64_t(blockIdx.x) * kWarpsPerCta + wid;
    const int64_t n_warps = int64_t(gridDim.x) * kWarpsPerCta;
    const int64_t n_rows = p.rows * p.n_kv;
    for (int64_t base = warp * kUnroll; base < n_rows; base += n_warps * kUnroll) {
        uint4 v[kUnroll];
        bool live[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            const int64_t r = base + j;
            live[j] = false;
            if (r >= n_rows) continue;
            const int64_t t = r / p.n_kv;
            const int h = int(r - t * p.n_kv);
            const int64_t cell = p.cells != nullptr ? int64_t(__ldg(p.cells + t)) : p.cell0 + t;
            if (cell < 0 || cell >= p.cache_slots) {
                if (lane == 0 && p.err != nullptr) atomicOr(p.err, FNB_ERR_SLOT);
                continue;
            }
            live[j] = true;
            if (lane < 17) v[j] = __ldg(reinterpret_cast<const uint4 *>(p.cache + (cell * p.n_kv + h) * 272) + lane);
        }
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            if (live[j] && lane < 17) reinterpret_cast<uint4 *>(s_rows[wid][j])[lane] = v[j];
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kUnroll; ++j) {
            if (!live[j]) continue;
            // code word k: bytes 2 + 4 (k % 8) .. of block k / 8; the lane takes words `lane` and `lane + 32`
            const uint16_t * b0 = reinterpret_cast<const uint16_t *>(s_rows[wid][j] + (lane / 8) * 34);
            const uint16_t * b1 = b0 + 4 * 17;
            const uint16_t * q0 = b0 + 1 + 2 * (lane % 8);
            const uint16_t * q1 = b1 + 1 + 2 * (lane % 8);
            const uint32_t w0 = uint32_t(q0[0]) | (uint32_t(q0[1]) << 16), w1 = uint32_t(q1[0]) | (uint32_t(q1[1]) << 16);
            float4 * dst = reinterpret_cast<float4 *>(p.out + (base + j) * 256) + lane;
            st_stream(dst, widen4(w0, f16_bits_to_f32(b0[0])));
            st_stream(dst + 32, widen4(w1, f16_bits_to_f32(b1[0])));
        }
        __syncwarp();
    }
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_kv_read_f32(const fnb_kv_read_args * a, void * stream) {
    using namespace fnb;
    if (a == nullptr || !ok_ptr(a->cache, 16) || !ok_ptr(a->out, 16) || !ok_opt(a->scale, 2) || !ok_opt(a->cells, 4) ||
        !ok_opt(a->err, 4)) {
        return FNB_REJECTED;
    }
    if (a->rows < 1 || a->rows > INT32_MAX || a->cache_slots < 1 || a->n_kv_heads < 1 || a->n_kv_heads > 64) return FNB_REJECTED;
    if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return FNB_REJECTED;
    if (a->cells == nullptr && (a->cell0 < 0 || a->cell0 + a->rows > a->cache_slots)) return FNB_REJECTED;
    kv_read_params p;
    p.cache = static_cast<const uint8_t *>(a->cache), p.scale = a->scale, p.cells = a->cells, p.out = a->out, p.err = a->err;
    p.rows = a->rows, p.cache_slots = a->cache_slots, p.cell0 = a->cell0, p.n_kv = a->n_kv_heads, p.head_dim = a->head_dim;
    const int rows_per_warp = 32 / (a->head_dim / 8);
    const int64_t per_warp = int64_t(rows_per_warp) * kUnroll;
    const int64_t warps = (a->rows * a->n_kv_heads + per_warp - 1) / per_warp;
    const int grid = grid_for((warps + kWarpsPerCta - 1) / kWarpsPerCta, 32);
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a->scale != nullptr) {
        kv_read_kernel<true><<<grid, kWarpsPerCta * 32, 0, s>>>(p);
    } else if (a->head_dim == 256) {
        kv_read_q8_0_256_kernel<<<grid, kWarpsPerCta * 32, 0, s>>>(p);
    } else {
        kv_read_kernel<false><<<grid, kWarpsPerCta * 32, 0, s>>>(p);
    }
    return launch_status();
}
