// Reading the 8-bit KV cache back as F32: the read format of whatever consumes the cache the rope / append kernel
// writes (attention widens cells exactly like this before its dot products).  One cache row is a (cell, kv head) pair
// of head_dim values:
//   Q8_0 cells:  value = fp16 d x code           (ggml dequantize_row_q8_0, ggml/src/ggml-quants.c:551-565)
//   KV8:         value = float(code) x f32(scale of the value's group of 64), exact in F32
//                (fn::qsa::kv8::decode4, fn/kernels/qsa/kv_q8.cuh:61-67; CPU: fn::quant::kv_q8_value)
// HBM-bound and write-dominated (272 or 264 bytes read, 1024 written per 256-value row): a warp takes a row, every
// lane eight consecutive values, two 128-bit streaming stores per lane; many more CTAs than are resident, as in
// get_rows, so that SMs which drain slower get fewer rows.
#include "common.cuh"

namespace fnb {
namespace {

constexpr int kWarpsPerCta = 8;

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
    for (int64_t r0 = warp * rows_per_warp; r0 < n_rows; r0 += n_warps * rows_per_warp) {
        const int64_t r = r0 + rw;
        if (r >= n_rows) continue;
        const int64_t t = r / p.n_kv;
        const int h = int(r - t * p.n_kv);
        const int64_t cell = p.cells != nullptr ? int64_t(__ldg(p.cells + t)) : p.cell0 + t;
        if (cell < 0 || cell >= p.cache_slots) {
            if (sub == 0 && p.err != nullptr) atomicOr(p.err, FNB_ERR_SLOT);
            continue;
        }
        const int64_t c = cell * p.n_kv + h;
        uint32_t w0, w1;
        float s;
        if (KV8) {
            const uint2 w = __ldg(reinterpret_cast<const uint2 *>(p.cache + c * HD) + sub);
            w0 = w.x, w1 = w.y;
            s = f16_bits_to_f32(__ldg(p.scale + c * (HD / 64) + sub / 8));
        } else {
            // a 34-byte block: fp16 d, 32 codes; this lane's eight codes start 2 + 8 (sub % 4) bytes into block sub / 4
            const uint16_t * blk = reinterpret_cast<const uint16_t *>(p.cache + (c * (HD / 32) + sub / 4) * 34);
            s = f16_bits_to_f32(__ldg(blk));
            const uint16_t * q = blk + 1 + 4 * (sub % 4);
            w0 = uint32_t(__ldg(q)) | (uint32_t(__ldg(q + 1)) << 16);
            w1 = uint32_t(__ldg(q + 2)) | (uint32_t(__ldg(q + 3)) << 16);
        }
        float4 * dst = reinterpret_cast<float4 *>(p.out + r * HD) + 2 * sub;
        st_stream(dst, widen4(w0, s));
        st_stream(dst + 1, widen4(w1, s));
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
    const int64_t warps = (a->rows * a->n_kv_heads + rows_per_warp - 1) / rows_per_warp;
    const int grid = grid_for((warps + kWarpsPerCta - 1) / kWarpsPerCta, 32);
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a->scale != nullptr) {
        kv_read_kernel<true><<<grid, kWarpsPerCta * 32, 0, s>>>(p);
    } else {
        kv_read_kernel<false><<<grid, kWarpsPerCta * 32, 0, s>>>(p);
    }
    return launch_status();
}
