// Per-head RMSNorm (optional) -> NeoX partial-rotary RoPE -> Q written back in F32, K and V quantised and
// appended to the 8-bit KV cache at the token's slot.  One launch does what the CPU graph does in five ops.
//
// HBM-bound and copy-like: per token (16 Q heads, 2 KV heads of 256) 20 KiB are read, 16 KiB of Q written
// and 1088 bytes of cache cells written; arithmetic is a handful of flops per value plus 32 sin/cos per token.
//
// Layout in HBM: q [rows][n_q][hd], k, v [rows][n_kv][hd] dense F32; caches are [slot][kv_head][hd/32] Q8_0
// blocks (a 256-wide head is 272 bytes = 17 x 16, so every cell starts 16-byte aligned), or for the
// reference's own format int8 codes [slot][kv_head][hd] with FP16 scales [slot][kv_head][hd/64].
//
// Work decomposition: one CTA per token.  A warp owns a head row (hd/32 consecutive values per lane, which
// keeps a Q8_0 block inside 32/(hd/32) neighbouring lanes and a rotary pair at a fixed lane distance) and
// takes two rows per trip so a lane has four 128-bit loads in flight.  The token's 32 (cos, sin) pairs are
// computed once per CTA into shared memory while those loads are in flight: the angle is the F32 product
// chain pos * ts^i, and sin/cos are evaluated bit-identically to the host C library (exact_math.cuh).
// Cells are assembled in shared memory and leave as aligned 128-bit stores.
#include "common.cuh"
#include "exact_math.cuh"
#include "rope_kv.cuh"

namespace fnb {
namespace {

template <int EPL>
struct row_regs {
    float v[EPL];
};

template <int EPL>
__device__ __forceinline__ void load_row(row_regs<EPL> & r, const float * src, int lane) {
    if constexpr (EPL == 8) {
        const float4 a = ld_stream(reinterpret_cast<const float4 *>(src) + 2 * lane);
        const float4 b = ld_stream(reinterpret_cast<const float4 *>(src) + 2 * lane + 1);
        r.v[0] = a.x, r.v[1] = a.y, r.v[2] = a.z, r.v[3] = a.w;
        r.v[4] = b.x, r.v[5] = b.y, r.v[6] = b.z, r.v[7] = b.w;
    } else if constexpr (EPL == 4) {
        const float4 a = ld_stream(reinterpret_cast<const float4 *>(src) + lane);
        r.v[0] = a.x, r.v[1] = a.y, r.v[2] = a.z, r.v[3] = a.w;
    } else {
        const float2 a = __ldcs(reinterpret_cast<const float2 *>(src) + lane);
        r.v[0] = a.x, r.v[1] = a.y;
    }
}

template <int EPL>
__device__ __forceinline__ void store_row(const row_regs<EPL> & r, float * dst, int lane) {
    if constexpr (EPL == 8) {
        st_stream(reinterpret_cast<float4 *>(dst) + 2 * lane, make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
        st_stream(reinterpret_cast<float4 *>(dst) + 2 * lane + 1, make_float4(r.v[4], r.v[5], r.v[6], r.v[7]));
    } else if constexpr (EPL == 4) {
        st_stream(reinterpret_cast<float4 *>(dst) + lane, make_float4(r.v[0], r.v[1], r.v[2], r.v[3]));
    } else {
        __stcs(reinterpret_cast<float2 *>(dst) + lane, make_float2(r.v[0], r.v[1]));
    }
}

// y = (x * scale) * w over the warp's row of 32 * EPL values
template <int EPL>
__device__ __forceinline__ void head_norm(row_regs<EPL> & r, const float * __restrict__ w, float eps, int lane) {
    double acc = 0.0;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc = __dadd_rn(acc, double(__fmul_rn(r.v[e], r.v[e])));
    acc = warp_sum_f64(acc);
    const float mean = __double2float_rn(__dmul_rn(acc, 1.0 / double(32 * EPL)));  // a power of two: exact, as the division is
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll
    for (int e = 0; e < EPL; ++e) r.v[e] = __fmul_rn(__fmul_rn(r.v[e], scale), __ldg(w + lane * EPL + e));
}

// pairs (i, i + half): the partner of a lane's e-th value is the e-th value of the lane half/EPL away
template <int EPL>
__device__ __forceinline__ void rope(row_regs<EPL> & r, const float2 * cs, int half, int lane) {
    const int dist = half / EPL;
    const bool rot = lane < 2 * dist;
    const bool low = lane < dist;
    const int partner = rot ? (low ? lane + dist : lane - dist) : lane;
    const int pair0 = (low ? lane : lane - dist) * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const float other = __shfl_sync(kFull, r.v[e], partner);
        if (rot) {
            const float2 t = cs[pair0 + e];  // (cos, sin)
            r.v[e] = low ? __fsub_rn(__fmul_rn(r.v[e], t.x), __fmul_rn(other, t.y))   // x0 c - x1 s
                         : __fadd_rn(__fmul_rn(other, t.y), __fmul_rn(r.v[e], t.x));  // x0 s + x1 c
        }
    }
}

// one head row -> hd/32 Q8_0 blocks at dst (16-byte aligned), staged through the warp's shared slot
template <int EPL>
__device__ __forceinline__ void put_q8_0(const row_regs<EPL> & r, uint8_t * dst, uint8_t * slot, int lane) {
    constexpr int G = 32 / EPL;  // lanes per block
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(r.v[e]));
    amax = group_max<G>(amax);
    const ggml_q8_rule rule(amax);
    const int blk = lane / G, pos = lane % G;
    uint16_t * s16 = reinterpret_cast<uint16_t *>(slot) + blk * 17;
    if (pos == 0) s16[0] = f32_to_f16_bits(rule.d);
#pragma unroll
    for (int e = 0; e < EPL; e += 2) {
        s16[1 + (pos * EPL + e) / 2] = uint16_t(__byte_perm(rule.code(r.v[e]), rule.code(r.v[e + 1]), 0x0040));
    }
    __syncwarp();
    // a 256-wide head is 272 bytes (17 x 16), a 128-wide one 136 (17 x 8), a 64-wide one 68 (17 x 4): the cell's
    // alignment, and so the widest store that is always legal, shrinks with the head
    if (lane < 17) {
        if constexpr (EPL == 8) {
            st_stream(reinterpret_cast<uint4 *>(dst) + lane, reinterpret_cast<const uint4 *>(slot)[lane]);
        } else if constexpr (EPL == 4) {
            st_stream(reinterpret_cast<uint2 *>(dst) + lane, reinterpret_cast<const uint2 *>(slot)[lane]);
        } else {
            st_stream(reinterpret_cast<uint32_t *>(dst) + lane, reinterpret_cast<const uint32_t *>(slot)[lane]);
        }
    }
    __syncwarp();
}

// one head row -> int8 codes (hd bytes) and hd/64 FP16 scales, the reference's group-64 rule
template <int EPL>
__device__ __forceinline__ void put_kv8(const row_regs<EPL> & r, uint8_t * codes, uint16_t * scales, int lane) {
    constexpr int G = 64 / EPL;  // lanes per group of 64 values
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(r.v[e]));
    amax = group_max<(G > 32 ? 32 : G)>(amax);
    const uint16_t sb = f32_to_f16_bits(__fdiv_rn(amax, 127.0f));
    const float s = f16_bits_to_f32(sb);
    uint32_t q[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        int c = 0;
        if (s > 0.0f) {
            const float t = rintf(__fdiv_rn(r.v[e], s));
            c = t < -127.0f ? -127 : t > 127.0f ? 127 : __float2int_rz(t);
        }
        q[e] = uint32_t(c) & 0xffu;
    }
    if constexpr (EPL == 8) {
        st_stream(reinterpret_cast<uint2 *>(codes) + lane,
                  make_uint2(q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24),
                             q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24)));
    } else if constexpr (EPL == 4) {
        st_stream(reinterpret_cast<uint32_t *>(codes) + lane, q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24));
    } else {
        reinterpret_cast<uint16_t *>(codes)[lane] = uint16_t(q[0] | (q[1] << 8));
    }
    if (lane % G == 0) scales[lane / G] = sb;
}

using kernel_args = rope_kernel_args;

constexpr int kMaxWarps = 16;

template <int HD, kv_fmt F>
__global__ void __launch_bounds__(kMaxWarps * 32) rope_kv_kernel(const kernel_args a) {
    constexpr int EPL = HD / 32;
    __shared__ float2 s_cs[HD / 2];
    __shared__ __align__(16) uint8_t s_slot[kMaxWarps][288];

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int heads = a.n_q + 2 * a.n_kv;
    const int half = a.n_rot / 2;

    for (int64_t t = blockIdx.x; t < a.rows; t += gridDim.x) {
        const int32_t p = __ldg(a.pos + t);
        const int64_t slot = a.slots != nullptr ? int64_t(__ldg(a.slots + t)) : int64_t(p);
        if (slot < 0 || slot >= a.cache_slots) {  // uniform over the CTA
            if (threadIdx.x == 0 && a.err != nullptr) atomicOr(a.err, FNB_ERR_SLOT);
            continue;
        }
        // this warp's first two rows are requested before the angles are computed
        row_regs<EPL> r[2];
        const float * src[2];
        int head[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            head[j] = wid + j * n_warps;
            const int h = head[j] < heads ? head[j] : 0;
            src[j] = h < a.n_q              ? a.q + (t * a.n_q + h) * HD
                     : h < a.n_q + a.n_kv ? a.k + (t * a.n_kv + (h - a.n_q)) * HD
                                            : a.v + (t * a.n_kv + (h - a.n_q - a.n_kv)) * HD;
            load_row<EPL>(r[j], src[j], lane);
        }
        __syncthreads();  // the previous token's readers of s_cs are done
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float theta = float(a.planes != nullptr ? __ldg(a.planes + 4 * t + rope_plane_of_pair(i)) : p);
            for (int c = 0; c < i; ++c) theta = __fmul_rn(theta, a.theta_scale);
            float sn, cs;
            exact_sincosf(theta, &sn, &cs);
            s_cs[i] = make_float2(cs, sn);
        }
        __syncthreads();

        for (int base = 0; base < heads; base += 2 * n_warps) {
            if (base > 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    head[j] = base + wid + j * n_warps;
                    const int h = head[j] < heads ? head[j] : 0;
                    src[j] = h < a.n_q              ? a.q + (t * a.n_q + h) * HD
                             : h < a.n_q + a.n_kv ? a.k + (t * a.n_kv + (h - a.n_q)) * HD
                                                    : a.v + (t * a.n_kv + (h - a.n_q - a.n_kv)) * HD;
                    load_row<EPL>(r[j], src[j], lane);
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int h = head[j];
                if (h >= heads) continue;  // uniform over the warp
                if (h < a.n_q) {
                    if (a.q_norm_w != nullptr) head_norm<EPL>(r[j], a.q_norm_w, a.eps, lane);
                    if (half > 0) rope<EPL>(r[j], s_cs, half, lane);
                    store_row<EPL>(r[j], a.q_out + (t * a.n_q + h) * HD, lane);
                    continue;
                }
                const bool is_k = h < a.n_q + a.n_kv;
                const int kvh = is_k ? h - a.n_q : h - a.n_q - a.n_kv;
                if (is_k) {
                    if (a.k_norm_w != nullptr) head_norm<EPL>(r[j], a.k_norm_w, a.eps, lane);
                    if (half > 0) rope<EPL>(r[j], s_cs, half, lane);
                    if (a.k_f32 != nullptr) store_row<EPL>(r[j], a.k_f32 + (t * a.n_kv + kvh) * HD, lane);
                }
                const int64_t cell = slot * a.n_kv + kvh;
                if (F == kv_fmt::q8_0) {
                    uint8_t * dst = (is_k ? a.k_cache : a.v_cache) + cell * (EPL * 34);
                    put_q8_0<EPL>(r[j], dst, s_slot[wid], lane);
                } else {
                    uint8_t * dst = (is_k ? a.k_cache : a.v_cache) + cell * HD;
                    uint16_t * sc = (is_k ? a.k_scale : a.v_scale) + cell * (HD / 64);
                    put_kv8<EPL>(r[j], dst, sc, lane);
                }
            }
        }
    }
}

template <kv_fmt F>
int32_t launch(const fnb_rope_kv_args * p, uint16_t * k_scale, uint16_t * v_scale, cudaStream_t s) {
    if (p == nullptr) return FNB_REJECTED;
    const int hd = p->head_dim;
    if (hd != 64 && hd != 128 && hd != 256) return FNB_REJECTED;
    const int epl = hd / 32;
    if (p->rows < 1 || p->rows > INT32_MAX || p->cache_slots < 1 || p->cache_slots > INT32_MAX) return FNB_REJECTED;
    if (p->n_q_heads < 0 || p->n_q_heads > 256 || p->n_kv_heads < 0 || p->n_kv_heads > 256) return FNB_REJECTED;
    if (p->n_q_heads + p->n_kv_heads < 1) return FNB_REJECTED;
    if (p->n_rot < 0 || p->n_rot > hd || p->n_rot % (2 * epl) != 0) return FNB_REJECTED;
    if (!ok_ptr(p->pos, 4) || !ok_opt(p->slots, 4) || !ok_opt(p->err, 4) || !ok_opt(p->planes, 4)) return FNB_REJECTED;
    if (p->planes != nullptr && p->n_rot != 64) return FNB_REJECTED;  // the plane sections are defined for 32 pairs
    if (!ok_opt(p->q_norm_w, 16) || !ok_opt(p->k_norm_w, 16) || !ok_opt(p->k_f32, 16)) return FNB_REJECTED;
    if (p->n_q_heads > 0 && (!ok_ptr(p->q, 16) || !ok_ptr(p->q_out, 16))) return FNB_REJECTED;
    if (p->n_kv_heads > 0) {
        if (!ok_ptr(p->k, 16) || !ok_ptr(p->v, 16) || !ok_ptr(p->k_cache, 16) || !ok_ptr(p->v_cache, 16)) {
            return FNB_REJECTED;
        }
        if (F == kv_fmt::kv8 && (!ok_ptr(k_scale, 2) || !ok_ptr(v_scale, 2))) return FNB_REJECTED;
        if (F == kv_fmt::kv8 && hd < 64) return FNB_REJECTED;
    }
    if (!(p->eps >= 0.0f) || !(p->theta_scale > 0.0f)) return FNB_REJECTED;

    kernel_args a;
    a.q = p->q, a.k = p->k, a.v = p->v, a.pos = p->pos, a.slots = p->slots, a.planes = p->planes;
    a.q_norm_w = p->q_norm_w, a.k_norm_w = p->k_norm_w, a.q_out = p->q_out, a.k_f32 = p->k_f32;
    a.k_cache = static_cast<uint8_t *>(p->k_cache), a.v_cache = static_cast<uint8_t *>(p->v_cache);
    a.k_scale = k_scale, a.v_scale = v_scale, a.err = p->err;
    a.rows = p->rows, a.cache_slots = p->cache_slots;
    a.n_q = p->n_q_heads, a.n_kv = p->n_kv_heads, a.n_rot = p->n_rot;
    a.theta_scale = p->theta_scale, a.eps = p->eps;

    if (rope_kv_pipe_try_launch(a, hd, F, s)) return launch_status();

    const int heads = a.n_q + 2 * a.n_kv;
    int warps = (heads + 1) / 2;
    warps = warps < 1 ? 1 : warps > kMaxWarps ? kMaxWarps : warps;
    const int threads = warps * 32;
    const int grid = grid_for(p->rows, 2048 / threads > 0 ? 2048 / threads : 1);
    switch (hd) {
        case 256: rope_kv_kernel<256, F><<<grid, threads, 0, s>>>(a); break;
        case 128: rope_kv_kernel<128, F><<<grid, threads, 0, s>>>(a); break;
        default: rope_kv_kernel<64, F><<<grid, threads, 0, s>>>(a); break;
    }
    return launch_status();
}

}  // namespace
}  // namespace fnb

extern "C" int32_t fnb_rope_neox_q8_0_append(const fnb_rope_kv_args * args, void * stream) {
    return fnb::launch<fnb::kv_fmt::q8_0>(args, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t fnb_rope_neox_kv8_append(const fnb_rope_kv8_args * args, void * stream) {
    if (args == nullptr) return FNB_REJECTED;
    return fnb::launch<fnb::kv_fmt::kv8>(&args->base, args->k_scale, args->v_scale, static_cast<cudaStream_t>(stream));
}

extern "C" float fnb_rope_theta_scale(float freq_base, int32_t n_rot) {
    return powf(freq_base, -2.0f / float(n_rot));
}
