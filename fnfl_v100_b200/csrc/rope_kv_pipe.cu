// Norm + NeoX RoPE + KV append as a bulk-copy pipeline: the form used whenever a tile of tokens fits in shared
// memory and the rotary halves are whole 32-value blocks apart (the benchmark shapes are; rope_kv.cu holds the
// row-per-warp kernel for everything else).
//
// Why a pipeline: the step is a copy with a little arithmetic (38 KB of HBM traffic per token), so what decides
// its speed is how many bytes each SM keeps in flight and how few instructions a row costs.  With loads into
// registers the first is tied to occupancy; with cp.async.bulk it is a shared-memory budget:
//
//   producer warps (2)  per tile of `tt` tokens: three bulk copies (the tile's Q, K and V rows are each one
//                       contiguous run in HBM) into stage s, completion counted in bytes on full[s]; while they
//                       fly the producers compute the tile's (cos, sin) pairs - the F32 angle chain pos * ts^i
//                       and the exact sincos, a token per warp - and resolve the tokens' cache slots, then arrive
//                       on full[s] themselves.
//   consumer warps (20) two groups of ten; tiles alternate between the groups so two tiles are in work while up to
//                       two more are in flight.  A warp takes four head rows at a time, EIGHT LANES PER ROW: lane
//                       `sub` of a row holds values 4 sub .. 4 sub + 3 of each of the row's 32-value blocks (one
//                       conflict-free 128-bit shared load per block).  That layout makes the per-row work cheap:
//                       the sum of squares needs a 3-step butterfly instead of 5, sqrt and divide are paid once per
//                       four rows, a rotary pair (i, i + 32) is two registers of the same lane (no shuffle), a Q8_0
//                       block's amax is a 3-step butterfly, and every lane of the warp does useful work in every
//                       phase.  Q leaves as 128-bit streaming stores (each row's eight lanes write one full
//                       128-byte line per block), K and V as whole cells assembled in shared memory.
//
// All barrier waits are bounded.  One persistent CTA per SM.
#include <atomic>

#include "bulk_pipe.cuh"
#include "exact_math.cuh"
#include "rope_kv.cuh"

namespace fnb {
namespace {

#ifndef FNB_ROPE_GROUPS
#define FNB_ROPE_GROUPS 2
#endif
#ifndef FNB_ROPE_GROUP_WARPS
#define FNB_ROPE_GROUP_WARPS 10
#endif
#ifndef FNB_ROPE_PRODUCERS
#define FNB_ROPE_PRODUCERS 2
#endif
#ifndef FNB_ROPE_MAX_STAGES
#define FNB_ROPE_MAX_STAGES 4
#endif
constexpr int kGroups = FNB_ROPE_GROUPS;
constexpr int kGroupWarps = FNB_ROPE_GROUP_WARPS;
constexpr int kConsumerWarps = kGroups * kGroupWarps;
constexpr int kProducerWarps = FNB_ROPE_PRODUCERS;  // a token's angles are one warp's work of ~1000 cycles latency
constexpr int kThreads = (kConsumerWarps + kProducerWarps) * 32;
constexpr int kSlotBytes = 288;    // a 272-byte cell, padded to 16
constexpr int kMaxTile = 8;        // tokens per tile at most

struct pipe_shape {
    int tt;            // tokens per stage
    int stages;        // a multiple of kGroups
    int nbh;           // n_rot / 64: blocks between the halves of a rotary pair (0: no rotation)
    uint32_t rpt_inv;  // ceil(2^32 / rows per token), for r / rpt by multiply-high
};

__device__ __forceinline__ float4 mul4(float4 a, float s) {
    return make_float4(__fmul_rn(a.x, s), __fmul_rn(a.y, s), __fmul_rn(a.z, s), __fmul_rn(a.w, s));
}
__device__ __forceinline__ float4 mul4(float4 a, float4 b) {
    return make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z), __fmul_rn(a.w, b.w));
}
__device__ __forceinline__ double sq4(double acc, float4 v) {
    acc = __dadd_rn(acc, double(__fmul_rn(v.x, v.x)));
    acc = __dadd_rn(acc, double(__fmul_rn(v.y, v.y)));
    acc = __dadd_rn(acc, double(__fmul_rn(v.z, v.z)));
    return __dadd_rn(acc, double(__fmul_rn(v.w, v.w)));
}
__device__ __forceinline__ float amax4(float4 v) { return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))); }

// rotate block j against block j + NBH for j < NBH; cs: the token's (cos, sin) pairs; only where `on`
template <int NJ, int NBH>
__device__ __forceinline__ void rope_blocks(float4 (&x)[NJ], const float2 * cs, int sub, bool on) {
    if constexpr (2 * NBH <= NJ) {
#pragma unroll
        for (int j = 0; j < NBH; ++j) {
            const float4 * t = reinterpret_cast<const float4 *>(cs + 32 * j + 4 * sub);  // pairs 32 j + 4 sub .. + 3
            const float4 c01 = t[0], c23 = t[1];                                          // (c0, s0, c1, s1), (c2, s2, c3, s3)
            const float4 a = x[j], b = x[j + NBH];
            float4 lo, hi;
            lo.x = __fsub_rn(__fmul_rn(a.x, c01.x), __fmul_rn(b.x, c01.y));
            hi.x = __fadd_rn(__fmul_rn(a.x, c01.y), __fmul_rn(b.x, c01.x));
            lo.y = __fsub_rn(__fmul_rn(a.y, c01.z), __fmul_rn(b.y, c01.w));
            hi.y = __fadd_rn(__fmul_rn(a.y, c01.w), __fmul_rn(b.y, c01.z));
            lo.z = __fsub_rn(__fmul_rn(a.z, c23.x), __fmul_rn(b.z, c23.y));
            hi.z = __fadd_rn(__fmul_rn(a.z, c23.y), __fmul_rn(b.z, c23.x));
            lo.w = __fsub_rn(__fmul_rn(a.w, c23.z), __fmul_rn(b.w, c23.w));
            hi.w = __fadd_rn(__fmul_rn(a.w, c23.w), __fmul_rn(b.w, c23.z));
            if (on) {
                x[j] = lo;
                x[j + NBH] = hi;
            }
        }
    }
}

// the select chain v[sub] without dynamic register indexing
template <int NJ>
__device__ __forceinline__ float pick(const float (&v)[NJ], int sub) {
    float r = v[0];
#pragma unroll
    for (int j = 1; j < NJ; ++j) r = sub == j ? v[j] : r;
    return r;
}

template <int HD, kv_fmt F>
__global__ void __launch_bounds__(kThreads, 1) rope_kv_pipe_kernel(const rope_kernel_args a, const pipe_shape sh) {
    constexpr int NJ = HD / 32;  // 32-value blocks per row = 128-bit vectors per lane
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const int tt = sh.tt, stages = sh.stages;
    const int n_q = a.n_q, n_kv = a.n_kv, rpt = n_q + 2 * n_kv;
    const uint32_t q_tok = uint32_t(n_q) * HD * 4, kv_tok = uint32_t(n_kv) * HD * 4;
    const uint32_t stage_bytes = uint32_t(tt) * (q_tok + 2 * kv_tok);
    const int half = a.n_rot / 2;

    uint8_t * data = smem;
    float2 * cs_all = reinterpret_cast<float2 *>(data + size_t(stages) * stage_bytes);      // [stages][tt][HD/2]
    float * w_tab = reinterpret_cast<float *>(cs_all + size_t(stages) * tt * (HD / 2));     // [3][HD]: q, k, ones
    uint8_t * slots = reinterpret_cast<uint8_t *>(w_tab + 3 * HD);                          // [warps][4][kSlotBytes]
    uint64_t * full = reinterpret_cast<uint64_t *>(slots + kConsumerWarps * 4 * kSlotBytes);
    uint64_t * empty = full + stages;
    int32_t * cell_of = reinterpret_cast<int32_t *>(empty + stages);                        // [stages][tt]

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full[s], kProducerWarps);
            mbar_init(&empty[s], kGroupWarps);
        }
        mbar_init_fence();
    }
    __syncthreads();  // nothing slow before this point: the producers start streaming at once
    pdl_wait();       // the predecessor's writes are visible from here on; no global memory was touched before

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t n_tiles = (a.rows + tt - 1) / tt;

    if (wid >= kConsumerWarps) {
        // ---------------- producers ----------------
        // Warp 0 of the pair issues the tile's copies; both compute the angles and resolve the cache slot of their
        // share of the tile's tokens (token tk belongs to warp tk % kProducerWarps), then arrive.
        const int pw = wid - kConsumerWarps;
        const uint64_t policy = l2_evict_first_policy();
        int it = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
            const int s = it % stages;
            const uint32_t ph = uint32_t(it / stages) & 1u;
            const int64_t t0 = tile * tt;
            const int live = int(a.rows - t0 < tt ? a.rows - t0 : tt);
            // positions and slots do not depend on the stage: fetch them before waiting for it
            int32_t p_of[kMaxTile / kProducerWarps];
            int64_t c_of[kMaxTile / kProducerWarps];
#pragma unroll
            for (int j = 0; j < kMaxTile / kProducerWarps; ++j) {
                const int tk = pw + j * kProducerWarps;
                p_of[j] = tk < live ? __ldg(a.pos + t0 + tk) : 0;
                c_of[j] = tk < live && a.slots != nullptr ? int64_t(__ldg(a.slots + t0 + tk)) : int64_t(p_of[j]);
            }
            if (it >= stages && !mbar_wait(&empty[s], ph ^ 1u, a.err)) {
                ok = false;
                break;
            }
            uint8_t * st = data + size_t(s) * stage_bytes;
            if (pw == 0 && lane == 0) {
                mbar_expect_tx(&full[s], uint32_t(live) * (q_tok + 2 * kv_tok));
                if (n_q > 0) bulk_g2s(st, a.q + t0 * n_q * HD, uint32_t(live) * q_tok, &full[s], policy);
                if (n_kv > 0) {
                    bulk_g2s(st + size_t(tt) * q_tok, a.k + t0 * n_kv * HD, uint32_t(live) * kv_tok, &full[s], policy);
                    bulk_g2s(st + size_t(tt) * (q_tok + kv_tok), a.v + t0 * n_kv * HD, uint32_t(live) * kv_tok, &full[s],
                             policy);
                }
            }
#pragma unroll
            for (int j = 0; j < kMaxTile / kProducerWarps; ++j) {
                const int tk = pw + j * kProducerWarps;
                if (tk >= live) break;
                float2 * cs = cs_all + (size_t(s) * tt + tk) * (HD / 2);
                // lane i walks the chain pos * ts^i: i multiplies to reach its first pair, 32 more for each further one
                // (with position planes, n_rot is 64: lane i is pair i and reads its own plane's position)
                float theta = float(a.planes != nullptr ? __ldg(a.planes + 4 * (t0 + tk) + rope_plane_of_pair(lane)) : p_of[j]);
#pragma unroll
                for (int c = 0; c < 31; ++c) theta = c < lane ? __fmul_rn(theta, a.theta_scale) : theta;
                for (int i = lane; i < half; i += 32) {
                    float sn, cn;
                    exact_sincosf(theta, &sn, &cn);
                    cs[i] = make_float2(cn, sn);
                    for (int c = 0; c < 32; ++c) theta = __fmul_rn(theta, a.theta_scale);
                }
                if (lane == 0) {
                    const bool good = c_of[j] >= 0 && c_of[j] < a.cache_slots;
                    if (!good && a.err != nullptr) atomicOr(a.err, FNB_ERR_SLOT);
                    cell_of[s * tt + tk] = good ? int32_t(c_of[j]) : -1;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
        // The copying producer leaves last: every copy it issued into this CTA's shared memory has landed (bounded)
        // before the CTA can exit and the memory be handed to another CTA.  After a normal run these waits pass at
        // once; after a wait that gave up, here or in a consumer, they are what keeps the exit safe.
        (void) ok;
        if (pw == 0 && lane == 0) {
            for (int j = 1; j <= stages && j <= it; ++j) {
                const int its = it - j;
                mbar_wait_landed(&full[its % stages], uint32_t(its / stages) & 1u);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // the norm weights reach shared memory while the first tiles are in flight
    for (int i = threadIdx.x; i < HD; i += kConsumerWarps * 32) {
        w_tab[i] = a.q_norm_w != nullptr ? __ldg(a.q_norm_w + i) : 1.0f;
        w_tab[HD + i] = a.k_norm_w != nullptr ? __ldg(a.k_norm_w + i) : 1.0f;
        w_tab[2 * HD + i] = 1.0f;
    }
    named_barrier<1>(kConsumerWarps * 32);
    const int grp = wid / kGroupWarps, gw = wid - grp * kGroupWarps;
    const int sub = lane & 7, rq = lane >> 3;
    uint8_t * my_slot = slots + (wid * 4 + rq) * kSlotBytes;  // this row's cell under assembly
    const bool any_norm = a.q_norm_w != nullptr || a.k_norm_w != nullptr;
    constexpr int cell_bytes = F == kv_fmt::q8_0 ? NJ * 34 : HD;

    int it = 0;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
        if (it % kGroups != grp) continue;
        const int s = it % stages;
        const uint32_t ph = uint32_t(it / stages) & 1u;
        if (!mbar_wait(&full[s], ph, a.err)) return;
        const int64_t t0 = tile * tt;
        const int live = int(a.rows - t0 < tt ? a.rows - t0 : tt);
        const uint8_t * st = data + size_t(s) * stage_bytes;
        const int n_rows = live * rpt;
        for (int qd = gw; 4 * qd < n_rows; qd += kGroupWarps) {
            // this lane's row of the quad: token tk, head slot h (q heads, then k heads, then v heads)
            const int r = 4 * qd + rq;
            const bool in_tile = r < n_rows;
            const int tk = in_tile ? int(__umulhi(uint32_t(r), sh.rpt_inv)) : 0;
            const int h = in_tile ? r - tk * rpt : 0;
            const int kind = !in_tile ? 3 : h < n_q ? 0 : h < n_q + n_kv ? 1 : 2;  // q, k, v, none
            const int hh = kind == 0 ? h : kind == 1 ? h - n_q : h - n_q - n_kv;
            const uint32_t off = kind == 0   ? uint32_t(tk * n_q + hh) * HD * 4
                                 : kind == 1 ? uint32_t(tt) * q_tok + uint32_t(tk * n_kv + hh) * HD * 4
                                             : uint32_t(tt) * (q_tok + kv_tok) + uint32_t(tk * n_kv + hh) * HD * 4;
            const int32_t cell = in_tile ? cell_of[s * tt + tk] : -1;
            const bool live_row = cell >= 0;  // a token with a bad slot writes nothing
            const float4 * src = reinterpret_cast<const float4 *>(st + (kind == 3 ? 0u : off));
            float4 x[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) x[j] = src[8 * j + sub];

            if (any_norm) {
                const bool do_norm = (kind == 0 && a.q_norm_w != nullptr) || (kind == 1 && a.k_norm_w != nullptr);
                double acc = 0.0;
#pragma unroll
                for (int j = 0; j < NJ; ++j) acc = sq4(acc, x[j]);
#pragma unroll
                for (int m = 1; m < 8; m <<= 1) acc = __dadd_rn(acc, shfl_xor_f64(acc, m));
                const float mean = __double2float_rn(__dmul_rn(acc, 1.0 / double(HD)));  // HD is a power of two: exact
                const float scale = do_norm ? __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps))) : 1.0f;
                const float4 * w4 = reinterpret_cast<const float4 *>(w_tab + (do_norm ? kind : 2) * HD);
#pragma unroll
                for (int j = 0; j < NJ; ++j) x[j] = mul4(mul4(x[j], scale), w4[8 * j + sub]);  // (x scale) w; 1 and 1 when off
            }
            if (sh.nbh > 0) {
                const float2 * cs = cs_all + (size_t(s) * tt + tk) * (HD / 2);
                const bool on = kind <= 1;
                switch (sh.nbh) {
                    case 1: rope_blocks<NJ, 1>(x, cs, sub, on); break;
                    case 2: rope_blocks<NJ, 2>(x, cs, sub, on); break;
                    default: rope_blocks<NJ, 4>(x, cs, sub, on); break;
                }
            }
            const int64_t t = t0 + tk;
            if (kind == 0 && live_row) {
                float4 * dst = reinterpret_cast<float4 *>(a.q_out + (t * n_q + hh) * HD);
#pragma unroll
                for (int j = 0; j < NJ; ++j) st_stream(dst + 8 * j + sub, x[j]);
            }
            const bool is_kv = (kind == 1 || kind == 2) && live_row;
            if (!__any_sync(kFull, is_kv)) continue;  // four Q rows: done

            if (kind == 1 && live_row && a.k_f32 != nullptr) {
                float4 * dst = reinterpret_cast<float4 *>(a.k_f32 + (t * n_kv + hh) * HD);
#pragma unroll
                for (int j = 0; j < NJ; ++j) st_stream(dst + 8 * j + sub, x[j]);
            }
            uint8_t * cache = kind == 1 ? a.k_cache : a.v_cache;
            const int64_t c = int64_t(cell) * n_kv + hh;
            float am[NJ];
#pragma unroll
            for (int j = 0; j < NJ; ++j) am[j] = group_max<8>(amax4(x[j]));
            if (F == kv_fmt::q8_0) {
                // lane `sub` owns block `sub`: one d and one 1/d per block, 1/d handed to the block's users by shuffle
                const ggml_q8_rule own(pick<NJ>(am, sub));
                uint16_t * s16 = reinterpret_cast<uint16_t *>(my_slot);
                if (sub < NJ) s16[17 * sub] = f32_to_f16_bits(own.d);
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    ggml_q8_rule rule = own;
                    rule.id = __shfl_sync(kFull, own.id, (lane & ~7) | j);
                    const uint32_t wrd = rule.code4(x[j]);
                    s16[17 * j + 1 + 2 * sub] = uint16_t(wrd);
                    s16[17 * j + 2 + 2 * sub] = uint16_t(wrd >> 16);
                }
                __syncwarp();
                // 4 rows x 17 units (272 = 17 x 16, 136 = 17 x 8, 68 = 17 x 4 bytes) leave as the widest aligned stores
                uint8_t * dst_row = cache + c * cell_bytes;
#pragma unroll
                for (int pass = 0; pass < 3; ++pass) {  // 68 units over 32 lanes; every lane joins every shuffle
                    const int u = lane + 32 * pass;
                    const int row = u < 4 * 17 ? u / 17 : 3, unit = u - row * 17;
                    const uint64_t d64 = __shfl_sync(kFull, is_kv ? uint64_t(reinterpret_cast<uintptr_t>(dst_row)) : 0ull, 8 * row);
                    uint8_t * d = reinterpret_cast<uint8_t *>(uintptr_t(d64));
                    const uint8_t * sl = slots + (wid * 4 + row) * kSlotBytes;
                    if (u < 4 * 17 && d != nullptr) {
                        if constexpr (HD == 256) {
                            st_stream(reinterpret_cast<uint4 *>(d) + unit, reinterpret_cast<const uint4 *>(sl)[unit]);
                        } else if constexpr (HD == 128) {
                            st_stream(reinterpret_cast<uint2 *>(d) + unit, reinterpret_cast<const uint2 *>(sl)[unit]);
                        } else {
                            st_stream(reinterpret_cast<uint32_t *>(d) + unit, reinterpret_cast<const uint32_t *>(sl)[unit]);
                        }
                    }
                }
                __syncwarp();
            } else {
                // the reference engine's format: FP16 scale per 64 values (two blocks), codes nearest-even of x / s
                uint8_t * codes = cache + c * HD;
                uint16_t * scl = (kind == 1 ? a.k_scale : a.v_scale) + c * (HD / 64);
#pragma unroll
                for (int g = 0; g < NJ / 2; ++g) {
                    const kv8_rule rule(fmaxf(am[2 * g], am[2 * g + 1]));
#pragma unroll
                    for (int j = 2 * g; j < 2 * g + 2; ++j) {
                        const uint32_t wrd = rule.code4(x[j]);
                        if (is_kv) st_stream(reinterpret_cast<uint32_t *>(codes) + 8 * j + sub, wrd);
                    }
                    if (is_kv && sub == 0) scl[g] = rule.sb;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
}

#ifndef FNB_ROPE_SMEM_KB
#define FNB_ROPE_SMEM_KB 212
#endif
constexpr size_t kSmemBudget = size_t(FNB_ROPE_SMEM_KB) * 1024;

// raises the kernel's dynamic shared-memory limit once per device
template <int HD, kv_fmt F>
bool ensure_configured() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(rope_kv_pipe_kernel<HD, F>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(kSmemBudget)) != cudaSuccess) {
            (void) cudaGetLastError();
            return false;
        }
        configured[dev].store(true, std::memory_order_release);
    }
    return true;
}

template <int HD, kv_fmt F>
bool launch_one(const rope_kernel_args & a, cudaStream_t s) {
    // the halves of a rotary pair must be whole blocks apart: n_rot a multiple of 64, at most head_dim
    if (a.n_rot % 64 != 0 || a.n_rot > HD) return false;
    const int nbh = a.n_rot / 64;
    if (nbh != 0 && nbh != 1 && nbh != 2 && nbh != 4) return false;
    if (F == kv_fmt::kv8 && HD < 64) return false;
    const int rpt = a.n_q + 2 * a.n_kv;
    if (rpt < 2) return false;  // r / rpt by multiply-high needs rpt >= 2
    const size_t tok_bytes = size_t(rpt) * HD * 4;
    int tt = (kGroupWarps * 4) / rpt;  // one quad of rows per consumer warp and tile
    tt = tt < 1 ? 1 : tt > kMaxTile ? kMaxTile : tt;
    const size_t fixed = size_t(3) * HD * 4 + size_t(kConsumerWarps) * 4 * kSlotBytes + 256;
    auto need = [&](int t, int st) {
        return size_t(st) * (size_t(t) * tok_bytes + size_t(t) * (HD / 2) * 8 + 16 + size_t(t) * 4) + fixed;
    };
    // the ring: a multiple of the group count (a stage always goes to the same group), as deep as the budget allows
    auto fit = [&](int t) {
        int st = (FNB_ROPE_MAX_STAGES / kGroups) * kGroups;
        while (st >= kGroups && need(t, st) > kSmemBudget) st -= kGroups;
        return st;
    };
    int stages = fit(tt);
    if (stages < kGroups && tt > 1) {
        tt = 1;
        stages = fit(tt);
    }
    if (stages < kGroups) return false;
    const size_t smem = need(tt, stages);

    if (!ensure_configured<HD, F>()) return false;
    const int64_t n_tiles = (a.rows + tt - 1) / tt;
    const int grid = int(n_tiles < kSmCount ? n_tiles : kSmCount);
    const pipe_shape sh{tt, stages, nbh, uint32_t((0x100000000ull + uint64_t(rpt) - 1) / uint64_t(rpt))};
    launch_pdl(rope_kv_pipe_kernel<HD, F>, grid, kThreads, smem, s, a, sh);
    return true;
}

}  // namespace

bool rope_kv_pipe_try_launch(const rope_kernel_args & a, int head_dim, kv_fmt fmt, cudaStream_t s) {
    const bool q8 = fmt == kv_fmt::q8_0;
    switch (head_dim) {
        case 256: return q8 ? launch_one<256, kv_fmt::q8_0>(a, s) : launch_one<256, kv_fmt::kv8>(a, s);
        case 128: return q8 ? launch_one<128, kv_fmt::q8_0>(a, s) : launch_one<128, kv_fmt::kv8>(a, s);
        case 64: return q8 ? launch_one<64, kv_fmt::q8_0>(a, s) : launch_one<64, kv_fmt::kv8>(a, s);
        default: return false;
    }
}

bool rope_prepare_device() {
    return ensure_configured<256, kv_fmt::q8_0>() && ensure_configured<256, kv_fmt::kv8>() &&
           ensure_configured<128, kv_fmt::q8_0>() && ensure_configured<128, kv_fmt::kv8>() &&
           ensure_configured<64, kv_fmt::q8_0>() && ensure_configured<64, kv_fmt::kv8>();
}

}  // namespace fnb
