// Declarations shared by the two implementations of the norm + RoPE + KV-append step: the bulk-copy pipeline
// (rope_kv_pipe.cu, used whenever a token tile fits in shared memory) and the row-per-warp kernel
// (rope_kv.cu, any shape the contract allows).
#pragma once

#include "common.cuh"

namespace fnb {

enum class kv_fmt { q8_0, kv8 };

struct rope_kernel_args {
    const float *q, *k, *v;
    const int32_t *pos, *slots;
    const int32_t * planes;  // [rows][4] or null: the reference's rotary position planes of image rows
    const float *q_norm_w, *k_norm_w;
    float *q_out, *k_f32;
    uint8_t *k_cache, *v_cache;
    uint16_t *k_scale, *v_scale;
    uint32_t * err;
    int64_t rows, cache_slots;
    int32_t n_q, n_kv, n_rot;
    float theta_scale, eps;
};

// the position plane rotary pair i reads (sections 11, 11, 10, 0 of 32 pairs, interleaved), as the reference's
// imrope_plane (fn/kernels/qsa/imrope.cuh:15-24)
__host__ __device__ __forceinline__ int rope_plane_of_pair(int i) {
    return i % 3 == 1 && i < 33 ? 1 : i % 3 == 2 && i < 30 ? 2 : i % 3 == 0 && i < 33 ? 0 : 3;
}

// Enqueues the pipelined kernel when the shape suits it and returns true; returns false (nothing enqueued) when
// the caller should use the row-per-warp kernel instead.
bool rope_kv_pipe_try_launch(const rope_kernel_args & a, int head_dim, kv_fmt fmt, cudaStream_t s);

}  // namespace fnb
