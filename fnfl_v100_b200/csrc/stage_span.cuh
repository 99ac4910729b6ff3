// Copying a run of global bytes that starts on a 4-byte boundary into a warp's shared-memory buffer with cp.async:
// 16-byte copies between the 16-byte boundaries of the source, whose offset within 16 bytes the shared-memory copy
// keeps (so both addresses of every 16-byte copy are aligned), and up to three 4-byte copies at either end.  The
// caller commits the group and waits for it (cp.async.wait_group, then __syncwarp before other lanes read).
#pragma once
#include <cstdint>

namespace fnb {

__device__ __forceinline__ void cp_async_16(uint32_t dst, const uint8_t * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const uint8_t * src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// `bytes` (a multiple of 4, at least 16) from src (4-byte aligned) to slot_sm + (src & 15); slot_sm is 16-byte aligned
// and has room for bytes + 12.  All 32 lanes of the warp call it.
__device__ __forceinline__ void stage_span(uint32_t slot_sm, const uint8_t * src, int bytes, int lane) {
    const int phase = int(reinterpret_cast<uintptr_t>(src) & 15);
    const uint32_t dst = slot_sm + phase;
    const int head = (16 - phase) & 15;
    const int body = (bytes - head) >> 4, tail = (bytes - head) & 15;
    for (int c = lane; c < body; c += 32) cp_async_16(dst + head + 16 * c, src + head + 16 * c);
    if (lane < (head >> 2)) {
        cp_async_4(dst + 4 * lane, src + 4 * lane);
    } else if (lane >= 8 && lane - 8 < (tail >> 2)) {
        const int o = head + 16 * body + 4 * (lane - 8);
        cp_async_4(dst + o, src + o);
    }
}

}  // namespace fnb
