// Library identity and status names.
#include "common.cuh"

extern "C" int32_t fnb_version(void) { return 200; }  // 0.2.0

extern "C" const char * fnb_status_name(int32_t status) {
    switch (status) {
        case FNB_OK: return "ok";
        case FNB_REJECTED: return "rejected: argument outside the contract, nothing enqueued";
        case FNB_LAUNCH_FAILED: return "launch failed: see cudaPeekAtLastError";
        default: return "unknown status";
    }
}

// One-time, per-device set-up of every kernel that needs more than the default shared memory, for the CURRENT device.
// After it no launcher of this library calls anything but the launch itself, so every entry point is capturable from
// its first call on.
extern "C" int32_t fnb_prepare_device(void) {
    const bool ok = fnb::glu_prepare_device() && fnb::rms_norm_quant_prepare_device() && fnb::rope_prepare_device() &&
                    fnb::expert_down_prepare_device() && fnb::expert_gate_up_prepare_device() &&
                    fnb::expert_down_iq4nl_prepare_device() && fnb::attend_prepare_device();
    return ok ? FNB_OK : FNB_LAUNCH_FAILED;
}
