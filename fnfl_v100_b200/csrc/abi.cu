// Library identity and status names.
#include "common.cuh"

extern "C" int32_t fnb_version(void) { return 100; }  // 0.1.0

extern "C" const char * fnb_status_name(int32_t status) {
    switch (status) {
        case FNB_OK: return "ok";
        case FNB_REJECTED: return "rejected: argument outside the contract, nothing enqueued";
        case FNB_LAUNCH_FAILED: return "launch failed: see cudaPeekAtLastError";
        default: return "unknown status";
    }
}
