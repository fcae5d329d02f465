// Status strings and version of the C ABI.
#include "mxq_common.cuh"

extern "C" const char* mxq_status_string(int status) {
    switch (status) {
        case MXQ_OK: return "ok";
        case MXQ_ERR_BAD_ARG: return "bad argument";
        case MXQ_ERR_UNSUPPORTED: return "unsupported request";
        case MXQ_ERR_CUDA: return "CUDA call failed";
        case MXQ_ERR_ALIGN: return "misaligned pointer or size";
        case MXQ_ERR_TOO_LARGE: return "size beyond the supported maximum";
        case MXQ_ERR_DEVICE: return "device-side time-out or fault word";
        default: return "unknown status";
    }
}
extern "C" int mxq_version(void) { return 1; }
