// Status strings and version of the C ABI.
#include "mxq_common.cuh"
#include <string.h>

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
extern "C" int mxq_version(void) { return 2; }

namespace mxq {
std::atomic<int64_t> g_launch_count[2];
std::atomic<int> g_gemm_sm_budget{0};
}
extern "C" int mxq_gemm_sm_budget(int sms) {
    if (sms < 0) return mxq::g_gemm_sm_budget.load(std::memory_order_relaxed);
    return mxq::g_gemm_sm_budget.exchange(sms, std::memory_order_relaxed);
}
extern "C" int64_t mxq_launch_count(int what) {
    return (what == 0 || what == 1) ? mxq::g_launch_count[what].load(std::memory_order_relaxed) : -1;
}

// ---------------------------------------------------------------------------
// Receive buffers that other processes of the node can map (CUDA IPC).  The
// importing process opens the handle while ITS OWN device is current, which is
// what makes the mapping usable by kernels of that device (peer access between
// the two GPUs is enabled by the open call); a mapping opened under the owner's
// device index is only good for kernels launched on that device.
// ---------------------------------------------------------------------------
extern "C" int mxq_peer_alloc(int64_t bytes, void** ptr, void* handle64) {
    if (bytes <= 0 || !ptr || !handle64) return MXQ_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return MXQ_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return MXQ_ERR_CUDA; }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return MXQ_OK;
}
extern "C" int mxq_peer_free(void* ptr) {
    if (!ptr) return MXQ_OK;
    return cudaFree(ptr) == cudaSuccess ? MXQ_OK : MXQ_ERR_CUDA;
}
extern "C" int mxq_peer_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return MXQ_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return MXQ_ERR_CUDA; }
    *ptr = p;
    return MXQ_OK;
}
extern "C" int mxq_peer_close(void* ptr) {
    if (!ptr) return MXQ_OK;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? MXQ_OK : MXQ_ERR_CUDA;
}
