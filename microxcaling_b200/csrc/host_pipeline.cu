// Host-buffer entry points: quantize a tensor that lives in (pinned) host
// memory and put the result back in host memory.  The tensor is cut into
// chunks of whole blocks; chunk i's host->device copy, kernel and device->host
// copy run on one of three internal streams, so the copy engines in both
// directions and the SMs work on different chunks at the same time (chunks are
// short at both ends of the tensor, where a copy has nothing to overlap).  PCIe is
// the bound here (two copies of 2-4 bytes per element against a kernel that
// needs a few percent of that time), so the pipeline's job is to keep both
// directions of the link busy.
#include <algorithm>
#include <mutex>
#include "mxq_common.cuh"

namespace mxq {

#ifndef MXQ_PIPE_SLOTS
#define MXQ_PIPE_SLOTS 3
#endif
#ifndef MXQ_PIPE_CHUNK_MB
#define MXQ_PIPE_CHUNK_MB 16
#endif
constexpr int kPipeSlots = MXQ_PIPE_SLOTS;
constexpr int64_t kChunkBytes = int64_t(MXQ_PIPE_CHUNK_MB) << 20;     // target of input bytes per chunk

static constexpr int64_t chunk_bytes() { return kChunkBytes; }

struct HostPipe {
    cudaStream_t s[kPipeSlots];
    cudaEvent_t slot_done[kPipeSlots];
    cudaEvent_t begin;
    bool ready = false;
};

static HostPipe* pipe_for_device() {
    static HostPipe pipes[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    HostPipe& p = pipes[dev];
    if (!p.ready) {
        for (int i = 0; i < kPipeSlots; ++i) {
            if (cudaStreamCreateWithFlags(&p.s[i], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
            if (cudaEventCreateWithFlags(&p.slot_done[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
        }
        if (cudaEventCreateWithFlags(&p.begin, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        p.ready = true;
    }
    return &p;
}

// units: indivisible groups of `unit_elems` consecutive elements; launch(d_in, d_out, first_unit, n_units, stream)
template <typename Launch>
static int run_chunks(const void* h_in, void* h_out, int in_es, int out_es, int64_t units, int64_t unit_elems,
                      int64_t total_elems, void* ws, int64_t ws_bytes, cudaStream_t user, Launch launch) {
    HostPipe* p = pipe_for_device();
    if (!p) return MXQ_ERR_CUDA;
    const int64_t slot_bytes = (ws_bytes / kPipeSlots) & ~int64_t(255);
    const int64_t per_elem = in_es + out_es;
    int64_t upc = std::max<int64_t>(1, chunk_bytes() / std::max<int64_t>(1, unit_elems * in_es));
    // a slot holds the input chunk followed (256-aligned) by the output chunk
    while (upc > 1 && upc * unit_elems * per_elem + 512 > slot_bytes) upc /= 2;
    if (upc * unit_elems * per_elem + 512 > slot_bytes) return MXQ_ERR_TOO_LARGE;
    if (cudaEventRecord(p->begin, user) != cudaSuccess) return MXQ_ERR_CUDA;
    for (int i = 0; i < kPipeSlots; ++i)
        if (cudaStreamWaitEvent(p->s[i], p->begin, 0) != cudaSuccess) return MXQ_ERR_CUDA;
    // Chunk sizes ramp up from upc / 8 and down again at the end: the first chunk's host->device copy and the
    // last chunk's device->host copy are the only transfers nothing overlaps, so they are kept short.
    const int64_t min_units = std::max<int64_t>(1, upc / 8);
    int64_t done_units = 0;
    for (int64_t c = 0; done_units < units; ++c) {
        const int slot = (int)(c % kPipeSlots);
        cudaStream_t st = p->s[slot];
        const int64_t left = units - done_units;
        const int64_t up = c < 3 ? std::min(upc, min_units << c) : upc;
        const int64_t down = std::max(min_units, (left + 1) / 2);
        const int64_t n = std::min(std::min(up, down), left);
        const int64_t first_elem = done_units * unit_elems;
        const int64_t elems = std::min(n * unit_elems, total_elems - first_elem);
        uint8_t* d_in = reinterpret_cast<uint8_t*>(ws) + slot * slot_bytes;
        uint8_t* d_out = d_in + ((upc * unit_elems * in_es + 255) & ~int64_t(255));
        if (cudaMemcpyAsync(d_in, reinterpret_cast<const uint8_t*>(h_in) + first_elem * in_es, (size_t)(elems * in_es),
                            cudaMemcpyHostToDevice, st) != cudaSuccess) return MXQ_ERR_CUDA;
        const int rc = launch(d_in, d_out, done_units, n, elems, st);
        if (rc) return rc;
        if (cudaMemcpyAsync(reinterpret_cast<uint8_t*>(h_out) + first_elem * out_es, d_out, (size_t)(elems * out_es),
                            cudaMemcpyDeviceToHost, st) != cudaSuccess) return MXQ_ERR_CUDA;
        done_units += n;
    }
    for (int i = 0; i < kPipeSlots; ++i) {
        if (cudaEventRecord(p->slot_done[i], p->s[i]) != cudaSuccess) return MXQ_ERR_CUDA;
        if (cudaStreamWaitEvent(user, p->slot_done[i], 0) != cudaSuccess) return MXQ_ERR_CUDA;
    }
    return MXQ_OK;
}

}  // namespace mxq

extern "C" int mxq_quantize_mx_host(const void* h_in, void* h_out, int dtype, int64_t pre, int64_t axis_len,
                                    int64_t post, int block, int scale_bits, int elem_ebits, int elem_mbits,
                                    float elem_max_norm, int flush_fp32_subnorms, int rmode, void* workspace,
                                    int64_t workspace_bytes, void* stream) {
    using namespace mxq;
    if (pre < 0 || axis_len < 0 || post < 0) return MXQ_ERR_BAD_ARG;
    if (pre == 0 || axis_len == 0 || post == 0) return MXQ_OK;
    if (!h_in || !h_out || !workspace) return MXQ_ERR_BAD_ARG;
    if (dtype < MXQ_F32 || dtype > MXQ_BF16 || rmode < 0 || rmode > MXQ_ROUND_EVEN) return MXQ_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
    if (block <= 0 || block > axis_len) block = (int)std::min<int64_t>(axis_len, 0x7fffffff);
    const int es = dtype_size(dtype);
    const int64_t total = pre * axis_len * post;
    // cut along `pre` when there is one, else along the blocked axis in whole blocks
    const bool by_pre = pre > 1;
    const int64_t unit_elems = by_pre ? axis_len * post : (int64_t)block * post;
    const int64_t units = by_pre ? pre : (axis_len + block - 1) / block;
    auto launch = [=](void* d_in, void* d_out, int64_t first, int64_t n, int64_t elems, cudaStream_t st) -> int {
        (void)first;
        const int64_t c_pre = by_pre ? n : 1;
        const int64_t c_axis = by_pre ? axis_len : elems / post;
        return mxq_quantize_mx(d_in, d_out, nullptr, nullptr, dtype, c_pre, c_axis, post, block, scale_bits,
                               elem_ebits, elem_mbits, elem_max_norm, flush_fp32_subnorms, rmode, nullptr, 0, 0, st);
    };
    return run_chunks(h_in, h_out, es, es, units, unit_elems, total, workspace, workspace_bytes,
                      (cudaStream_t)stream, launch);
}

extern "C" int mxq_quantize_elemwise_host(const void* h_in, void* h_out, int in_dtype, int out_dtype, int64_t n,
                                          int bits, int exp_bits, float max_norm, int rmode, int saturate_normals,
                                          int allow_denorm, void* workspace, int64_t workspace_bytes, void* stream) {
    using namespace mxq;
    if (n < 0) return MXQ_ERR_BAD_ARG;
    if (n == 0) return MXQ_OK;
    if (!h_in || !h_out || !workspace) return MXQ_ERR_BAD_ARG;
    if (in_dtype < MXQ_F32 || in_dtype > MXQ_BF16 || out_dtype < MXQ_F32 || out_dtype > MXQ_BF16) return MXQ_ERR_BAD_ARG;
    if (rmode < 0 || rmode > MXQ_ROUND_EVEN) return MXQ_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MXQ_ERR_ALIGN;
    const int64_t unit = 4096;                              // elements; keeps every chunk 16-byte aligned
    auto launch = [=](void* d_in, void* d_out, int64_t first, int64_t nu, int64_t elems, cudaStream_t st) -> int {
        (void)first; (void)nu;
        return mxq_quantize_elemwise(d_in, d_out, in_dtype, out_dtype, elems, bits, exp_bits, max_norm, rmode,
                                     saturate_normals, allow_denorm, nullptr, st);
    };
    return run_chunks(h_in, h_out, dtype_size(in_dtype), dtype_size(out_dtype), (n + unit - 1) / unit, unit, n,
                      workspace, workspace_bytes, (cudaStream_t)stream, launch);
}

extern "C" int64_t mxq_host_workspace_bytes(void) {
    // three slots of (input chunk + output chunk) at the target chunk size for 4-byte elements
    return mxq::kPipeSlots * (2 * (int64_t(64) << 20) + 1024);
}
