// Instantiates the MX quantization kernels for one storage type (kept in its
// own translation unit so the three types compile in parallel).
#include "quantize_mx_impl.cuh"
namespace mxq { template int dispatch_dt<DT_F32>(const MxArgs&, cudaStream_t); }
