"""Drop-in for the reference's mx/custom_extensions.py (:11-19), which JIT-builds its C++/CUDA sources and
exposes them as `funcs`: here `funcs` carries the same seven names on top of libmxq's C ABI
(quantize_mx_by_tile_func_cuda, quantize_mx_func_cuda, quantize_elemwise_func_cuda, their *_cpp host twins,
reduce_sum_inner_dim, reduce_max_inner_dim)."""
from ._backend import funcs  # noqa: F401
