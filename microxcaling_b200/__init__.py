"""B200-native (sm_100a) implementation of microxcaling's quantization path.

Public names follow the reference's mx/__init__.py:6-38 for the operators this
package covers; `mx_ops.quantize_mx_op`, `elemwise_ops.quantize_elemwise_op` and
`mx_mapping.inject_pyt_ops` are imported from their submodules, as there."""
from .specs import MxSpecs, add_mx_args, finalize_mx_specs, get_mx_specs, get_backwards_mx_specs  # noqa: F401
from .quantize import quantize_bfloat  # noqa: F401
from .linear import Linear, linear  # noqa: F401
from .matmul import matmul  # noqa: F401
from .bmm import bmm  # noqa: F401
from .activations import sigmoid, tanh, relu, relu6, leaky_relu, silu, gelu  # noqa: F401
from .activations import Sigmoid, Tanh, ReLU, ReLU6, LeakyReLU, SiLU, GELU  # noqa: F401
from .adaptive_avg_pooling import adaptive_avg_pool2d, AdaptiveAvgPool2d  # noqa: F401
from .batchnorm import BatchNorm1d, BatchNorm2d, BatchNorm3d  # noqa: F401
from .layernorm import LayerNorm, RMSNorm, layer_norm  # noqa: F401
from .groupnorm import GroupNorm  # noqa: F401
from .simd_ops import simd_add, simd_sub, simd_mul, simd_div, simd_split  # noqa: F401
from .simd_ops import simd_sqrt, simd_square, simd_exp, simd_log  # noqa: F401
from .simd_ops import simd_reduce_sum, simd_reduce_mean, simd_norm  # noqa: F401
from .softmax import Softmax, softmax  # noqa: F401
from .convolution import Conv1d, Conv2d, Conv3d, ConvTranspose2d, conv1d, conv2d, conv3d, conv_transpose2d  # noqa: F401
from .rnn import LSTM  # noqa: F401
