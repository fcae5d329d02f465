"""B200-native (sm_100a) implementation of microxcaling's quantization path.

Public names follow the reference's mx/__init__.py:6-38 for the operators this
package covers; `mx_ops.quantize_mx_op`, `elemwise_ops.quantize_elemwise_op` and
`mx_mapping.inject_pyt_ops` are imported from their submodules, as there."""
from .specs import MxSpecs, add_mx_args, finalize_mx_specs, get_mx_specs, get_backwards_mx_specs  # noqa: F401
from .quantize import quantize_bfloat  # noqa: F401
from .linear import Linear, linear  # noqa: F401
from .matmul import matmul  # noqa: F401
from .bmm import bmm  # noqa: F401
from .activations import SiLU, silu, sigmoid, tanh  # noqa: F401
from .layernorm import RMSNorm  # noqa: F401
from .simd_ops import simd_add, simd_sub, simd_mul, simd_div  # noqa: F401
from .softmax import Softmax, softmax  # noqa: F401
from .convolution import Conv1d, Conv2d, Conv3d, ConvTranspose2d, conv1d, conv2d, conv3d, conv_transpose2d  # noqa: F401
from .rnn import LSTM  # noqa: F401
