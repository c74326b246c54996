from .activation import QUnaryFunctionLUT
from .attn.mha import QMultiHeadAttention
from .conv import QConv2D
from .core import QDense, QEinsumDense, QLayerBase, QLayerBaseMultiInputs, QLayerBaseSingleInput
from .softmax import QSoftmax

__all__ = ['QDense', 'QEinsumDense', 'QConv2D', 'QSoftmax', 'QUnaryFunctionLUT', 'QMultiHeadAttention', 'QLayerBase',
           'QLayerBaseSingleInput', 'QLayerBaseMultiInputs']
