from .conv import QConv2D
from .core import QDense, QEinsumDense, QLayerBase, QLayerBaseMultiInputs, QLayerBaseSingleInput

__all__ = ['QDense', 'QEinsumDense', 'QConv2D', 'QLayerBase', 'QLayerBaseSingleInput', 'QLayerBaseMultiInputs']
