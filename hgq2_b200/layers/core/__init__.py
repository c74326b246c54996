from .base import MultipleQuantizers, QLayerBase, QLayerBaseMultiInputs, QLayerBaseSingleInput
from .dense import QDense
from .einsum_dense import QEinsumDense

__all__ = ['QLayerBase', 'QLayerBaseSingleInput', 'QLayerBaseMultiInputs', 'MultipleQuantizers', 'QDense', 'QEinsumDense']
