from .base import MultipleQuantizers, QLayerBase, QLayerBaseMultiInputs, QLayerBaseSingleInput
from .dense import QBatchNormDense, QDense
from .einsum_dense import QEinsumDense

__all__ = ['QLayerBase', 'QLayerBaseSingleInput', 'QLayerBaseMultiInputs', 'MultipleQuantizers', 'QDense', 'QBatchNormDense',
           'QEinsumDense']
