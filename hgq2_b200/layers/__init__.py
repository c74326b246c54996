from .activation import QUnaryFunctionLUT
from .batch_normalization import QBatchNormalization
from .attn.mha import QMultiHeadAttention
from .conv import QConv1D, QConv2D
from .core import QBatchNormDense, QDense, QEinsumDense, QLayerBase, QLayerBaseMultiInputs, QLayerBaseSingleInput
from .einsum_dense_batchnorm import QEinsumDenseBatchnorm
from .ops import QAdd, QAveragePow2, QMaximum, QMeanPow2, QMinimum, QMultiply, QSubtract, QSum
from .pooling import (
    QAveragePooling1D,
    QAveragePooling2D,
    QGlobalAveragePooling1D,
    QGlobalAveragePooling2D,
    QGlobalMaxPooling1D,
    QGlobalMaxPooling2D,
    QMaxPooling1D,
    QMaxPooling2D,
)
from .softmax import QSoftmax

__all__ = [
    'QDense', 'QEinsumDense', 'QConv1D', 'QConv2D', 'QSoftmax', 'QUnaryFunctionLUT', 'QMultiHeadAttention', 'QLayerBase',
    'QLayerBaseSingleInput', 'QLayerBaseMultiInputs', 'QSum', 'QMeanPow2', 'QAdd', 'QAveragePow2', 'QSubtract', 'QMultiply',
    'QMaximum', 'QMinimum', 'QMaxPooling1D', 'QAveragePooling1D', 'QMaxPooling2D', 'QAveragePooling2D', 'QGlobalAveragePooling1D', 'QGlobalAveragePooling2D',
    'QGlobalMaxPooling1D', 'QGlobalMaxPooling2D', 'QBatchNormalization', 'QBatchNormDense', 'QEinsumDenseBatchnorm',
]
