from .accum import QMeanPow2, QSum
from .merge import QAdd, QAveragePow2, QMaximum, QMinimum, QMultiply, QSubtract

__all__ = ['QMeanPow2', 'QSum', 'QAdd', 'QAveragePow2', 'QMaximum', 'QMinimum', 'QMultiply', 'QSubtract']
