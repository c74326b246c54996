from .config import QuantizerConfig
from .quantizer import Quantizer

__all__ = ['QuantizerConfig', 'Quantizer']
