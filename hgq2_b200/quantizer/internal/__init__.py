from .base import BitwidthMapperBase, DefaultBitwidthMapper, DummyQuantizer, TrainableQuantizerBase, numbers
from .fixed_point_quantizer import FixedPointQuantizerBase, FixedPointQuantizerKBI, FixedPointQuantizerKIF

__all__ = [
    'BitwidthMapperBase',
    'DefaultBitwidthMapper',
    'DummyQuantizer',
    'TrainableQuantizerBase',
    'FixedPointQuantizerBase',
    'FixedPointQuantizerKBI',
    'FixedPointQuantizerKIF',
    'numbers',
]
