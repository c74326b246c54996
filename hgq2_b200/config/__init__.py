from ..quantizer.config import HardSigmoidConfig, HardTanhConfig, QuantizerConfig, QuantizerConfigScope, default_configs
from .layer import LayerConfigScope, global_config

__all__ = [
    'LayerConfigScope',
    'QuantizerConfigScope',
    'QuantizerConfig',
    'global_config',
    'default_configs',
    'HardTanhConfig',
    'HardSigmoidConfig',
]
