"""B200-native implementation of the HGQ2 quantisation-aware-training hot path.

Layout follows HGQ2: ``config`` (scopes), ``quantizer`` (``Quantizer`` and the internal KBI/KIF
quantizers), ``layers`` (``QDense``, ``QEinsumDense``, ``QConv2D``, ...), ``constraints``,
``regularizers``.  All tensor work runs in the CUDA library ``lib/libhgq_b200.so`` (built by
``python -m hgq2_b200.build``); there is no CPU fallback.
"""

from . import config, constraints, layers, quantizer, regularizers  # noqa: F401

__all__ = ['config', 'layers', 'quantizer', 'constraints', 'regularizers']
