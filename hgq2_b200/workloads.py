"""The benchmark models of this package: the layer stacks the throughput figures are quoted on.

Each builder returns a ``Sequential`` of hgq2_b200 layers with the quantizer configuration of the workload:
weights kbi (SAT_SYM, RND) with per-weight ``b`` drawn uniformly from an integer range by assignment after build,
activations kif (WRAP, RND) per activation, EBOPs on.
"""

from __future__ import annotations

import numpy as np
import torch

from .backend import Flatten, Lambda, MaxPooling2D, Sequential
from .config import LayerConfigScope, QuantizerConfigScope
from .layers import QConv2D, QDense, QEinsumDense, QMultiHeadAttention
from .quantizer import QuantizerConfig
from .quantizer.internal import FixedPointQuantizerKBI


def _scopes(act_i, act_f, beta0):
    w = QuantizerConfigScope(place='weight', default_q_type='kbi', overflow_mode='SAT_SYM', round_mode='RND', b0=8, i0=2)
    a = QuantizerConfigScope(place='datalane', default_q_type='kif', overflow_mode='WRAP', round_mode='RND', i0=act_i,
                             f0=act_f)
    return w, a, LayerConfigScope(beta0=beta0, enable_ebops=True)


def randomize_weight_bits(model, lo: int, hi: int, seed: int = 3) -> None:
    """Assign integer ``b`` ~ U[lo, hi] to every weight quantizer (per weight), the way the reference's tests perturb
    bitwidths: by assignment after build."""
    rng = np.random.default_rng(seed)
    for q in model._flatten_layers():
        if isinstance(q, FixedPointQuantizerKBI) and q._is_weight:
            b = rng.integers(lo, hi + 1, q._b.shape).astype(np.float32)
            q._b.assign(torch.from_numpy(b))


def _seeded(layers, seed=0):
    """Glorot-uniform kernels drawn from consecutive seeds so that builds are reproducible."""
    from .backend import GlorotUniform

    for j, layer in enumerate(layers):
        if hasattr(layer, 'kernel_initializer'):
            layer.kernel_initializer = GlorotUniform(seed + j)
        elif hasattr(layer, '_kernel_initializer'):  # attention: its four projections draw from seed, seed + 1, ...
            layer._kernel_initializer = GlorotUniform(1000 * (seed + j + 1))
    return layers


def jet_tagger_mlp(beta0=1e-5):
    """Small jet tagger: QDense 16 -> 64 -> 32 -> 32 -> 5, ReLU, activations kif i=3 f=4, weights kbi b in [4, 8]."""
    w, a, l = _scopes(3, 4, beta0)
    with w, a, l:
        layers = _seeded([QDense(64, activation='relu'), QDense(32, activation='relu'), QDense(32, activation='relu'),
                          QDense(5)])
    model = Sequential(layers, name='jet_tagger_mlp')
    model.input_shape = (16,)
    model.weight_bits = (4, 8)
    return model


def particle_tagger(n_particles=64, n_features=16, beta0=1e-5):
    """Particle-set tagger: per-particle QEinsumDense 16 -> 64 -> 64, sum over particles, QDense 64 -> 64 -> 5."""
    w, a, l = _scopes(4, 6, beta0)
    with w, a, l:
        layers = _seeded([
            QEinsumDense('bpc,cd->bpd', (n_particles, 64), bias_axes='d', activation='relu'),
            QEinsumDense('bpc,cd->bpd', (n_particles, 64), bias_axes='d', activation='relu'),
            Lambda(lambda x: x.sum(dim=1), name='sum_particles'),
            QDense(64, activation='relu'),
            QDense(5),
        ])
    model = Sequential(layers, name='particle_tagger')
    model.input_shape = (n_particles, n_features)
    model.weight_bits = (4, 8)
    return model


def small_cnn(beta0=1e-5):
    """Small CNN on 32x32x3: QConv2D 3x3 16/32/64 + ReLU + 2x2 max-pool each, Flatten, QDense 10."""
    w, a, l = _scopes(2, 5, beta0)
    with w, a, l:
        layers = _seeded([
            QConv2D(16, 3, activation='relu'), MaxPooling2D(2),
            QConv2D(32, 3, activation='relu'), MaxPooling2D(2),
            QConv2D(64, 3, activation='relu'), MaxPooling2D(2),
            Flatten(), QDense(10),
        ])
    model = Sequential(layers, name='small_cnn')
    model.input_shape = (32, 32, 3)
    model.weight_bits = (3, 8)
    return model


def transformer_block(seq=64, d_model=64, heads=4, beta0=1e-5):
    """Transformer block: QMultiHeadAttention (4 heads, key_dim 16, bit-accurate softmax with 10-bit exp / inverse
    tables), QDense 64 -> 128 -> 64 feed-forward, mean over the sequence, QDense -> 5 classes.  Score and softmax
    activations kif i=4 f=8."""
    w, a, l = _scopes(4, 8, beta0)
    t = QuantizerConfigScope(place='table', b0=10, i0=1)
    with w, a, t, l:
        table_in = dict(k0=0, i0=4, f0=6)  # 10-bit table index
        mha = QMultiHeadAttention(
            heads, d_model // heads,
            softmax_exp_iq_conf=QuantizerConfig(place='datalane', overflow_mode='SAT', **table_in),
            softmax_inv_iq_conf=QuantizerConfig(place='datalane', **dict(k0=0, i0=7, f0=3)),
        )
        layers = _seeded([
            mha,
            QDense(128, activation='relu'),
            QDense(d_model),
            Lambda(lambda x: x.mean(dim=1), name='mean_sequence'),
            QDense(5),
        ])
    model = Sequential(layers, name='transformer_block')
    model.input_shape = (seq, d_model)
    model.weight_bits = (4, 8)
    return model


def build(model, batch: int = 2, device=None):
    """Run one eval forward on zeros to create the variables, then randomise the weight bitwidths."""
    from .backend import default_device

    device = device or default_device()
    x = torch.zeros((batch,) + tuple(model.input_shape), device=device)
    model(x, training=False)
    randomize_weight_bits(model, *model.weight_bits)
    return model
