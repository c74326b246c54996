"""QMultiHeadAttention (mirror of src/hgq/layers/attn/mha.py:25-537) for [batch, sequence, features] inputs.

Q, K, V and output projections are QEinsumDense layers with an output quantizer; the scores go through QSoftmax
(bit-accurate, the 1/sqrt(key_dim) scale folded into the exp table's input); EBOPs of the two activation-activation
products (Q K^T and attention x V) are added by this layer from the projections' output bitwidths.
Masks, dropout and attention axes other than the sequence axis are outside the accelerated path.
"""

from __future__ import annotations

import math

import torch

from ... import routes
from ...backend import Constant, queue_params
from ...quantizer.config import QuantizerConfig
from .._functions import AttnContextFn, AttnScoresFn, EbopsDenseFn, attn_products_supported
from ..core.base import QLayerBase
from ..core.einsum_dense import QEinsumDense
from ..softmax import QSoftmax


class QMultiHeadAttention(QLayerBase):
    __output_quantizer_handled__ = True

    def __init__(self, num_heads, key_dim, value_dim=None, dropout=0.0, use_bias=True, output_shape=None,
                 attention_axes=None, kernel_initializer='glorot_uniform', bias_initializer='zeros', fuse='none',
                 qkvo_iq_conf: QuantizerConfig | None = None, qkvo_kq_conf: QuantizerConfig | None = None,
                 qkvo_bq_conf: QuantizerConfig | None = None, qkvo_oq_conf: QuantizerConfig | None = None,
                 softmax_iq_conf: QuantizerConfig | None = None, softmax_exp_iq_conf: QuantizerConfig | None = None,
                 softmax_exp_oq_conf: QuantizerConfig | None = None, softmax_inv_iq_conf: QuantizerConfig | None = None,
                 softmax_inv_oq_conf: QuantizerConfig | None = None, softmax_oq_conf: QuantizerConfig | None = None,
                 stable_softmax=True, softmax_allow_heterogeneous_table: bool = False, parallelization_factor=-1, **kwargs):
        if dropout:
            raise NotImplementedError('attention dropout is not supported')
        if attention_axes is not None:
            raise NotImplementedError('custom attention_axes are not supported')
        self._qkvo_iq_conf = qkvo_iq_conf or QuantizerConfig(place='datalane')
        self._qkvo_kq_conf = qkvo_kq_conf or QuantizerConfig(place='weight')
        self._qkvo_bq_conf = qkvo_bq_conf or QuantizerConfig(place='bias')
        self._qkvo_oq_conf = qkvo_oq_conf or QuantizerConfig(place='datalane')
        self._softmax_iq_conf = softmax_iq_conf or QuantizerConfig(place='datalane')
        self._softmax_exp_iq_conf = softmax_exp_iq_conf or QuantizerConfig(place='datalane', overflow_mode='SAT')
        self._softmax_exp_oq_conf = softmax_exp_oq_conf or QuantizerConfig(place='table')
        self._softmax_inv_iq_conf = softmax_inv_iq_conf or QuantizerConfig(place='datalane')
        self._softmax_inv_oq_conf = softmax_inv_oq_conf or QuantizerConfig(place='table')
        self._softmax_oq_conf = softmax_oq_conf or QuantizerConfig(place='datalane')
        self._softmax_allow_heterogeneous_table = softmax_allow_heterogeneous_table
        self.parallelization_factor = parallelization_factor
        self._stable_softmax = stable_softmax
        self._fuse = fuse.lower()
        self._num_heads, self._key_dim = int(num_heads), int(key_dim)
        self._value_dim = int(value_dim) if value_dim else int(key_dim)
        self._use_bias = use_bias
        self._output_shape = output_shape
        self._kernel_initializer, self._bias_initializer = kernel_initializer, bias_initializer
        self._inverse_sqrt_key_dim = 1.0 / math.sqrt(float(key_dim))
        self._n_projections = 0
        super().__init__(**kwargs)

    def _common(self):
        init = self._kernel_initializer
        if getattr(init, 'seed', None) is not None:  # a seeded initializer: each projection gets its own stream
            init = init.clone()
            init.seed = init.seed + self._n_projections
            self._n_projections += 1
        return dict(kernel_initializer=init, bias_initializer=self._bias_initializer,
                    iq_conf=self._qkvo_iq_conf, kq_conf=self._qkvo_kq_conf, bq_conf=self._qkvo_bq_conf,
                    oq_conf=self._qkvo_oq_conf, enable_ebops=self.enable_ebops, beta0=self._beta0.clone(),
                    parallelization_factor=self.parallelization_factor)

    def build(self, query_shape, value_shape=None, key_shape=None):
        value_shape = query_shape if value_shape is None else value_shape
        key_shape = value_shape if key_shape is None else key_shape
        if len(query_shape) != 3:
            raise NotImplementedError('only [batch, sequence, features] inputs are supported')
        if self._fuse == 'qkv':
            assert tuple(query_shape) == tuple(value_shape) == tuple(key_shape)
        if self._fuse == 'kv':
            assert tuple(value_shape) == tuple(key_shape)
        H, dk, dv = self._num_heads, self._key_dim, self._value_dim
        proj, bias_axes = 'abc,cde->abde', 'de'
        self._query_dense = QEinsumDense(proj, (query_shape[1], H, dk), bias_axes=bias_axes if self._use_bias else None,
                                         name=f'{self.name}_query', enable_iq=self.enable_iq and self._fuse != 'qkv',
                                         enable_oq=True, **self._common())
        self._key_dense = QEinsumDense(proj, (key_shape[1], H, dk), bias_axes=None, name=f'{self.name}_key',
                                       enable_iq=self.enable_iq and self._fuse not in ('qkv', 'kv'), enable_oq=True,
                                       **self._common())
        self._value_dense = QEinsumDense(proj, (value_shape[1], H, dv), bias_axes=bias_axes if self._use_bias else None,
                                         name=f'{self.name}_value', enable_iq=self.enable_iq, enable_oq=True, **self._common())
        self._value_dense.build(value_shape)
        self._value_dense.built = True
        if self._fuse == 'qkv' and self.enable_iq:
            self._query_dense._iq = self._value_dense._iq
            self._query_dense._enable_iq = True
        if self._fuse in ('qkv', 'kv') and self.enable_iq:
            self._key_dense._iq = self._value_dense._iq
            self._key_dense._enable_iq = True
        self._query_dense.build(query_shape)
        self._query_dense.built = True
        self._key_dense.build(key_shape)
        self._key_dense.built = True
        # scores [B, N, T, S] = einsum('aecd,abcd->acbe', key, query); output [B, T, N, H] = einsum('acbe,aecd->abcd', attn, value)
        self._dot_product_equation, self._combine_equation = 'aecd,abcd->acbe', 'acbe,aecd->abcd'
        self._softmax = QSoftmax(enable_oq=True, axis=(3,), stable=self._stable_softmax, iq_conf=self._softmax_iq_conf,
                                 exp_iq_conf=self._softmax_exp_iq_conf, exp_oq_conf=self._softmax_exp_oq_conf,
                                 inv_iq_conf=self._softmax_inv_iq_conf, inv_oq_conf=self._softmax_inv_oq_conf,
                                 oq_conf=self._softmax_oq_conf, allow_heterogeneous_table=self._softmax_allow_heterogeneous_table,
                                 input_scaler=self._inverse_sqrt_key_dim, enable_ebops=self.enable_ebops,
                                 name=f'{self.name}_softmax')
        self._inverse_sqrt_key_dim = 1.0
        self._softmax.build((None, H, query_shape[1], value_shape[1]))
        self._softmax.built = True
        out_dims = [query_shape[-1]] if not self._output_shape else (
            [self._output_shape] if isinstance(self._output_shape, int) else list(self._output_shape))
        assert len(out_dims) == 1, 'only a 1-D output_shape is supported'
        self._output_dense = QEinsumDense('abcd,cde->abe', (query_shape[1], out_dims[0]),
                                          bias_axes='e' if self._use_bias else None, name=f'{self.name}_attention_output',
                                          enable_iq=True, enable_oq=self.enable_oq, **self._common())
        self._output_dense.build((query_shape[0], query_shape[1], H, dv))
        self._output_dense.built = True
        if self.enable_ebops:
            self._beta = self.add_weight(name='beta', shape=(), initializer=self._beta0, trainable=False)
            self._ebops = self.add_weight(name='ebops', shape=(), initializer=Constant(0.0), trainable=False, dtype='uint32')
        else:
            self._beta = None
            self._ebops = None
        if self.enable_oq and not self.oq.built:
            self.oq.build((query_shape[0], query_shape[1], out_dims[0]))
            self.oq.built = True
        self.built = True

    def _compute_ebops(self, query_shape, value_shape=None, key_shape=None):
        Q_shape = (1,) + tuple(self._query_dense.full_output_shape[1:])
        K_shape = (1,) + tuple(self._key_dense.full_output_shape[1:])
        V_shape = (1,) + tuple(self._value_dense.full_output_shape[1:])
        value_shape = query_shape if value_shape is None else value_shape
        attn_shape = (1, self._num_heads, query_shape[1], value_shape[1])
        bw_q = self._query_dense.oq.bits_(Q_shape)[0]      # [T, N, H]
        bw_k = self._key_dense.oq.bits_(K_shape)[0]        # [S, N, H]
        bw_v = self._value_dense.oq.bits_(V_shape)[0]      # [S, N, Hv]
        bw_attn = self._softmax.oq.bits_(attn_shape)[0]    # [N, T, S]
        T, N, H = bw_q.shape
        S = bw_k.shape[0]
        # sum_{e,b,c,d} k[e,c,d] q[b,c,d]: contraction index (c,d), free e and b
        ebops_qk = EbopsDenseFn.apply(bw_k.reshape(S, N * H), bw_q.reshape(T, N * H).t(), None, 0.0, 1.0)
        # sum_{c,b,e,d} attn[c,b,e] v[e,c,d]: contraction index (c,e), free b and d
        ebops_av = EbopsDenseFn.apply(bw_attn.permute(1, 0, 2).reshape(T, N * S), bw_v.permute(1, 0, 2).reshape(N * S, -1), None,
                                      0.0, 1.0)
        ebops = ebops_qk + ebops_av
        if self.parallelization_factor > 0:
            return ebops * self.parallelization_factor
        return ebops

    @property
    def ebops(self):
        if self._ebops is None:
            return torch.zeros((), dtype=torch.uint32)
        parts = (self._query_dense.ebops, self._key_dense.ebops, self._value_dense.ebops, self._output_dense.ebops,
                 self._ebops.value.detach())
        return sum(p.to(torch.int64) for p in parts) + self._softmax.ebops

    def call(self, query, value=None, key=None, attention_mask=None, return_attention_scores=False, training=None):
        if attention_mask is not None:
            raise NotImplementedError('attention masks are not supported')
        if value is None:
            value = query
        if key is None:
            key = value
        if training and query.is_cuda:
            queue_params((self._query_dense, self._key_dense, self._value_dense, self._output_dense))
        query = self._query_dense(query)
        key = self._key_dense(key)
        value = self._value_dense(value)
        attention_output, attention_scores = self._compute_attention(query, key, value, training)
        attention_output = self._output_dense(attention_output)
        if self.enable_oq:
            attention_output = self.oq(attention_output, training=training)
        if return_attention_scores:
            return attention_output, attention_scores
        return attention_output

    def _compute_attention(self, query, key, value, training=None):
        if self._inverse_sqrt_key_dim != 1.0:  # 1.0 after build: the scale lives in the exp table's input
            query = query * self._inverse_sqrt_key_dim
        if attn_products_supported(query, key, value):
            scores = self._softmax(AttnScoresFn.apply(key, query))
            return AttnContextFn.apply(scores, value), scores
        routes.fallback('torch.einsum', f'attention products of {self.name}')
        scores = torch.einsum(self._dot_product_equation, key, query)
        scores = self._softmax(scores)
        return torch.einsum(self._combine_equation, scores, value), scores

    def compute_output_shape(self, query_shape, value_shape=None, key_shape=None):
        return tuple(query_shape)
