"""Quantised element-wise merges of several inputs (mirror of src/hgq/layers/ops/merge.py)."""

from __future__ import annotations

from math import log2

import torch

from ..core.base import QLayerBaseMultiInputs


class QMerge(QLayerBaseMultiInputs):
    """Each input goes through its own quantizer, then the merge function (merge.py:10-15)."""

    def _merge_function(self, inputs):
        raise NotImplementedError

    def compute_output_shape(self, input_shape):
        return tuple(torch.broadcast_shapes(*[tuple(s) for s in input_shape]))

    def call(self, inputs, training=None):
        if self.enable_iq:
            inputs = self.iq(inputs, training=training)
        return self._merge_function(list(inputs))


def _ebops_from_sum_bits_excl_max(self: QMerge, shapes):
    bitss = [iq.bits_(tuple(shape)) for iq, shape in zip(self.iq, shapes)]
    total = torch.sum(sum(bitss))
    least = bitss[0]
    for bits in bitss[1:]:
        least = torch.minimum(least, bits)
    return total - torch.sum(least)


class QAdd(QMerge):
    def _merge_function(self, inputs):
        out = inputs[0]
        for t in inputs[1:]:
            out = out + t
        return out

    def _compute_ebops(self, *shapes):
        return _ebops_from_sum_bits_excl_max(self, shapes) * 0.65


class QAveragePow2(QAdd):
    """Average with the divisor rounded to a power of two (merge.py:33-42)."""

    def build(self, input_shape):
        super().build(input_shape)
        self._scale = 2.0 ** round(log2(1.0 / len(input_shape)))

    def _merge_function(self, inputs):
        return super()._merge_function(inputs) * self._scale


class QSubtract(QMerge):
    def _merge_function(self, inputs):
        if len(inputs) != 2:
            raise ValueError(f'A subtract layer takes exactly 2 inputs, got {len(inputs)}')
        return inputs[0] - inputs[1]

    def _compute_ebops(self, *shapes):
        bits0, bits1 = (iq.bits_(tuple(shape)) for iq, shape in zip(self.iq, shapes))
        return torch.sum(torch.maximum(bits0, bits1))


class QMultiply(QMerge):
    def _merge_function(self, inputs):
        out = inputs[0]
        for t in inputs[1:]:
            out = out * t
        return out

    def _compute_ebops(self, *shapes):
        bitss = [iq.bits_(tuple(shape)) for iq, shape in zip(self.iq, shapes)]
        out = bitss[0]
        for bits in bitss[1:]:
            out = out * bits
        return torch.sum(out)


class QMaximum(QMerge):
    def _merge_function(self, inputs):
        out = inputs[0]
        for t in inputs[1:]:
            out = torch.maximum(out, t)
        return out

    def _compute_ebops(self, *shapes):
        return 1.0 * _ebops_from_sum_bits_excl_max(self, shapes)


class QMinimum(QMerge):
    def _merge_function(self, inputs):
        out = inputs[0]
        for t in inputs[1:]:
            out = torch.minimum(out, t)
        return out

    def _compute_ebops(self, *shapes):
        return 1.0 * _ebops_from_sum_bits_excl_max(self, shapes)
