"""Bitwidth regulariser (mirror of src/hgq/regularizers/__init__.py:8-17)."""

from __future__ import annotations

import torch

__all__ = ['Regularizer', 'MonoL1']


class Regularizer:
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class MonoL1(Regularizer):
    """l1 * sum(x): signed, not absolute -- it pushes bitwidths down at a constant rate."""

    def __init__(self, l1):
        self.l1 = float(l1)

    def __call__(self, x):
        return self.l1 * torch.sum(x)

    def get_config(self):
        return {'l1': self.l1}
