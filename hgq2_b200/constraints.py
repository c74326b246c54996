"""Clamps applied to bitwidth variables after every optimizer update.

Interface of src/hgq/constraints/__init__.py:11-69 (``MinMax``, ``Min``, ``Max``, ``Constant`` with Keras'
``__call__`` / ``get_config`` protocol).  All four are one class of clamp with optional bounds; the fused optimizer
kernel reads ``min_value`` / ``max_value`` straight from the instances.
"""

from __future__ import annotations

import math

import torch

__all__ = ['Constraint', 'MinMax', 'Min', 'Max', 'Constant']


class Constraint:
    """Identity; subclasses set the bounds they enforce."""

    _fields: tuple = ()

    def __call__(self, w: torch.Tensor) -> torch.Tensor:
        return w

    def get_config(self) -> dict:
        return {name: getattr(self, name) for name in self._fields}


class _Clamp(Constraint):
    min_value = -math.inf
    max_value = math.inf

    def __call__(self, w):
        lo = None if self.min_value == -math.inf else self.min_value
        hi = None if self.max_value == math.inf else self.max_value
        return w if lo is None and hi is None else torch.clamp(w, min=lo, max=hi)


class MinMax(_Clamp):
    """min_value <= w <= max_value."""

    _fields = ('min_value', 'max_value')

    def __init__(self, min_value, max_value):
        self.min_value, self.max_value = float(min_value), float(max_value)


class Min(_Clamp):
    """w >= min_value."""

    _fields = ('min_value',)

    def __init__(self, min_value):
        self.min_value = float(min_value)


class Max(_Clamp):
    """w <= max_value."""

    _fields = ('max_value',)

    def __init__(self, max_value):
        self.max_value = float(max_value)


class Constant(Constraint):
    """w == value everywhere."""

    _fields = ('value',)

    def __init__(self, value):
        self.value = float(value)

    def __call__(self, w):
        return torch.full_like(w, self.value)
