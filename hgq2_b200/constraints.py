"""Post-update clamps for bitwidth variables (mirror of src/hgq/constraints/__init__.py:11-69)."""

from __future__ import annotations

import torch

__all__ = ['Constraint', 'MinMax', 'Min', 'Max', 'Constant']


class Constraint:
    def __call__(self, w: torch.Tensor) -> torch.Tensor:
        return w

    def get_config(self):
        return {}


class MinMax(Constraint):
    """Constrains the weights to between min_value and max_value."""

    def __init__(self, min_value, max_value):
        self.min_value = float(min_value)
        self.max_value = float(max_value)

    def __call__(self, w):
        return torch.clamp(w, self.min_value, self.max_value)

    def get_config(self):
        return {'min_value': self.min_value, 'max_value': self.max_value}


class Constant(Constraint):
    """Constrains the weights to a constant value."""

    def __init__(self, value):
        self.value = float(value)

    def __call__(self, w):
        return torch.full_like(w, self.value)

    def get_config(self):
        return {'value': self.value}


class Min(Constraint):
    """Constrains the weights to greater or equal than min_value."""

    def __init__(self, min_value):
        self.min_value = float(min_value)

    def __call__(self, w):
        return torch.clamp(w, min=self.min_value)

    def get_config(self):
        return {'min_value': self.min_value}


class Max(Constraint):
    """Constrains the weights to less or equal than max_value."""

    def __init__(self, max_value):
        self.max_value = float(max_value)

    def __call__(self, w):
        return torch.clamp(w, max=self.max_value)

    def get_config(self):
        return {'max_value': self.max_value}
