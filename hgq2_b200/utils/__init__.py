"""Utilities around the quantised layers (mirror of src/hgq/utils): calibration, weight files."""

from .minmax_trace import TrainingFlagWrapper, trace_minmax
from .weights import load_weights, save_weights, state_tree

__all__ = ['TrainingFlagWrapper', 'trace_minmax', 'save_weights', 'load_weights', 'state_tree']
