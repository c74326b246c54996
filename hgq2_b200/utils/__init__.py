"""Utilities around the quantised layers (mirror of src/hgq/utils): calibration."""

from .minmax_trace import TrainingFlagWrapper, trace_minmax

__all__ = ['TrainingFlagWrapper', 'trace_minmax']
