"""Layer-level defaults and their scope (mirror of src/hgq/config/layer.py:14-41)."""

from __future__ import annotations

global_config = dict(
    beta0=1e-5,
    enable_ebops=True,
    enable_oq=False,
    enable_iq=True,
    enable_sq=True,
)


class LayerConfigScope:
    """Overrides entries of ``global_config`` inside a ``with`` block and restores them on exit."""

    def __init__(self, **kwargs):
        self._override = kwargs

    def __enter__(self):
        self._tmp = global_config.copy()
        for k, v in self._override.items():
            global_config[k] = v

    def __exit__(self, exc_type, exc_val, exc_tb):
        for k in self._override:
            del global_config[k]
        global_config.update(self._tmp)
