"""Layer-level defaults (``global_config``) and the ``with`` scope that overrides them.

Interface of src/hgq/config/layer.py:14-41: a module-level dict that layers read at construction time, and a context
manager that puts every entry back the way it found it.
"""

from __future__ import annotations

_ABSENT = object()

global_config: dict = {'beta0': 1e-5, 'enable_ebops': True, 'enable_oq': False, 'enable_iq': True, 'enable_sq': True}


class LayerConfigScope:
    """``with LayerConfigScope(beta0=1e-3, enable_oq=True): ...`` -- layers constructed inside see the given values."""

    def __init__(self, **overrides):
        self._overrides = dict(overrides)
        self._saved: dict = {}

    def __enter__(self):
        self._saved = {key: global_config.get(key, _ABSENT) for key in self._overrides}
        global_config.update(self._overrides)

    def __exit__(self, exc_type, exc_value, traceback):
        for key, old in self._saved.items():
            if old is _ABSENT:
                global_config.pop(key, None)
            else:
                global_config[key] = old
        self._saved = {}
