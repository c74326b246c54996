"""Which code path a call took: per-entry-point call counters and a strict mode that refuses library fallbacks.

Every call into ``libhgq_b200.so`` is counted under the name of its C-ABI entry point (``hgq_qdense_fwd``,
``hgq_attn_heads_matmul``, ...).  Every place where a layer leaves the package's own kernels for a library routine
(``torch.matmul`` / cuBLAS, cuDNN, ``torch.einsum``, the element-wise softmax chain) reports it through ``fallback``:
the event is counted under ``fallback:<what>`` and, in strict mode, raises ``FallbackError`` instead of running the
library routine.  Strict mode is what the benchmark and the model-level tests run under, so a shape that silently
drops off the fused path shows up as an error and not as a slower number.

    with routes.strict_mode():
        trainer.step(x, y)          # raises if any layer would call a library contraction
    routes.counts['hgq_qdense_bwd_strided']

The environment variable ``HGQ_STRICT=1`` turns strict mode on for the whole process.
"""

from __future__ import annotations

import os
from collections import Counter
from contextlib import contextmanager

counts: Counter = Counter()
strict: bool = os.environ.get('HGQ_STRICT', '0') not in ('', '0')


class FallbackError(RuntimeError):
    """A layer would have left the package's kernels for a library routine while strict mode was on."""


def took(name: str) -> None:
    counts[name] += 1


def fallback(what: str, why: str = '') -> None:
    """Report that the caller is about to run library routine ``what`` instead of a kernel of this package."""
    counts['fallback:' + what] += 1
    if strict:
        raise FallbackError(f'strict mode: {what} would run instead of a fused kernel' + (f' ({why})' if why else ''))


def fallbacks() -> dict[str, int]:
    return {k[len('fallback:'):]: v for k, v in counts.items() if k.startswith('fallback:')}


def reset() -> None:
    counts.clear()


@contextmanager
def strict_mode(on: bool = True):
    global strict
    prev, strict = strict, on
    try:
        yield
    finally:
        strict = prev


class CountingLibrary:
    """The ctypes handle with every function wrapped so that a call is counted under the symbol's name."""

    def __init__(self, handle):
        self.__dict__['_handle'] = handle

    def __getattr__(self, name):
        fn = getattr(self._handle, name)
        if not name.startswith('hgq_') or name.endswith(('_workspace', '_supported', '_count', '_string', '_version')):
            self.__dict__[name] = fn
            return fn

        def counted(*args, _fn=fn, _name=name):
            counts[_name] += 1
            return _fn(*args)

        self.__dict__[name] = counted
        return counted
