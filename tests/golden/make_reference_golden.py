"""Writes ``quantizer_golden_reference.npz``: the same keys as ``quantizer_golden.npz``, but computed by the REAL
third-party ``quantizers`` package (the one HGQ2 imports at src/hgq/quantizer/internal/fixed_point_quantizer.py:9-10)
instead of this repository's oracle.

    KERAS_BACKEND=torch python tests/golden/make_reference_golden.py

It needs ``keras`` (>= 3.11) and ``quantizers`` (>= 1.2.2) to be importable; neither is installed in the image this
repository was built in, so the file it writes is not committed and parity of the oracle with the reference's arithmetic
stays unpinned until someone runs it.  When the file is present, ``tests/test_oracle.py`` and the GPU golden test compare
against it in preference to the oracle-made file, which turns every convention the oracle had to choose into a checked
fact in one place:

* forward, eval mode (``training=False``): WRAP wraps, SAT / SAT_SYM clip; behaviour where ``i + f < 0`` (upper bound
  below lower bound);
* forward, training mode (``training=True``): what WRAP does to an out-of-range value;
* backward through ``q(x, k, i, f, training=True)``: gradients w.r.t. ``x``, ``i`` and ``f`` obtained by autograd from
  an upstream gradient ``g`` (the surrogate gradients: straight-through in ``x`` with the SAT clip mask, the
  -ln2 * (round(x) - x) term in ``f``, the routing of clipped elements to ``i`` / ``f``).
"""

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parent.parent))

from make_quantizer_golden import make_inputs  # noqa: E402  (same seeded inputs as the oracle-made file)

ROUND_MODES = ('TRN', 'RND', 'RND_CONV')
OVERFLOW_MODES = ('WRAP', 'SAT', 'SAT_SYM')


def main():
    try:
        import torch
        from quantizers import get_fixed_quantizer
    except ImportError as why:
        raise SystemExit(f'the reference stack is not importable here ({why}); nothing written')

    x, k, i, f, g = make_inputs()
    out = dict(x=x, k=k, i=i, f=f, g=g)
    for rm in ROUND_MODES:
        for om in OVERFLOW_MODES:
            q = get_fixed_quantizer(rm, om)
            tx = torch.from_numpy(x)
            tk, ti, tf = (torch.from_numpy(a.astype(np.float32)) for a in (k, i, f))
            out[f'y_eval_{rm}_{om}'] = np.asarray(q(tx, tk, ti, tf, False, None).detach())
            lx, li, lf = tx.clone().requires_grad_(), ti.clone().requires_grad_(), tf.clone().requires_grad_()
            y = q(lx, tk, li, lf, True, None)
            out[f'y_train_{rm}_{om}'] = np.asarray(y.detach())
            y.backward(torch.from_numpy(g))
            zero = torch.zeros_like(tx)
            out[f'dx_{rm}_{om}'] = np.asarray(lx.grad if lx.grad is not None else zero)
            out[f'di_{rm}_{om}'] = np.asarray(li.grad if li.grad is not None else zero)
            out[f'df_{rm}_{om}'] = np.asarray(lf.grad if lf.grad is not None else zero)
    np.savez_compressed(HERE / 'quantizer_golden_reference.npz', **out)
    print('wrote', HERE / 'quantizer_golden_reference.npz')


if __name__ == '__main__':
    main()
