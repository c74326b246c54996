"""Writes the golden fixtures of the stateless quantizer.

    python tests/golden/make_quantizer_golden.py

Two files are produced next to this script:

quantizer_kat.json
    Known-answer table worked out by hand from the fixed-point semantics (step 2^-f, range
    [-k 2^i, 2^i - 2^-f], ap_fixed rounding/overflow modes); it does not come from running any
    code and pins the oracle itself.  Each row: x, (k, i, f) and, per round mode, the expected
    eval-mode output under WRAP / SAT / SAT_SYM.

quantizer_golden.npz
    Seeded inputs and the outputs of oracle/fixed_point_ops.py (forward in eval and training
    mode, closed-form backward) for every round x overflow mode.  The GPU tests compare the CUDA
    kernels against these arrays so that a change in either side shows up.
"""

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import fixed_point_ops as O  # noqa: E402

KAT = [
    # x, (k, i, f), {round_mode: [WRAP, SAT, SAT_SYM]}
    (1.30, (1, 1, 2), {'RND': [1.25, 1.25, 1.25], 'TRN': [1.25, 1.25, 1.25], 'RND_CONV': [1.25, 1.25, 1.25]}),
    (1.90, (1, 1, 2), {'RND': [-2.0, 1.75, 1.75], 'TRN': [1.75, 1.75, 1.75], 'RND_CONV': [-2.0, 1.75, 1.75]}),
    (-2.20, (1, 1, 2), {'RND': [1.75, -2.0, -1.75], 'TRN': [1.75, -2.0, -1.75], 'RND_CONV': [1.75, -2.0, -1.75]}),
    (0.625, (1, 1, 2), {'RND': [0.75] * 3, 'TRN': [0.5] * 3, 'RND_CONV': [0.5] * 3}),
    (-0.625, (1, 1, 2), {'RND': [-0.5] * 3, 'TRN': [-0.75] * 3, 'RND_CONV': [-0.5] * 3}),
    (0.375, (1, 1, 2), {'RND': [0.5] * 3, 'TRN': [0.25] * 3, 'RND_CONV': [0.5] * 3}),
    (-0.30, (0, 1, 2), {'RND': [1.75, 0.0, 0.0], 'TRN': [1.5, 0.0, 0.0], 'RND_CONV': [1.75, 0.0, 0.0]}),
    (2.60, (0, 1, 2), {'RND': [0.5, 1.75, 1.75], 'TRN': [0.5, 1.75, 1.75], 'RND_CONV': [0.5, 1.75, 1.75]}),
    (5.10, (1, 2, 0), {'RND': [-3.0, 3.0, 3.0], 'TRN': [-3.0, 3.0, 3.0], 'RND_CONV': [-3.0, 3.0, 3.0]}),
]


def make_inputs(n=4096, seed=1234):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 4.0).astype(np.float32)
    # adversarial values: grid points, ties, range edges, +-1 ulp around them, zeros, large values
    special = []
    for f in (0, 2, 5, 8):
        for m in (-9, -1, 0, 1, 3, 63, 64, 255):
            for d in (0.0, 0.5):
                v = np.float32((m + d) / 2.0**f)
                special += [v, np.nextafter(v, np.float32(np.inf)), np.nextafter(v, np.float32(-np.inf))]
    special += [0.0, -0.0, 1e-30, -1e-30, 300.0, -300.0, 65504.0, -7.999, 7.999]
    special = np.array(special, dtype=np.float32)
    x[: special.size] = special
    k = rng.integers(0, 2, n).astype(np.uint8)
    i = rng.integers(-2, 7, n).astype(np.float32)
    f = rng.integers(0, 9, n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    return x, k, i, f, g


def main():
    (HERE / 'quantizer_kat.json').write_text(
        json.dumps([{'x': x, 'kif': list(kif), 'expect': exp} for x, kif, exp in KAT], indent=1) + '\n'
    )
    x, k, i, f, g = make_inputs()
    out = dict(x=x, k=k, i=i, f=f, g=g)
    tx, tk, ti, tf, tg = (torch.from_numpy(a.astype(np.float32)) for a in (x, k, i, f, g))
    for rm in O.ROUND_MODES:
        for om in O.OVERFLOW_MODES:
            out[f'y_eval_{rm}_{om}'] = O.quantize_fwd(tx, tk, ti, tf, rm, om, training=False).numpy()
            out[f'y_train_{rm}_{om}'] = O.quantize_fwd(tx, tk, ti, tf, rm, om, training=True).numpy()
            dx, di, df = O.quantize_bwd(tg, tx, tk, ti, tf, rm, om)
            out[f'dx_{rm}_{om}'], out[f'di_{rm}_{om}'], out[f'df_{rm}_{om}'] = dx.numpy(), di.numpy(), df.numpy()
    np.savez_compressed(HERE / 'quantizer_golden.npz', **out)
    print('wrote', HERE / 'quantizer_kat.json', HERE / 'quantizer_golden.npz')


if __name__ == '__main__':
    main()
