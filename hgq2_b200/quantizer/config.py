"""Quantizer configuration: per-(type, place) defaults, ``QuantizerConfig`` and ``QuantizerConfigScope``.

Mirror of src/hgq/quantizer/config.py.  The defaults table (reference :75-220) and the scope
semantics (reference :550-638: a ``with`` block mutates the module-level tables and restores them on
exit; ``override()`` makes the change permanent) are the same, so model-building code written for
HGQ2 produces identically configured quantizers.  The minifloat ('float') quantizer type is outside
the accelerated path and is not provided.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence

from ..constraints import Constant, MinMax
from ..regularizers import MonoL1
from .internal import DummyQuantizer, FixedPointQuantizerKBI, FixedPointQuantizerKIF, TrainableQuantizerBase

default_q_type = {
    'weight': 'kbi',
    'datalane': 'kif',
    'bias': 'kbi',
    'table': 'kbi',
}

_COMMON = ('homogeneous_axis', 'heterogeneous_axis', 'bw_mapper', 'trainable', 'is_weight')


def _kbi(overflow_mode, bc, i_decay_speed, homogeneous_axis, is_weight):
    return dict(
        k0=True, b0=8, i0=2, round_mode='RND', overflow_mode=overflow_mode, bc=bc, ic=None, br=MonoL1(1e-8), ir=None,
        i_decay_speed=i_decay_speed, homogeneous_axis=homogeneous_axis, heterogeneous_axis=None, bw_mapper=None,
        trainable=True, is_weight=is_weight,
    )


def _kif(overflow_mode, i_decay_speed, homogeneous_axis, is_weight):
    return dict(
        k0=True, i0=2, f0=6, round_mode='RND', overflow_mode=overflow_mode, ic=MinMax(-23, 23), ir=MonoL1(1e-8),
        fc=MinMax(-24, 24), fr=MonoL1(1e-8), i_decay_speed=i_decay_speed, homogeneous_axis=homogeneous_axis,
        heterogeneous_axis=None, bw_mapper=None, trainable=True, is_weight=is_weight,
    )


kbi_weight_default = _kbi('SAT_SYM', MinMax(0, 23), float('inf'), (), True)
kbi_datalane_default = _kbi('WRAP', MinMax(0, 24), 0.01, (0,), False)
kif_weight_default = _kif('SAT_SYM', float('inf'), (), True)
kif_datalane_default = _kif('WRAP', 0.01, (0,), False)

kbi_table_default = dict(kbi_weight_default, homogeneous_axis=None, heterogeneous_axis=(), is_weight=False)
kif_table_default = dict(kif_weight_default, homogeneous_axis=None, heterogeneous_axis=(), is_weight=False)
kbi_bias_default = dict(kbi_datalane_default, homogeneous_axis=())
kif_bias_default = dict(kif_datalane_default, homogeneous_axis=())

default_configs: dict[tuple[str, str], dict] = {
    ('kbi', 'weight'): kbi_weight_default,
    ('kbi', 'bias'): kbi_bias_default,
    ('kbi', 'table'): kbi_table_default,
    ('kbi', 'datalane'): kbi_datalane_default,
    ('kif', 'weight'): kif_weight_default,
    ('kif', 'bias'): kif_bias_default,
    ('kif', 'table'): kif_table_default,
    ('kif', 'datalane'): kif_datalane_default,
}

all_quantizer_keys = {k for v in default_configs.values() for k in v.keys()} | {
    'q_type',
    'place',
    'scaler',
    'affine',
    'qnoise_factor',
}


def all_quantizer_types():
    return {k[0] for k in default_configs.keys()}


def all_places():
    return {k[1] for k in default_configs.keys()}


def _exclusive_axes(kwargs: dict) -> None:
    assert kwargs.get('homogeneous_axis') is None or kwargs.get('heterogeneous_axis') is None, (
        'homogeneous_axis and heterogeneous_axis are mutually exclusive. Set only one of them.'
    )
    if kwargs.get('homogeneous_axis') is not None:
        kwargs['heterogeneous_axis'] = None
    if kwargs.get('heterogeneous_axis') is not None:
        kwargs['homogeneous_axis'] = None


class QuantizerConfig(Mapping):
    """Everything needed to instantiate one quantizer: its type, where it sits, and the internal quantizer's
    constructor arguments (taken from the defaults of (q_type, place) unless overridden).

    ``q_type``: 'kbi', 'kif', 'dummy' or 'default' (resolved through ``default_q_type[place]``);
    ``place``: 'weight', 'datalane', 'bias' or 'table'; ``scaler``: divide before / multiply after;
    ``affine``: (scale, shift) applied after quantization; ``qnoise_factor``: blend factor in training.
    """

    def __init__(self, q_type: str = 'default', place: str = 'datalane', scaler=None, affine=None, qnoise_factor=None,
                 **kwargs) -> None:
        place = place.lower()
        q_type = q_type.lower()
        if q_type == 'default':
            q_type = default_q_type[place]
        if q_type == 'float':
            raise NotImplementedError("the minifloat quantizer ('float') is outside the accelerated path")
        if q_type != 'dummy':
            assert (q_type, place) in default_configs, f'Default config for ({q_type}, {place}) not found.'
        self.place = place
        self.q_type = q_type
        self.scaler = None
        self.qnoise_factor = None
        self.affine = None
        if scaler is not None:
            assert scaler != 0, 'scaler must not be 0.'
            self.scaler = float(scaler)
        if affine is not None:
            assert len(affine) == 2, 'affine must be a tuple of (scale, shift).'
            assert affine[0] != 0, 'affine scale must not be 0.'
            self.affine = (float(affine[0]), float(affine[1]))
        if qnoise_factor is not None:
            assert 0 <= qnoise_factor <= 1, 'qnoise_factor must be between 0 and 1.'
            self.qnoise_factor = float(qnoise_factor)
        if q_type == 'dummy':
            self.config = {}
            return
        _exclusive_axes(kwargs)
        self.config = default_configs[(q_type, place)].copy()
        for k, v in kwargs.items():
            if k not in self.config:
                raise ValueError(f'{k} is not a valid parameter for {q_type} quantizer config.')
            self.config[k] = v

    def __getitem__(self, key):
        return self.config[key]

    def __iter__(self):
        return iter(self.config)

    def __len__(self) -> int:
        return len(self.config)

    def __bool__(self):
        return True

    def get_config(self):
        return {
            'q_type': self.q_type,
            'place': self.place,
            'scaler': self.scaler,
            'qnoise_factor': self.qnoise_factor,
            'affine': self.affine,
            **self.config,
        }

    @classmethod
    def from_config(cls, config):
        return cls(**config)

    def get_quantizer(self) -> TrainableQuantizerBase:
        if self.q_type == 'kif':
            return FixedPointQuantizerKIF(**self)
        if self.q_type == 'kbi':
            return FixedPointQuantizerKBI(**self)
        if self.q_type == 'dummy':
            return DummyQuantizer()
        raise ValueError(f'Unknown quantizer type: {self.q_type}')


class QuantizerConfigScope:
    """Overrides default quantizer configs for the selected (q_type, place) pairs inside a ``with`` block.

    ``default_q_type`` additionally changes which quantizer type 'default' resolves to for the selected
    places.  If exactly two of ``i0``, ``f0``, ``b0`` are given the third is derived (b = i + f).
    """

    def __init__(self, q_type: str | Sequence[str] | set[str] = 'all', place: str | Sequence[str] | set[str] = 'all',
                 default_q_type=None, **kwargs):
        if q_type == 'all':
            q_type = all_quantizer_types()
        if place == 'all':
            place = all_places()
        q_type = (q_type,) if isinstance(q_type, str) else q_type
        place = (place,) if isinstance(place, str) else place
        q_type = {t.lower() for t in q_type}
        place = {p.lower() for p in place}
        for t in q_type:
            for p in place:
                assert (t, p) in default_configs, f'Default config for ({t}, {p}) not found.'
        _exclusive_axes(kwargs)
        i, f, b = kwargs.get('i0'), kwargs.get('f0'), kwargs.get('b0')
        if sum((i is not None, f is not None, b is not None)) == 2:
            if i is None:
                kwargs['i0'] = b - f
            if f is None:
                kwargs['f0'] = b - i
            if b is None:
                kwargs['b0'] = i + f
        for k in kwargs:
            if k not in all_quantizer_keys:
                raise ValueError(f'{k} is not a valid parameter for any known quantizer configs.')
        self.q_types = q_type
        self.places = place
        self.kwargs = kwargs
        self.default_q_type = default_q_type
        self._tmp_storage = {}
        self.original_default_q_type = None

    def __enter__(self):
        for (q_type, place), conf in default_configs.items():
            if q_type in self.q_types and place in self.places:
                self._tmp_storage[(q_type, place)] = conf.copy()
                for k, v in self.kwargs.items():
                    if k in conf:
                        conf[k] = v
        if self.default_q_type is not None:
            self.original_default_q_type = default_q_type.copy()
            for place in self.places:
                default_q_type[place] = self.default_q_type

    def __exit__(self, exc_type, exc_value, traceback):
        if self.original_default_q_type is not None:
            default_q_type.clear()
            default_q_type.update(self.original_default_q_type)
            self.original_default_q_type = None
        for key, saved in self._tmp_storage.items():
            default_configs[key].update(saved)
        self._tmp_storage.clear()

    def override(self):
        """Apply the overrides permanently."""
        self.__enter__()
        self._tmp_storage.clear()


class HardTanhConfig(QuantizerConfig):
    """A kif quantizer pinned to k=1, i=0 with saturation: a hard tanh."""

    def __init__(self, q_type: str = 'kif', place: str = 'datalane', symmetric: bool = False, **kwargs) -> None:
        assert not any(k in kwargs for k in ('k0', 'ic', 'affine', 'overflow_node')), (
            'k0, ic, affine, overflow_mode must not be set for HardTanhConfig.'
        )
        kwargs.pop('i0', None)
        super().__init__(q_type=q_type, place=place, k0=1, ic=Constant(0), i0=0,
                         overflow_mode='SAT_SYM' if symmetric else 'SAT', affine=None, **kwargs)


class HardSigmoidConfig(QuantizerConfig):
    """A kif quantizer pinned to k=1, i=1, SAT, followed by the affine map 0.25 x + 0.5: a hard sigmoid."""

    def __init__(self, q_type: str = 'kif', place: str = 'datalane', **kwargs) -> None:
        assert not any(k in kwargs for k in ('k0', 'ic', 'affine', 'overflow_mode')), (
            'k0, ic, affine, overflow_mode must not be set for HardSigmoidConfig.'
        )
        kwargs.pop('i0', None)
        super().__init__(q_type=q_type, place=place, k0=1, ic=Constant(1), i0=1, overflow_mode='SAT', affine=(0.25, 0.5),
                         **kwargs)
