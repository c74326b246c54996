"""ctypes binding of libhgq_b200.so, the C-ABI CUDA library of this package.

The library is the only compute path of the package: there is no CPU or eager-PyTorch fallback.
Loading fails loudly when the shared object is missing, and every call raises ``HGQError`` on a
non-zero status.  PyTorch is used for device memory and streams only; the functions here take
``torch.Tensor`` arguments and pass their raw device pointers across the ABI declared in
``include/hgq_b200.h``.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_uint, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / 'lib' / 'libhgq_b200.so'

ROUND_MODES = {'TRN': 0, 'RND': 1, 'RND_CONV': 2}
OVERFLOW_MODES = {'NONE': 0, 'WRAP': 1, 'SAT': 2, 'SAT_SYM': 3}
FLAG_TRAINING = 1
FLAG_ZERO_NONPOS = 2
FLAG_ABSMAX_ACCUMULATE = 4


class HGQError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().hgq_status_string(status).decode() if _lib is not None else '?'
        super().__init__(f'{where} failed with status {status}: {msg}')


# name -> (restype, argtypes).  Every symbol declared in include/hgq_b200.h is listed here; the
# CPU test-suite checks the two against each other.
SIGNATURES: dict[str, tuple] = {
    'hgq_status_string': (c_char_p, [c_int]),
    'hgq_abi_version': (c_int, []),
    'hgq_launch_count': (c_int64, []),
    'hgq_quantize_fwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_uint, c_void_p],
    ),
    'hgq_quantize_bwd_workspace': (c_size_t, [c_int64, c_int64]),
    'hgq_quantize_bwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
         c_uint, c_void_p, c_size_t, c_void_p],
    ),
    'hgq_quantize_bwd_noalloc': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
         c_uint, c_void_p],
    ),
    'hgq_qdense_fwd_workspace': (c_size_t, [c_int64, c_int, c_int, c_int]),
    'hgq_qdense_fwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_uint, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
         c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_qdense_fwd_pooled_supported': (c_int, [c_int64, c_int, c_int, c_int, c_int, c_int]),
    'hgq_qdense_fwd_pooled': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_uint, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
         c_void_p, c_int, c_float, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_qdense_bwd_workspace': (c_size_t, [c_int64, c_int, c_int, c_int]),
    'hgq_qdense_bwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
         c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_qdense_bwd_strided': (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
         c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_qdense_bwd_accumulate_supported': (c_int, [c_int, c_int, c_int, c_int, c_int]),
    'hgq_qdense_bwd_accumulate': (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_void_p,
         c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_qsoftmax_fwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p,
         c_int64, c_int, c_int, c_void_p],
    ),
    'hgq_qsoftmax_bwd_workspace': (c_size_t, [c_int64, c_int, c_int]),
    'hgq_qsoftmax_bwd': (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p,
         c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p],
    ),
    'hgq_qconv2d_supported': (c_int, [c_int64] + [c_int] * 8),
    'hgq_qconv2d_unit_stride_supported': (c_int, [c_int64] + [c_int] * 10),
    'hgq_qconv2d_fwd': (
        c_int,
        [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p] + [c_int] * 11 + [c_void_p, c_void_p],
    ),
    'hgq_qconv2d_wgrad_workspace': (c_size_t, [c_int64] + [c_int] * 8),
    'hgq_qconv2d_wgrad': (
        c_int,
        [c_void_p] * 6 + [c_int64] + [c_int] * 14 + [c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    'hgq_maxpool2d_fwd': (c_int, [c_void_p, c_void_p, c_void_p, c_int64] + [c_int] * 9 + [c_void_p]),
    'hgq_maxpool2d_bwd': (c_int, [c_void_p, c_void_p, c_void_p, c_int64] + [c_int] * 9 + [c_void_p]),
    'hgq_attn_heads_supported': (c_int, [c_int64, c_int, c_int, c_int]),
    'hgq_attn_heads_matmul': (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    'hgq_track_kif': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    'hgq_track_kbi': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_int64, c_void_p]),
    'hgq_softmax_xent_workspace': (c_size_t, [c_int64]),
    'hgq_softmax_xent': (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    'hgq_ebops_dense': (
        c_int,
        [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_double, c_double, c_void_p] + [c_void_p] * 7,
    ),
    'hgq_ebops_dense_batch': (c_int, [c_void_p, c_int, c_void_p]),
    'hgq_ebops_conv2d': (
        c_int,
        [c_void_p, c_int, c_int, c_int, c_void_p] + [c_int] * 11 + [c_void_p, c_int64, c_double, c_double, c_double, c_void_p]
        + [c_void_p] * 7,
    ),
    'hgq_adam_step': (c_int, [c_void_p] * 7 + [c_int64] + [c_float] * 5 + [c_void_p, c_void_p]),
    'hgq_peer_exchange_bytes': (c_size_t, [c_int64]),
    'hgq_peer_buffer_create': (c_int, [c_size_t, c_void_p, c_void_p]),
    'hgq_peer_buffer_open': (c_int, [c_void_p, c_void_p]),
    'hgq_peer_buffer_close': (c_int, [c_void_p]),
    'hgq_peer_buffer_destroy': (c_int, [c_void_p]),
    'hgq_adam_step_peers': (c_int, [c_void_p] * 7 + [c_int64] + [c_float] * 4 + [c_void_p, c_void_p, c_int, c_int, c_uint, c_void_p, c_void_p]),
    'hgq_dense_chain_supported': (c_int, [c_int, c_void_p]),
    'hgq_dense_chain_workspace': (c_size_t, [c_int64, c_int, c_void_p]),
    'hgq_dense_chain_fwd': (c_int, [c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    'hgq_dense_chain_bwd': (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    'hgq_tables_forward': (c_int, [c_void_p, c_int, c_int64, c_void_p]),
    'hgq_tables_track_bits': (c_int, [c_void_p, c_int, c_int64, c_void_p]),
    'hgq_tables_backward': (c_int, [c_void_p, c_int, c_int64, c_void_p]),
    'hgq_weights_forward': (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    'hgq_weights_backward': (c_int, [c_void_p, c_int, c_int64, c_void_p, c_void_p]),
    'hgq_quantize_host_workspace': (c_size_t, [c_int64]),
    'hgq_quantize_fwd_bwd_host': (
        c_int,
        [c_void_p] * 9 + [c_int64, c_int, c_int, c_uint, c_void_p, c_size_t, c_int64],
    ),
}



class SlotDesc(ctypes.Structure):
    """hgq_slot_desc of include/hgq_b200.h."""

    _fields_ = [('a_raw', c_void_p), ('i_raw', c_void_p), ('k', c_void_p), ('I', c_void_p), ('F', c_void_p), ('BITS', c_void_p),
                ('dI', c_void_p), ('dF', c_void_p), ('dBITS', c_void_p), ('g_a', c_void_p), ('g_i', c_void_p),
                ('absmax', c_void_p), ('decay', c_void_p), ('n', c_int64), ('kind', ctypes.c_int32), ('om', ctypes.c_int32),
                ('rm', ctypes.c_int32), ('symmetric', ctypes.c_int32), ('tracked_weight', ctypes.c_int32), ('i_lo', c_float),
                ('i_hi', c_float)]


class EbopsDenseDesc(ctypes.Structure):
    """hgq_ebops_dense_desc of include/hgq_b200.h."""

    _fields_ = [('bw_in', c_void_p), ('P', c_int64), ('K', c_int64), ('bw_w', c_void_p), ('N', c_int64), ('bw_bias', c_void_p),
                ('n_bias', c_int64), ('out_size', ctypes.c_double), ('scale', ctypes.c_double), ('beta', c_void_p),
                ('ebops', c_void_p), ('ebops_f', c_void_p), ('loss', c_void_p), ('d_bw_in', c_void_p), ('d_bw_w', c_void_p),
                ('d_bw_bias', c_void_p)]


class ChainLayer(ctypes.Structure):
    """hgq_chain_layer of include/hgq_b200.h."""

    _fields_ = [('K', ctypes.c_int32), ('N', ctypes.c_int32), ('relu', ctypes.c_int32), ('round_mode', ctypes.c_int32),
                ('qf', c_void_p), ('wq', c_void_p), ('bq', c_void_p), ('y', c_void_p), ('absmax', c_void_p), ('dwq', c_void_p),
                ('dbq', c_void_p), ('df', c_void_p)]


class WeightDesc(ctypes.Structure):
    """hgq_weight_desc of include/hgq_b200.h."""

    _fields_ = [('w_raw', c_void_p), ('wq', c_void_p), ('dwq', c_void_p), ('g_w', c_void_p), ('n', c_int64),
                ('slot', ctypes.c_int32), ('mode', ctypes.c_int32)]


_lib = None  # the loaded library behind a call-counting proxy (hgq2_b200.routes)


def lib():
    """The loaded library.  Raises if it has not been built (``python -m hgq2_b200.build``)."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get('HGQ_B200_LIB', LIB_PATH))
        if not path.exists():
            raise ImportError(
                f'{path} is missing: build it with `python -m hgq2_b200.build` (needs nvcc). '
                'hgq2_b200 has no CPU fallback.'
            )
        handle = ctypes.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        from .routes import CountingLibrary

        _lib = CountingLibrary(handle)
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise HGQError(status, where)


def ptr(t) -> int | None:
    """Device pointer of a tensor (None passes NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_handle() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                'hgq2_b200 runs on CUDA tensors only (sm_100a kernels); got a tensor on ' + str(t.device)
            )
