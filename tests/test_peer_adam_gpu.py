"""The fused gradient-exchange + Adam kernel (``hgq_adam_step_peers``) on ONE GPU: the second rank is emulated by a buffer
whose slot and flags the test writes itself, so no kernel ever waits for another kernel.  The two-GPU run is in
test_dp_gpu.py."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CHUNK = 2048  # floats per CTA of the kernel (the layout of an exchange buffer is part of the C ABI's contract)


class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {'shape': (nbytes,), 'typestr': '|u1', 'data': (ptr, False), 'version': 2}


def _buffer(L, n):
    nbytes = L.hgq_peer_exchange_bytes(n)
    ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
    assert L.hgq_peer_buffer_create(nbytes, ctypes.byref(ptr), handle) == 0
    view = torch.as_tensor(_Raw(ptr.value, nbytes), device='cuda')
    return ptr, view


def _state(n, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    w = torch.randn(n, device='cuda', generator=g)
    m = torch.randn(n, device='cuda', generator=g) * 0.1
    v = torch.rand(n, device='cuda', generator=g) * 0.01
    lo = torch.full((n,), -1.5, device='cuda')
    hi = torch.full((n,), 1.5, device='cuda')
    l1 = torch.full((n,), 1e-4, device='cuda')
    return w, m, v, lo, hi, l1


@pytest.mark.parametrize('n', [5003, 2048, 7])
def test_sum_over_two_ranks_and_update(n):
    from hgq2_b200 import _lib, kernels

    L = _lib.lib()
    torch.cuda.set_device(0)
    dev = torch.device('cuda', 0)
    n_pad = (n + CHUNK - 1) // CHUNK * CHUNK
    chunks = n_pad // CHUNK
    own, _ = _buffer(L, n)
    peer, peer_view = _buffer(L, n)
    gen = torch.Generator(device='cuda').manual_seed(1)
    g0 = torch.randn(n, device='cuda', generator=gen)
    g1 = torch.randn(n, device='cuda', generator=gen)
    w, m, v, lo, hi, l1 = _state(n, 2)
    w_ref, m_ref, v_ref = w.clone(), m.clone(), v.clone()
    step = torch.zeros((), dtype=torch.int64, device='cuda')
    step_ref = step.clone()
    ptrs = (ctypes.c_void_p * 2)(own.value, peer.value)
    status = kernels.status_word(dev)
    status.zero_()
    for t in (1, 2, 3):  # three steps: both slots, and a slot used for the second time
        slot = t & 1
        # the emulated rank 1 publishes its gradients of step t: data of the slot, then the flags
        data = peer_view[: 2 * n_pad * 4].view(torch.float32)
        data[slot * n_pad: slot * n_pad + n] = g1 * t
        flags = peer_view[2 * n_pad * 4:].view(torch.int64)
        flags[slot * chunks:(slot + 1) * chunks] = t
        torch.cuda.synchronize()
        st = L.hgq_adam_step_peers(w.data_ptr(), (g0 * t).data_ptr(), m.data_ptr(), v.data_ptr(), lo.data_ptr(), hi.data_ptr(),
                                   l1.data_ptr(), n, 1e-3, 0.9, 0.999, 1e-7, step.data_ptr(), ptrs, 2, 0, 1000, status.data_ptr(),
                                   None)
        assert st == 0
        gsum = (0.0 + g0 * t) + g1 * t  # the kernel adds rank 0, then rank 1, then scales by 1 / world
        st = L.hgq_adam_step(w_ref.data_ptr(), gsum.data_ptr(), m_ref.data_ptr(), v_ref.data_ptr(), lo.data_ptr(), hi.data_ptr(),
                             l1.data_ptr(), n, 1e-3, 0.9, 0.999, 1e-7, 0.5, step_ref.data_ptr(), None)
        assert st == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert int(step.item()) == t
        for a, b, name in ((w, w_ref, 'w'), (m, m_ref, 'm'), (v, v_ref, 'v')):
            assert torch.equal(a, b), (name, t, float((a - b).abs().max()))
    assert L.hgq_peer_buffer_destroy(own) == 0 and L.hgq_peer_buffer_destroy(peer) == 0


def test_a_wait_that_runs_out_sets_the_status_word_and_leaves_the_parameters():
    """The emulated peer never publishes: the bounded wait gives up after max_polls polls, bit 1 of the status word is set,
    the parameters and moments stay as they were, and the context stays usable."""
    from hgq2_b200 import _lib, kernels

    L = _lib.lib()
    torch.cuda.set_device(0)
    dev = torch.device('cuda', 0)
    n = 3000
    own, _ = _buffer(L, n)
    peer, _ = _buffer(L, n)
    g0 = torch.randn(n, device='cuda')
    w, m, v, lo, hi, l1 = _state(n, 3)
    before = [t.clone() for t in (w, m, v)]
    step = torch.zeros((), dtype=torch.int64, device='cuda')
    ptrs = (ctypes.c_void_p * 2)(own.value, peer.value)
    status = kernels.status_word(dev)
    status.zero_()
    st = L.hgq_adam_step_peers(w.data_ptr(), g0.data_ptr(), m.data_ptr(), v.data_ptr(), lo.data_ptr(), hi.data_ptr(), l1.data_ptr(),
                               n, 1e-3, 0.9, 0.999, 1e-7, step.data_ptr(), ptrs, 2, 0, 200, status.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    assert int(status.item()) & 2
    for a, b in zip((w, m, v), before):
        assert torch.equal(a, b)
    status.zero_()
    assert float((w + 1).sum()) == float((before[0] + 1).sum())  # the device still answers
    assert L.hgq_peer_buffer_destroy(own) == 0 and L.hgq_peer_buffer_destroy(peer) == 0


def test_argument_errors():
    from hgq2_b200 import _lib

    L = _lib.lib()
    assert L.hgq_peer_exchange_bytes(0) == 0
    assert L.hgq_peer_exchange_bytes(1) == 2 * CHUNK * 4 + 2 * 8
    assert L.hgq_peer_buffer_create(0, None, None) == -1
    assert L.hgq_adam_step_peers(None, None, None, None, None, None, None, 16, 1e-3, 0.9, 0.999, 1e-7, None, None, 2, 0, 10, None,
                                 None) == -1


def test_a_handle_that_cannot_be_opened_is_an_error_code_not_a_sticky_failure():
    """A rank that cannot map a peer's buffer (here: a handle of zeros) gets an error code -- the trainer then keeps the NCCL
    route -- and the next kernel launch check of the library is clean."""
    from hgq2_b200 import _lib, kernels

    L = _lib.lib()
    torch.cuda.set_device(0)
    bogus = (ctypes.c_ubyte * 64)()
    p = ctypes.c_void_p()
    assert L.hgq_peer_buffer_open(bogus, ctypes.byref(p)) != 0
    x = torch.randn(1024, device='cuda')
    f = torch.full((1024,), 4.0, device='cuda')
    y = kernels.quantize_fwd(x, None, None, f, 'RND', 'NONE', training=True)
    y = y[0] if isinstance(y, tuple) else y
    assert torch.equal(y, torch.floor(x * 16 + 0.5) / 16)
