"""Tensor-level entry to the CUDA kernels: allocates outputs with torch, calls the C ABI.

These functions are the seam between the Python mirror of the reference interface and
``libhgq_b200.so``.  They do no arithmetic themselves.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import FLAG_ABSMAX_ACCUMULATE, FLAG_TRAINING, FLAG_ZERO_NONPOS, OVERFLOW_MODES, ROUND_MODES, check, lib, ptr, require_cuda, stream_handle

_workspaces: dict[tuple[int, int, int], torch.Tensor] = {}


def workspace(nbytes: int, device: torch.device, slot: int = 0) -> torch.Tensor | None:
    """A scratch buffer that only ever grows (kept so steady-state steps allocate nothing), one per device, purpose
    (``slot``) and stream: kernels queued on different streams may run at the same time and must not share scratch."""
    if nbytes <= 0:
        return None
    if torch.cuda.is_current_stream_capturing():
        # Inside a graph capture the scratch is a temporary of the graph's own memory pool, like any other tensor of the
        # captured step.  A cached buffer must not be used here: one that an earlier capture allocated belongs to that
        # graph's pool, and once it is replaced (a later call needs a larger one) and that graph is gone, the pool hands
        # its memory back to the driver while this graph's kernels still hold the address.
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    dev = device.index if device.index is not None else torch.cuda.current_device()
    key = (dev, slot, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _modes(round_mode: str, overflow_mode: str) -> tuple[int, int]:
    try:
        return ROUND_MODES[round_mode.upper()], OVERFLOW_MODES[overflow_mode.upper()]
    except KeyError as e:
        raise ValueError(f'unsupported mode {e}; round modes {list(ROUND_MODES)}, overflow modes {list(OVERFLOW_MODES)}')


def _period(x: torch.Tensor, p: torch.Tensor) -> int:
    n, m = x.numel(), p.numel()
    if m == n:
        return n
    if m == 0 or n % m != 0:
        raise ValueError(f'parameter tensor with {m} entries cannot be broadcast over {n} elements')
    return m


def quantize_fwd(
    x: torch.Tensor,
    k: torch.Tensor | None,
    i: torch.Tensor | None,
    f: torch.Tensor,
    round_mode: str,
    overflow_mode: str,
    training: bool = False,
    zero_nonpos: bool = False,
    want_absmax: bool = False,
    out: torch.Tensor | None = None,
    absmax_out: torch.Tensor | None = None,
):
    """y = overflow(round(x, f), k, i, f); optionally also max_rows |round(x, f)| per parameter entry (into ``absmax_out``
    when given).

    ``k`` is uint8, ``i``/``f`` fp32 with integer values.  Parameters either match ``x`` element
    for element or hold ``period`` entries that repeat along the leading axes of ``x``.
    """
    require_cuda(x, k, i, f)
    rm, om = _modes(round_mode, overflow_mode)
    assert x.dtype == torch.float32 and f.dtype == torch.float32
    x = x.contiguous()
    f = f.contiguous()
    k = k.contiguous() if k is not None else None
    i = i.contiguous() if i is not None else None
    if k is not None:
        assert k.dtype == torch.uint8
    period = _period(x, f)
    y = out if out is not None else torch.empty_like(x)
    absmax = (absmax_out if absmax_out is not None else torch.empty(period, dtype=torch.float32, device=x.device)) if want_absmax else None
    flags = (FLAG_TRAINING if training else 0) | (FLAG_ZERO_NONPOS if zero_nonpos else 0)
    with torch.cuda.device(x.device):
        st = lib().hgq_quantize_fwd(
            ptr(x), ptr(k), ptr(i), ptr(f), ptr(y), ptr(absmax), x.numel(), period, rm, om, flags, stream_handle()
        )
    check(st, 'hgq_quantize_fwd')
    return (y, absmax) if want_absmax else y


def quantize_bwd(
    g: torch.Tensor,
    x: torch.Tensor,
    k: torch.Tensor | None,
    i: torch.Tensor | None,
    f: torch.Tensor,
    round_mode: str,
    overflow_mode: str,
    want_dx: bool = True,
    want_di: bool = True,
    out_df: torch.Tensor | None = None,
    out_di: torch.Tensor | None = None,
):
    """Surrogate gradients (dx, di, df) of the training-mode quantizer; di/df are reduced to the parameter shape (and
    written to ``out_di`` / ``out_df`` when given)."""
    require_cuda(g, x, k, i, f)
    rm, om = _modes(round_mode, overflow_mode)
    g = g.contiguous()
    x = x.contiguous()
    f = f.contiguous()
    k = k.contiguous() if k is not None else None
    i = i.contiguous() if i is not None else None
    n = x.numel()
    period = _period(x, f)
    dx = torch.empty_like(x) if (want_dx or period == n) else None
    di = (out_di if out_di is not None else torch.empty(period, dtype=torch.float32, device=x.device)) if want_di else None
    df = out_df if out_df is not None else torch.empty(period, dtype=torch.float32, device=x.device)
    nbytes = lib().hgq_quantize_bwd_workspace(n, period)
    ws = workspace(nbytes, x.device)
    with torch.cuda.device(x.device):
        st = lib().hgq_quantize_bwd(
            ptr(g), ptr(x), ptr(k), ptr(i), ptr(f), ptr(dx), ptr(di), ptr(df), n, period, rm, om, 0,
            ptr(ws), ws.numel() if ws is not None else 0, stream_handle(),
        )
    check(st, 'hgq_quantize_bwd')
    if period == n:
        di = di.view(f.shape) if di is not None else None
        df = df.view(f.shape)
    else:
        di = di.view(f.shape) if di is not None else None
        df = df.view(f.shape)
    return dx, di, df


def launch_count() -> int:
    return int(lib().hgq_launch_count())




def quantize_fwd_bwd_host(hx, hk, hi, hf, hg, hy, hdx, hdi, hdf, round_mode: str, overflow_mode: str,
                          training: bool, dev_ws: torch.Tensor, chunk_elems: int) -> None:
    """Host-buffer sweep: CPU tensors in (ideally pinned), CPU tensors out; see hgq_quantize_fwd_bwd_host."""
    rm, om = _modes(round_mode, overflow_mode)
    for t in (hx, hk, hi, hf, hg, hy, hdx, hdi, hdf):
        if t is not None and (t.is_cuda or not t.is_contiguous()):
            raise ValueError('host entry takes contiguous CPU tensors')
    require_cuda(dev_ws)
    with torch.cuda.device(dev_ws.device):
        st = lib().hgq_quantize_fwd_bwd_host(
            ptr(hx), ptr(hk), ptr(hi), ptr(hf), ptr(hg), ptr(hy), ptr(hdx), ptr(hdi), ptr(hdf), hx.numel(), rm, om,
            FLAG_TRAINING if training else 0, ptr(dev_ws), dev_ws.numel() * dev_ws.element_size(), chunk_elems,
        )
    check(st, 'hgq_quantize_fwd_bwd_host')


def quantize_host_workspace(chunk_elems: int) -> int:
    return int(lib().hgq_quantize_host_workspace(chunk_elems))


def ebops_dense(bw_in, bw_w, bw_bias, out_size: float, scale: float, beta, want_grads: bool = True, out=None):
    """K3 for a dense / einsum-dense layer.  bw_in [P, K], bw_w [K, N]; returns (ebops_u32, ebops_f, loss, d_in, d_w, d_bias).
    ``out``: caller-owned (ebops_u32, loss, d_in, d_w, d_bias) destinations instead of fresh tensors."""
    require_cuda(bw_in, bw_w, bw_bias, beta)
    bw_in, bw_w = bw_in.contiguous(), bw_w.contiguous()
    P, K = bw_in.shape
    K2, N = bw_w.shape
    assert K == K2
    dev = bw_in.device
    nb = 0 if bw_bias is None else bw_bias.numel()
    bw_bias = None if bw_bias is None else bw_bias.contiguous()
    if out is not None:
        e_u, loss, d_in, d_w, d_b = out
        e_f = None
    else:
        e_u = torch.empty((), dtype=torch.uint32, device=dev)
        e_f = torch.empty((), dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        d_in = torch.empty_like(bw_in) if want_grads else None
        d_w = torch.empty_like(bw_w) if want_grads else None
        d_b = torch.empty_like(bw_bias) if (want_grads and nb) else None
    with torch.cuda.device(dev):
        st = lib().hgq_ebops_dense(ptr(bw_in), P, K, ptr(bw_w), N, ptr(bw_bias), nb, float(out_size), float(scale), ptr(beta),
                                   ptr(e_u), ptr(e_f), ptr(loss), ptr(d_in), ptr(d_w), ptr(d_b), stream_handle())
    check(st, 'hgq_ebops_dense')
    return e_u, e_f, loss, d_in, d_w, d_b


EBOPS_BATCH_MAX = 16


def ebops_dense_batch(items) -> None:
    """K3 for several dense layers in one launch per 16 layers.  ``items``: tuples (bw_in [P, K], bw_w [K, N], bw_bias or None,
    out_size, scale, beta, out) with ``out`` = (ebops_u32, loss, d_in, d_w, d_bias) destinations as for ``ebops_dense``."""
    for start in range(0, len(items), EBOPS_BATCH_MAX):
        chunk = items[start:start + EBOPS_BATCH_MAX]
        arr = (_lib.EbopsDenseDesc * len(chunk))()
        keep = []
        for a, (bw_in, bw_w, bw_bias, out_size, scale, beta, out) in zip(arr, chunk):
            require_cuda(bw_in, bw_w, bw_bias, beta)
            bw_in, bw_w = bw_in.contiguous(), bw_w.contiguous()
            bw_bias = None if bw_bias is None else bw_bias.contiguous()
            keep.append((bw_in, bw_w, bw_bias))
            e_u, loss, d_in, d_w, d_b = out
            a.bw_in, (a.P, a.K), a.bw_w, a.N = bw_in.data_ptr(), bw_in.shape, bw_w.data_ptr(), bw_w.shape[1]
            a.bw_bias, a.n_bias = (None, 0) if bw_bias is None else (bw_bias.data_ptr(), bw_bias.numel())
            a.out_size, a.scale, a.beta = float(out_size), float(scale), beta.data_ptr()
            for name, t in (('ebops', e_u), ('ebops_f', None), ('loss', loss), ('d_bw_in', d_in), ('d_bw_w', d_w), ('d_bw_bias', d_b)):
                setattr(a, name, None if t is None else t.data_ptr())
        with torch.cuda.device(chunk[0][0].device):
            check(lib().hgq_ebops_dense_batch(arr, len(chunk), stream_handle()), 'hgq_ebops_dense_batch')


def ebops_conv2d(bw_in, bw_w, bw_bias, out_hw, strides, dilation, pad_tl, out_size: float, scale_main: float,
                 scale_bias: float, beta, want_grads: bool = True, out=None):
    """K3 for a channels-last conv2d.  bw_in [H, W, C], bw_w [KH, KW, C, N]."""
    require_cuda(bw_in, bw_w, bw_bias, beta)
    bw_in, bw_w = bw_in.contiguous(), bw_w.contiguous()
    H, W, C = bw_in.shape
    KH, KW, C2, N = bw_w.shape
    assert C == C2
    dev = bw_in.device
    nb = 0 if bw_bias is None else bw_bias.numel()
    bw_bias = None if bw_bias is None else bw_bias.contiguous()
    if out is not None:
        e_u, loss, d_in, d_w, d_b = out
        e_f = None
    else:
        e_u = torch.empty((), dtype=torch.uint32, device=dev)
        e_f = torch.empty((), dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        d_in = torch.empty_like(bw_in) if want_grads else None
        d_w = torch.empty_like(bw_w) if want_grads else None
        d_b = torch.empty_like(bw_bias) if (want_grads and nb) else None
    with torch.cuda.device(dev):
        st = lib().hgq_ebops_conv2d(ptr(bw_in), H, W, C, ptr(bw_w), KH, KW, N, out_hw[0], out_hw[1], strides[0], strides[1],
                                    dilation[0], dilation[1], pad_tl[0], pad_tl[1], ptr(bw_bias), nb, float(out_size),
                                    float(scale_main), float(scale_bias), ptr(beta), ptr(e_u), ptr(e_f), ptr(loss),
                                    ptr(d_in), ptr(d_w), ptr(d_b), stream_handle())
    check(st, 'hgq_ebops_conv2d')
    return e_u, e_f, loss, d_in, d_w, d_b


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device status word the tensor-core kernels set when a bounded device-side wait gives up."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def check_status(device: torch.device) -> None:
    """Synchronising check of the status word (tests and debugging; the hot path does not call it)."""
    v = int(status_word(device).item())
    if v != 0:
        raise _lib.HGQError(-7, f'device status word = {v}')


def qdense_supported(M: int, K: int, N: int, rows_period: int) -> bool:
    return M > 0 and lib().hgq_qdense_fwd_workspace(M, K, N, rows_period) > 0


def qdense_fwd(x, qk, qi, qf, rows_period: int, round_mode: str, overflow_mode: str, training: bool, zero_nonpos: bool,
               wq, bq, activation: str | None, want_absmax: bool, absmax_out=None, absmax_accumulate: bool = False,
               pool_rows: int = 0, pool_scale: float = 1.0):
    """Fused y = act(iq(x) @ wq + bq); x is treated as [M, K] with K = wq.shape[0].  Returns (y [M, N], absmax or None).
    With ``absmax_accumulate`` the statistic is merged into ``absmax_out`` by atomic max (the caller zeroed it).
    With ``pool_rows`` > 0 a third value is returned: ``pool_scale`` times the sum of y over every group of ``pool_rows``
    consecutive rows, [M / pool_rows, N] (shapes for which ``qdense_pooled_supported`` is true)."""
    require_cuda(x, qk, qi, qf, wq, bq)
    rm, om = _modes(round_mode, overflow_mode)
    x = x.contiguous()
    qk, qi, qf = (None if t is None else t.contiguous() for t in (qk, qi, qf))
    bq = None if bq is None else bq.contiguous()
    N = wq.shape[-1]
    K = wq.shape[0]
    M = x.numel() // K
    wq = wq.contiguous()
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    absmax = (absmax_out if absmax_out is not None else torch.empty(rows_period * K, dtype=torch.float32, device=x.device)) if want_absmax else None
    accumulate = want_absmax and absmax_accumulate and absmax_out is not None
    ws = workspace(lib().hgq_qdense_fwd_workspace(M, K, N, rows_period), x.device, slot=1) if (want_absmax and not accumulate) else None
    act = {None: 0, 'relu': 1}[activation]
    flags = (FLAG_TRAINING if training else 0) | (FLAG_ZERO_NONPOS if zero_nonpos else 0) | (FLAG_ABSMAX_ACCUMULATE if accumulate else 0)
    pooled = torch.empty((M // pool_rows, N), dtype=torch.float32, device=x.device) if pool_rows else None
    with torch.cuda.device(x.device):
        if pool_rows:
            st = lib().hgq_qdense_fwd_pooled(
                ptr(x), ptr(qk), ptr(qi), ptr(qf), rows_period, rm, om, flags, ptr(wq), ptr(bq), act, ptr(y), ptr(absmax),
                ptr(pooled), pool_rows, float(pool_scale), M, K, N, ptr(ws), ws.numel() if ws is not None else 0,
                ptr(status_word(x.device)), stream_handle(),
            )
        else:
            st = lib().hgq_qdense_fwd(
                ptr(x), ptr(qk), ptr(qi), ptr(qf), rows_period, rm, om, flags, ptr(wq), ptr(bq), act, ptr(y), ptr(absmax), M, K, N,
                ptr(ws), ws.numel() if ws is not None else 0, ptr(status_word(x.device)), stream_handle(),
            )
    check(st, 'hgq_qdense_fwd_pooled' if pool_rows else 'hgq_qdense_fwd')
    if pool_rows:
        return y, absmax, pooled
    return y, absmax


def qdense_pooled_supported(M: int, K: int, N: int, rows_period: int, pool_rows: int, want_absmax: bool = True) -> bool:
    return bool(lib().hgq_qdense_fwd_pooled_supported(M, K, N, rows_period, pool_rows, int(want_absmax)))


_QB_KBLOCK = 64  # input columns one backward launch covers


def qdense_bwd_supported(M: int, K: int, N: int, rows_period: int) -> bool:
    if M <= 0:
        return False
    if K <= _QB_KBLOCK:
        return lib().hgq_qdense_bwd_workspace(M, K, N, rows_period) > 0
    # wider layers run as one launch per block of 64 input columns (each re-reads dY and y: meant for layers whose outputs are
    # few, such as a classifier head behind a Flatten)
    return K % 4 == 0 and K <= 64 * _QB_KBLOCK and all(
        lib().hgq_qdense_bwd_workspace(M, min(_QB_KBLOCK, K - k0), N, rows_period) > 0 for k0 in range(0, K, _QB_KBLOCK))


def qdense_bwd(gy, y, x, qf, rows_period: int, round_mode: str, wq, want_dx: bool, want_db: bool, want_df: bool,
               gy_repeat: int = 1, out_dwq=None, out_dbq=None, out_df=None, dx_into=None):
    """Fused backward of qdense_fwd (rounding-only input quantizer or none).  gy/y are [M, N], x [M, K]; with
    ``gy_repeat`` > 1, gy is [M / gy_repeat, N] and each of its rows serves gy_repeat consecutive rows.
    Returns (dx or None, dwq, dbq or None, df or None).
    ``dx_into``: an [M, K] tensor the input gradient is ADDED to (and returned as dx); see ``qdense_bwd_accumulates``."""
    require_cuda(gy, y, x, qf, wq)
    rm = ROUND_MODES[round_mode.upper()]
    gy, x, wq = gy.contiguous(), x.contiguous(), wq.contiguous()
    y = None if y is None else y.contiguous()
    K, N = wq.shape
    M = x.numel() // K
    dev = x.device
    want_df = want_df and qf is not None
    dx = (dx_into.view(M, K) if dx_into is not None else torch.empty((M, K), dtype=torch.float32, device=dev)) if want_dx else None
    dwq = out_dwq if out_dwq is not None else torch.empty((K, N), dtype=torch.float32, device=dev)
    dbq = (out_dbq if out_dbq is not None else torch.empty(N, dtype=torch.float32, device=dev)) if want_db else None
    direct_df = want_df and out_df is not None and K <= _QB_KBLOCK  # one launch: the kernel writes the caller's table
    dfs = []
    x2 = x.view(M, K)
    qf2 = None if qf is None else qf.reshape(rows_period, K)
    with torch.cuda.device(dev):
        for k0 in range(0, K, _QB_KBLOCK):
            kb = min(_QB_KBLOCK, K - k0)
            qf_b = None if qf2 is None else qf2[:, k0:k0 + kb].contiguous()
            df_b = (out_df if direct_df else torch.empty(rows_period * kb, dtype=torch.float32, device=dev)) if want_df else None
            ws = workspace(lib().hgq_qdense_bwd_workspace(M, kb, N, rows_period), dev, slot=2)
            if dx_into is not None and want_dx:
                st = lib().hgq_qdense_bwd_accumulate(
                    ptr(gy), gy_repeat, ptr(y), x2.data_ptr() + 4 * k0, K, ptr(qf_b), rows_period, rm, wq.data_ptr() + 4 * k0 * N,
                    dx.data_ptr() + 4 * k0, K, 1, dwq.data_ptr() + 4 * k0 * N, ptr(dbq) if k0 == 0 else None, ptr(df_b), M, kb, N,
                    ptr(ws), ws.numel(), ptr(status_word(dev)), stream_handle())
                check(st, 'hgq_qdense_bwd_accumulate')
            else:
                st = lib().hgq_qdense_bwd_strided(
                    ptr(gy), gy_repeat, ptr(y), x2.data_ptr() + 4 * k0, K, ptr(qf_b), rows_period, rm, wq.data_ptr() + 4 * k0 * N,
                    (dx.data_ptr() + 4 * k0) if dx is not None else None, K, dwq.data_ptr() + 4 * k0 * N,
                    ptr(dbq) if k0 == 0 else None, ptr(df_b), M, kb, N, ptr(ws), ws.numel(), ptr(status_word(dev)), stream_handle())
                check(st, 'hgq_qdense_bwd_strided')
            if want_df:
                dfs.append(df_b.view(rows_period, kb))
    df = None
    if want_df:
        if direct_df:
            df = out_df
        elif out_df is not None:
            torch.cat(dfs, dim=1, out=out_df.view(rows_period, K))
            df = out_df
        else:
            df = (dfs[0] if len(dfs) == 1 else torch.cat(dfs, dim=1)).reshape(-1)
    return dx, dwq, dbq, df


def dense_chain_layers(specs):
    """A host array of hgq_chain_layer from dicts with the keys K, N, relu, round_mode and the tensors qf, wq, bq, y, absmax,
    dwq, dbq, df (None where absent)."""
    arr = (_lib.ChainLayer * len(specs))()
    for a, s in zip(arr, specs):
        a.K, a.N, a.relu, a.round_mode = int(s['K']), int(s['N']), int(bool(s['relu'])), ROUND_MODES[s['round_mode'].upper()]
        for name in ('qf', 'wq', 'bq', 'y', 'absmax', 'dwq', 'dbq', 'df'):
            t = s.get(name)
            setattr(a, name, None if t is None else t.data_ptr())
    return arr


def dense_chain_supported(widths) -> bool:
    """Whether a stack of dense layers with these widths (inputs of the first layer, then every layer's outputs) fits the
    single-launch kernels."""
    if len(widths) < 2 or len(widths) - 1 > 8:
        return False
    arr = (_lib.ChainLayer * (len(widths) - 1))()
    for a, k, n in zip(arr, widths[:-1], widths[1:]):
        a.K, a.N = int(k), int(n)
    return bool(lib().hgq_dense_chain_supported(len(arr), arr))


def dense_chain_fwd(x, layers, n_layers: int) -> None:
    """Forward of the stack described by ``layers`` (see dense_chain_layers) on x [M, K0]: fills every layer's y."""
    require_cuda(x)
    M = x.shape[0]
    with torch.cuda.device(x.device):
        check(lib().hgq_dense_chain_fwd(ptr(x), M, n_layers, layers, stream_handle()), 'hgq_dense_chain_fwd')


def dense_chain_bwd(gy, x, dx, layers, n_layers: int) -> None:
    """Backward of the stack: fills dwq / dbq / df of every layer and dx (when not None)."""
    require_cuda(gy, x, dx)
    M = x.shape[0]
    ws = workspace(lib().hgq_dense_chain_workspace(M, n_layers, layers), x.device, slot=6)
    if ws is None:
        raise _lib.HGQError(-2, 'hgq_dense_chain_bwd: unsupported stack')
    with torch.cuda.device(x.device):
        check(lib().hgq_dense_chain_bwd(ptr(gy), ptr(x), ptr(dx), M, n_layers, layers, ptr(ws), ws.numel(), stream_handle()),
              'hgq_dense_chain_bwd')


def qdense_bwd_accumulates(K: int, N: int, rows_period: int, relu: bool, has_quantizer: bool = True) -> bool:
    """Whether ``qdense_bwd(..., dx_into=...)`` is available for a layer of this shape."""
    return K <= _QB_KBLOCK and bool(lib().hgq_qdense_bwd_accumulate_supported(K, N, rows_period, int(relu), int(has_quantizer)))


def _quant_arrays(quants):
    """quants: five (k, i, f, round_mode, overflow_mode) tuples -> ctypes arrays for the softmax entry points."""
    import ctypes

    def arr(vals):
        return (ctypes.c_void_p * 5)(*[None if v is None else v.data_ptr() for v in vals])

    ks = [None if q[0] is None else q[0].contiguous() for q in quants]
    is_ = [None if q[1] is None else q[1].contiguous() for q in quants]
    fs = [q[2].contiguous() for q in quants]
    rms = (ctypes.c_int * 5)(*[ROUND_MODES[q[3]] for q in quants])
    oms = (ctypes.c_int * 5)(*[OVERFLOW_MODES[q[4]] for q in quants])
    keep = (ks, is_, fs)
    return arr(ks), arr(is_), arr(fs), rms, oms, keep


def qsoftmax_supported(L: int) -> bool:
    return L in (32, 64, 128)


def qsoftmax_fwd(s, quants, scaler: float, eps: float, rows_period: int, want_amax3: bool, want_amax5: bool,
                 want_amax1: bool = False, out_amax=(None, None, None)):
    """Fused training-mode QSoftmax forward over the last axis of s.  Returns (y, amax3 or None, amax5 or None, amax1 or
    None): the abs-max statistics of the inverse table's input, the layer output and the exp table's input."""
    require_cuda(s)
    s = s.contiguous()
    L = s.shape[-1]
    R = s.numel() // L
    y = torch.empty_like(s)
    o1, o3, o5 = out_amax  # caller-owned destinations of the three statistics (None: allocate)
    a1 = (o1 if o1 is not None else torch.empty(1, dtype=torch.float32, device=s.device)) if want_amax1 else None
    a3 = (o3 if o3 is not None else torch.empty(1, dtype=torch.float32, device=s.device)) if want_amax3 else None
    a5 = (o5 if o5 is not None else torch.empty(rows_period * L, dtype=torch.float32, device=s.device)) if want_amax5 else None
    qk, qi, qf, rms, oms, keep = _quant_arrays(quants)
    with torch.cuda.device(s.device):
        st = lib().hgq_qsoftmax_fwd(ptr(s), ptr(y), qk, qi, qf, rms, oms, float(scaler), float(eps), ptr(a1), ptr(a3), ptr(a5),
                                    R, L, rows_period, stream_handle())
    check(st, 'hgq_qsoftmax_fwd')
    del keep
    return y, a3, a5, a1


def qsoftmax_bwd(gy, s, quants, scaler: float, eps: float, rows_period: int, want_di5: bool):
    """Fused QSoftmax backward.  Returns (ds, scalars8, df5, di5 or None)."""
    require_cuda(gy, s)
    gy, s = gy.contiguous(), s.contiguous()
    L = s.shape[-1]
    R = s.numel() // L
    ds = torch.empty_like(s)
    sc = torch.empty(8, dtype=torch.float32, device=s.device)
    df5 = torch.empty(rows_period * L, dtype=torch.float32, device=s.device)
    di5 = torch.empty(rows_period * L, dtype=torch.float32, device=s.device) if want_di5 else None
    ws = workspace(lib().hgq_qsoftmax_bwd_workspace(R, L, rows_period), s.device, slot=3)
    qk, qi, qf, rms, oms, keep = _quant_arrays(quants)
    with torch.cuda.device(s.device):
        st = lib().hgq_qsoftmax_bwd(ptr(gy), ptr(s), ptr(ds), qk, qi, qf, rms, oms, float(scaler), float(eps), ptr(sc), ptr(df5),
                                    ptr(di5), R, L, rows_period, ptr(ws), ws.numel(), stream_handle())
    check(st, 'hgq_qsoftmax_bwd')
    del keep
    return ds, sc, df5, di5


def qconv2d_supported(B, H, W, C, KH, KW, N, OH, OW) -> bool:
    return bool(lib().hgq_qconv2d_supported(B, H, W, C, KH, KW, N, OH, OW))


def qconv2d_unit_stride_supported(B, H, W, C, KH, KW, N, OH, OW, dilation=(1, 1)) -> bool:
    return bool(lib().hgq_qconv2d_unit_stride_supported(B, H, W, C, KH, KW, N, OH, OW, dilation[0], dilation[1]))


def qconv2d_fwd(x, wq2d, bq, activation, KH, KW, out_hw, strides, dilation, pad_tl):
    """Implicit-GEMM conv2d forward.  x [B, H, W, C] (already quantised; C % 4 == 0 unless the unit-stride kernel takes the
    shape), wq2d [KH*KW*C, N]."""
    require_cuda(x, wq2d, bq)
    x, wq2d = x.contiguous(), wq2d.contiguous()
    bq = None if bq is None else bq.contiguous()
    B, H, W, C = x.shape
    N = wq2d.shape[1]
    OH, OW = out_hw
    y = torch.empty((B, OH, OW, N), dtype=torch.float32, device=x.device)
    act = {None: 0, 'relu': 1}[activation]
    with torch.cuda.device(x.device):
        st = lib().hgq_qconv2d_fwd(ptr(x), B, H, W, C, ptr(wq2d), ptr(bq), act, ptr(y), KH, KW, N, OH, OW, strides[0], strides[1],
                                   dilation[0], dilation[1], pad_tl[0], pad_tl[1], ptr(status_word(x.device)), stream_handle())
    check(st, 'hgq_qconv2d_fwd')
    return y


def qconv2d_wgrad_supported(B, H, W, C, KH, KW, N, OH, OW) -> bool:
    return lib().hgq_qconv2d_wgrad_workspace(B, H, W, C, KH, KW, N, OH, OW) > 0


def qconv2d_wgrad(x, gy, y, KH, KW, strides, dilation, pad_tl, want_db: bool, out_dwq=None, out_dbq=None):
    """Weight / bias gradient of the implicit-GEMM convolution.  x [B, H, W, C] (C % 4 == 0), gy / y [B, OH, OW, N];
    y is the forward output when the activation was ReLU, else None.  Returns (G, dwq [KH*KW*C, N], dbq or None) with
    G the masked upstream gradient (gy itself without activation)."""
    require_cuda(x, gy, y)
    x, gy = x.contiguous(), gy.contiguous()
    y = None if y is None else y.contiguous()
    B, H, W, C = x.shape
    _, OH, OW, N = gy.shape
    dev = x.device
    gm = torch.empty_like(gy) if y is not None else None
    dwq = out_dwq if out_dwq is not None else torch.empty((KH * KW * C, N), dtype=torch.float32, device=dev)
    dbq = (out_dbq if out_dbq is not None else torch.empty(N, dtype=torch.float32, device=dev)) if want_db else None
    ws = workspace(lib().hgq_qconv2d_wgrad_workspace(B, H, W, C, KH, KW, N, OH, OW), dev, slot=4)
    if ws is None:
        raise _lib.HGQError(-2, 'hgq_qconv2d_wgrad: unsupported shape')
    with torch.cuda.device(dev):
        st = lib().hgq_qconv2d_wgrad(ptr(x), ptr(gy), ptr(y), ptr(gm), ptr(dwq), ptr(dbq), B, H, W, C, KH, KW, N, OH, OW, strides[0],
                                     strides[1], dilation[0], dilation[1], pad_tl[0], pad_tl[1], ptr(ws), ws.numel(),
                                     ptr(status_word(dev)), stream_handle())
    check(st, 'hgq_qconv2d_wgrad')
    return (gm if gm is not None else gy), dwq, dbq


def maxpool2d_fwd(x, pool, strides):
    """channels-last 'valid' max pooling.  Returns (y, argmax uint8)."""
    require_cuda(x)
    x = x.contiguous()
    B, H, W, C = x.shape
    OH, OW = (H - pool[0]) // strides[0] + 1, (W - pool[1]) // strides[1] + 1
    y = torch.empty((B, OH, OW, C), dtype=torch.float32, device=x.device)
    arg = torch.empty((B, OH, OW, C), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        st = lib().hgq_maxpool2d_fwd(ptr(x), ptr(y), ptr(arg), B, H, W, C, pool[0], pool[1], strides[0], strides[1], OH, OW,
                                     stream_handle())
    check(st, 'hgq_maxpool2d_fwd')
    return y, arg


def maxpool2d_bwd(gy, arg, in_shape, pool, strides):
    require_cuda(gy, arg)
    gy = gy.contiguous()
    B, H, W, C = in_shape
    _, OH, OW, _ = gy.shape
    dx = torch.empty(in_shape, dtype=torch.float32, device=gy.device)
    with torch.cuda.device(gy.device):
        st = lib().hgq_maxpool2d_bwd(ptr(gy), ptr(arg), ptr(dx), B, H, W, C, pool[0], pool[1], strides[0], strides[1], OH, OW,
                                     stream_handle())
    check(st, 'hgq_maxpool2d_bwd')
    return dx


def attn_heads_supported(B: int, L: int, H: int, D: int) -> bool:
    return bool(lib().hgq_attn_heads_supported(B, L, H, D))


def attn_heads_matmul(kind: int, x, y, B: int, L: int, H: int, D: int):
    """Per-head attention products (see hgq_attn_heads_matmul).  kind 0: x, y [B, L, H, D] -> [B, H, L, L];
    kinds 1, 2: x [B, H, L, L], y [B, L, H, D] -> [B, L, H, D]."""
    require_cuda(x, y)
    x, y = x.contiguous(), y.contiguous()
    shape = (B, H, L, L) if kind == 0 else (B, L, H, D)
    out = torch.empty(shape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        st = lib().hgq_attn_heads_matmul(kind, ptr(x), ptr(y), ptr(out), B, L, H, D, ptr(status_word(x.device)), stream_handle())
    check(st, 'hgq_attn_heads_matmul')
    return out


def track_supported(*tensors) -> bool:
    return all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() for t in tensors) and \
        len({t.numel() for t in tensors}) == 1


def track_kif(absmax, f_raw, i_state, decay) -> None:
    """In place: i_state <- max(i_state - decay, ceil(log2(absmax + 2^-rint(f_raw))))."""
    with torch.cuda.device(absmax.device):
        st = lib().hgq_track_kif(ptr(absmax), ptr(f_raw), ptr(i_state), ptr(decay), absmax.numel(), stream_handle())
    check(st, 'hgq_track_kif')


def track_kbi(absmax, b_raw, i_state, decay, symmetric: bool, lo: float, hi: float) -> None:
    """In place: i_state <- clamp(max(i_state - decay, minimal_i_given_xb(absmax, rint(b_raw))), lo, hi)."""
    with torch.cuda.device(absmax.device):
        st = lib().hgq_track_kbi(ptr(absmax), ptr(b_raw), ptr(i_state), ptr(decay), 1 if symmetric else 0, float(lo), float(hi),
                                 absmax.numel(), stream_handle())
    check(st, 'hgq_track_kbi')


def softmax_xent(logits, labels):
    """Mean softmax cross-entropy of [B, C] logits against int64 labels.  Returns (loss scalar, dloss/dlogits)."""
    require_cuda(logits, labels)
    logits, labels = logits.contiguous(), labels.contiguous()
    B, C = logits.shape
    loss = torch.empty((), dtype=torch.float32, device=logits.device)
    dlogits = torch.empty_like(logits)
    ws = workspace(lib().hgq_softmax_xent_workspace(B), logits.device, slot=5)
    with torch.cuda.device(logits.device):
        st = lib().hgq_softmax_xent(ptr(logits), ptr(labels), ptr(loss), ptr(dlogits), B, C, ptr(ws), ws.numel(), stream_handle())
    check(st, 'hgq_softmax_xent')
    return loss, dlogits


# ---- batched parameter-side kernels (descriptor tables in device memory, see hgq2_b200.engine) -------------------------
def tables_forward(slots_dev, n_slots: int, max_n: int) -> None:
    with torch.cuda.device(slots_dev.device):
        check(lib().hgq_tables_forward(ptr(slots_dev), n_slots, max_n, stream_handle()), 'hgq_tables_forward')


def tables_track_bits(slots_dev, n_slots: int, max_n: int) -> None:
    with torch.cuda.device(slots_dev.device):
        check(lib().hgq_tables_track_bits(ptr(slots_dev), n_slots, max_n, stream_handle()), 'hgq_tables_track_bits')


def tables_backward(slots_dev, n_slots: int, max_n: int) -> None:
    with torch.cuda.device(slots_dev.device):
        check(lib().hgq_tables_backward(ptr(slots_dev), n_slots, max_n, stream_handle()), 'hgq_tables_backward')


def weights_forward(weights_dev, n_weights: int, max_n: int, slots_dev) -> None:
    with torch.cuda.device(slots_dev.device):
        check(lib().hgq_weights_forward(ptr(weights_dev), n_weights, max_n, ptr(slots_dev), stream_handle()), 'hgq_weights_forward')


def weights_backward(weights_dev, n_weights: int, max_n: int, slots_dev) -> None:
    with torch.cuda.device(slots_dev.device):
        check(lib().hgq_weights_backward(ptr(weights_dev), n_weights, max_n, ptr(slots_dev), stream_handle()), 'hgq_weights_backward')
