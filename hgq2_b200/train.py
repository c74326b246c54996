"""The QAT training step: flat parameter bucket, fused Adam, data-parallel gradient exchange.

What Keras' torch trainer does around the layers of the hot path (forward with ``training=True``,
task loss + ``sum(model.losses)``, backward, optimizer update, constraints) is restated here on one
flat fp32 bucket:

* every trainable variable of the model becomes a view into ``params``; its ``.grad`` is a view into
  ``grads``.  One memset clears the gradients, one NCCL all-reduce averages them over the ranks, one
  fused kernel (``hgq_adam_step``) applies Adam, the MonoL1 regularisers and the MinMax constraints.
* data parallelism shards the batch; the only other exchange is a MAX all-reduce of the per-column
  abs-max statistics that drive the WRAP integer-bit tracking, so that every rank keeps identical
  quantizer state (and therefore identical EBOPs).
"""

from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from . import _lib
from .backend import Layer, Variable, join_bookkeeping
from .constraints import Constant as ConstantConstraint
from .constraints import Max, Min, MinMax
from .quantizer.internal import fixed_point_quantizer as _fpq
from .regularizers import MonoL1


class FlatState:
    """Packs the trainable variables of ``model`` into one fp32 buffer (plus a matching gradient buffer and the
    per-element constraint / regulariser tables the fused optimizer reads)."""

    def __init__(self, model: Layer):
        self.variables: list[Variable] = [v for v in model.trainable_variables]
        if not self.variables:
            raise ValueError('model has no trainable variables (is it built?)')
        dev = self.variables[0].value.device
        sizes = [v.value.numel() for v in self.variables]
        # 4-element alignment keeps every view 16-byte aligned for the vectorised kernels
        self.offsets, off = [], 0
        for n in sizes:
            self.offsets.append(off)
            off += (n + 3) // 4 * 4
        self.n = off
        # one concatenation instead of a copy per variable (padding pieces are slices of one small zero tensor)
        pad = torch.zeros(3, dtype=torch.float32, device=dev)
        pieces = []
        for v, n in zip(self.variables, sizes):
            pieces.append(v.value.detach().reshape(-1).to(torch.float32))
            if (-n) % 4:
                pieces.append(pad[:(-n) % 4])
        self.params = torch.cat(pieces)
        assert self.params.numel() == self.n
        self.grads = torch.zeros(self.n, dtype=torch.float32, device=dev)
        lo = torch.full((self.n,), -math.inf, dtype=torch.float32)
        hi = torch.full((self.n,), math.inf, dtype=torch.float32)
        l1 = torch.zeros(self.n, dtype=torch.float32)
        for v, o, n in zip(self.variables, self.offsets, sizes):
            v.value.data = self.params[o:o + n].view(v.value.shape)
            v.value.grad = self.grads[o:o + n].view(v.value.shape)
            c = v.constraint
            if c is None:
                pass
            elif isinstance(c, MinMax):
                lo[o:o + n], hi[o:o + n] = c.min_value, c.max_value
            elif isinstance(c, Min):
                lo[o:o + n] = c.min_value
            elif isinstance(c, Max):
                hi[o:o + n] = c.max_value
            elif isinstance(c, ConstantConstraint):
                lo[o:o + n] = hi[o:o + n] = c.value
            else:
                raise NotImplementedError(f'constraint {type(c).__name__} on {v.path} cannot be fused')
            r = v.regularizer
            if r is None:
                pass
            elif isinstance(r, MonoL1):
                l1[o:o + n] = r.l1
            else:
                raise NotImplementedError(f'regularizer {type(r).__name__} on {v.path} cannot be fused')
        self.lo, self.hi, self.l1 = lo.to(dev), hi.to(dev), l1.to(dev)

    def zero_grad(self) -> None:
        self.grads.zero_()

    def check_views(self) -> None:
        """Autograd must have accumulated into the bucket views, not replaced them."""
        base = self.grads.data_ptr()
        for v, o in zip(self.variables, self.offsets):
            g = v.value.grad
            if g is None or g.data_ptr() != base + 4 * o:
                raise RuntimeError(f'gradient of {v.path} left the flat bucket')

    def regularization_loss(self) -> torch.Tensor:
        return torch.dot(self.l1, self.params)


class FusedAdam:
    """Keras-flavoured Adam on a ``FlatState`` through the C-ABI kernel (regulariser and constraints included)."""

    def __init__(self, state: FlatState, learning_rate=1e-3, beta_1=0.9, beta_2=0.999, epsilon=1e-7):
        self.state = state
        self.lr, self.b1, self.b2, self.eps = learning_rate, beta_1, beta_2, epsilon
        dev = state.params.device
        self.m = torch.zeros_like(state.params)
        self.v = torch.zeros_like(state.params)
        self.step_count = torch.zeros((), dtype=torch.int64, device=dev)

    def step(self, grad_scale: float = 1.0) -> None:
        s = self.state
        _lib.require_cuda(s.params)
        with torch.cuda.device(s.params.device):
            st = _lib.lib().hgq_adam_step(
                s.params.data_ptr(), s.grads.data_ptr(), self.m.data_ptr(), self.v.data_ptr(), s.lo.data_ptr(),
                s.hi.data_ptr(), s.l1.data_ptr(), s.n, self.lr, self.b1, self.b2, self.eps, grad_scale,
                self.step_count.data_ptr(), _lib.stream_handle(),
            )
        _lib.check(st, 'hgq_adam_step')

    def step_peers(self, peers: 'PeerExchange') -> None:
        """The update from the MEAN of the ranks' gradient buckets, read over peer memory inside the optimizer kernel
        (``hgq_adam_step_peers``).  ``state.grads`` keeps this rank's local gradients."""
        from . import kernels

        s = self.state
        _lib.require_cuda(s.params)
        with torch.cuda.device(s.params.device):
            st = _lib.lib().hgq_adam_step_peers(
                s.params.data_ptr(), s.grads.data_ptr(), self.m.data_ptr(), self.v.data_ptr(), s.lo.data_ptr(),
                s.hi.data_ptr(), s.l1.data_ptr(), s.n, self.lr, self.b1, self.b2, self.eps, self.step_count.data_ptr(),
                peers.ptrs, peers.world, peers.rank, peers.max_polls, kernels.status_word(s.params.device).data_ptr(),
                _lib.stream_handle(),
            )
        _lib.check(st, 'hgq_adam_step_peers')


class PeerExchange:
    """This rank's gradient exchange buffer and its mappings of the other ranks' buffers (CUDA IPC over NVLink), for
    ``FusedAdam.step_peers``: the gradient sum over the ranks and the optimizer update as one kernel per rank, with plain
    peer loads instead of an NCCL all-reduce.  One node, one process per GPU.  ``PeerExchange.create`` returns None when
    some rank cannot map some other rank's buffer (the ranks then agree to keep the NCCL all-reduce)."""

    def __init__(self, own, ptrs, opened, world, rank, device):
        self.own, self.ptrs, self.opened = own, ptrs, opened
        self.world, self.rank, self.device = world, rank, device
        self.max_polls = int(os.environ.get('HGQ_PEER_MAX_POLLS', str(1 << 25)))  # a few seconds of polling at most

    @classmethod
    def create(cls, dp: 'DataParallel', n: int, device: torch.device):
        import ctypes

        L = _lib.lib()
        world, rank = dp.world, dp.rank
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        ok = 1
        with torch.cuda.device(device):
            st = L.hgq_peer_buffer_create(L.hgq_peer_exchange_bytes(n), ctypes.byref(own), handle)
            if st != 0:
                ok, own = 0, ctypes.c_void_p()
            mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=device)
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine, group=dp.group)
            ptrs = (ctypes.c_void_p * world)()
            opened = []
            for r, h in enumerate(gathered):
                if r == rank:
                    ptrs[r] = own.value
                    continue
                raw = (ctypes.c_ubyte * 64)(*h.cpu().tolist())
                p = ctypes.c_void_p()
                if ok and L.hgq_peer_buffer_open(raw, ctypes.byref(p)) == 0:
                    ptrs[r] = p.value
                    opened.append(p.value)
                else:
                    ok = 0
            agreed = torch.tensor([ok], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=dp.group)
            self = cls(own.value, ptrs, opened, world, rank, device)
            if int(agreed.item()) == 0:
                self.close()
                return None
            return self

    def close(self) -> None:
        L = _lib.lib()
        with torch.cuda.device(self.device):
            for p in self.opened:
                L.hgq_peer_buffer_close(p)
            if self.own:
                L.hgq_peer_buffer_destroy(self.own)
        self.opened, self.own = [], None


def shard_batch(n: int, rank: int, world: int) -> slice:
    """Contiguous, equal shard of a batch of n samples (n must divide evenly so per-rank means average correctly)."""
    if n % world != 0:
        raise ValueError(f'batch {n} does not divide over {world} ranks')
    per = n // world
    return slice(rank * per, (rank + 1) * per)


class DataParallel:
    """Batch-sharded training over the ranks of a torch.distributed process group (NCCL on GPUs).

    ``sync_gradients`` averages the flat gradient bucket; ``absmax_sync`` is installed as the hook the WRAP
    quantizers call on their abs-max statistics (a MAX all-reduce), which keeps ``i`` -- and with it the EBOPs
    term -- identical on every rank and equal to what one rank would compute on the whole batch.
    """

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError('torch.distributed is not initialised')
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def sync_gradients(self, grads: torch.Tensor, average: bool = True) -> None:
        """Sum the gradient bucket over the ranks; ``average=False`` leaves the division by the number of ranks to the
        caller (the trainer folds it into the optimizer kernel's gradient scale instead of a pass of its own)."""
        if self.world > 1:
            dist.all_reduce(grads, op=dist.ReduceOp.SUM, group=self.group)
            if average:
                grads.div_(self.world)

    def absmax_sync(self, absmax: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(absmax, op=dist.ReduceOp.MAX, group=self.group)
        return absmax

    def __enter__(self):
        from . import backend

        self._prev = (_fpq.absmax_sync_hook, backend.moments_group)
        _fpq.absmax_sync_hook = self.absmax_sync
        backend.moments_group = self.group  # synchronized batch statistics are averaged over this group's ranks
        return self

    def __exit__(self, *exc):
        from . import backend

        _fpq.absmax_sync_hook, backend.moments_group = self._prev


class _SoftmaxXentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        from . import kernels

        loss, dlogits = kernels.softmax_xent(logits, labels)
        ctx.save_for_backward(dlogits)
        return loss

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits * g, None


def sparse_categorical_crossentropy(logits, labels):
    """Mean softmax cross-entropy from logits with integer labels (what the reference's models are compiled with), on the
    fused kernel when the logits are a CUDA [B, C <= 64] fp32 matrix with int64 labels; torch's otherwise."""
    if logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.shape[1] <= 64 and labels.dtype == torch.int64:
        return _SoftmaxXentFn.apply(logits, labels)
    return torch.nn.functional.cross_entropy(logits, labels)


class Trainer:
    """One model, one flat bucket, one fused optimizer; ``step(x, y)`` runs a full QAT step and returns the loss.

    ``capture(x, y)`` records the whole step (forward, backward, gradient exchange, optimizer) into a CUDA graph over
    static input buffers; afterwards ``step`` copies the batch into those buffers and replays the graph, which removes
    the per-kernel launch and Python cost that dominates the small models.
    """

    def __init__(self, model: Layer, loss_fn, learning_rate=1e-3, dp: DataParallel | None = None, engine: bool | None = None):
        """``engine``: run forward and backward through the static step plan of ``hgq2_b200.engine`` (batched bitwidth
        arithmetic, no autograd graph).  None (default): use it when it covers the model, else the autograd path; True:
        require it (raises ``engine.Unsupported`` otherwise); False: always the autograd path.  The environment variable
        ``HGQ_ENGINE=0`` turns the default off."""
        self.model = model
        self.loss_fn = loss_fn
        self.dp = dp
        self.state = FlatState(model)
        self.opt = FusedAdam(self.state, learning_rate=learning_rate)
        self.engine = None
        self.engine_refusal = None  # why the static step plan is not in use (None: it is, or it was not asked for)
        if engine is None:
            engine = None if os.environ.get('HGQ_ENGINE', '1') != '0' else False
        if engine is not False and self.state.params.is_cuda:
            from .engine import Engine, Unsupported

            try:
                self.engine = Engine(model, self.state)
                self.engine.dp = dp
            except Unsupported as why:
                if engine is True:
                    raise
                self.engine_refusal = str(why)
        # gradient exchange over peer memory inside the optimizer kernel (one node, NCCL process group on GPUs);
        # HGQ_PEER_EXCHANGE=0 keeps the NCCL all-reduce
        self.peers = None
        if (dp is not None and dp.world > 1 and self.state.params.is_cuda and dist.get_backend(dp.group) == 'nccl'
                and os.environ.get('HGQ_PEER_EXCHANGE', '1') != '0'):
            self.peers = PeerExchange.create(dp, self.state.n, self.state.params.device)
        self._graphs = []      # captured steps, one per set of static input buffers
        self._sbuf = []        # the static (x, y) buffers the graphs read
        self._next_buf = 0
        # status word of the tensor-core kernels (set when a bounded device-side wait gives up), read back without a sync
        self._status_dev = None
        self._status_host = None
        self._status_event = None

    def forward_backward(self, x, y):
        if self.engine is not None:
            from .engine import Unsupported

            try:
                self.engine.check(int(x.shape[0]))
            except Unsupported as why:  # this batch size is outside some kernel: the autograd path takes over for good
                self.engine, self.engine_refusal = None, str(why)
            else:
                return self.engine.forward_backward(x, y, self.loss_fn)
        self.state.zero_grad()
        pred = self.model(x, training=True)
        task = self.loss_fn(pred, y)
        join_bookkeeping()  # the EBOPs terms were computed on the bookkeeping stream
        total = task
        for extra in self.model._losses:  # the beta * EBOPs terms; the weight regularisers are fused into the optimizer
            total = total + extra
        total.backward()
        return task.detach(), total.detach() + self.state.regularization_loss()

    def _eager_step(self, x, y):
        if self.dp is not None:
            with self.dp:
                task, total = self.forward_backward(x, y)
            if self.peers is not None:
                self.opt.step_peers(self.peers)  # gradient sum over peer memory and update in one kernel
            else:
                self.dp.sync_gradients(self.state.grads, average=False)
                self.opt.step(grad_scale=1.0 / self.dp.world)  # the mean over the ranks, folded into the optimizer kernel
        else:
            task, total = self.forward_backward(x, y)
            self.opt.step()
        self._queue_status_read()
        return total

    # -- device status ---------------------------------------------------------------------------------------------------
    def _queue_status_read(self) -> None:
        """Copy the device status word to pinned host memory behind the step (no synchronisation; part of a captured
        step like any other node)."""
        if not self.state.params.is_cuda:
            return
        from . import kernels

        if self._status_dev is None:
            self._status_dev = kernels.status_word(self.state.params.device)
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_host.copy_(self._status_dev, non_blocking=True)
        if not torch.cuda.is_current_stream_capturing():
            self._status_event = torch.cuda.Event()
            self._status_event.record()

    def check_status(self, wait: bool = False) -> None:
        """Raise ``HGQError`` (HGQ_ERR_TIMEOUT) if a kernel of an earlier step reported that one of its bounded waits gave
        up: that step's outputs, gradients and the update made from them are garbage.  Without ``wait`` only a read-back
        that has already landed is looked at, so calling this at the start of every step costs no synchronisation; the
        word is cleared once reported."""
        if self._status_host is None:
            return
        ev = self._status_event
        if ev is not None:
            if wait:
                ev.synchronize()
            elif not ev.query():
                return
        if int(self._status_host[0]) != 0:
            v = int(self._status_host[0])
            self._status_host.zero_()
            self._status_dev.zero_()
            raise _lib.HGQError(-7, f'training step (device status word = {v})')

    def capture(self, x, y, warmup: int = 3, double_buffer: bool = False) -> None:
        """Record the step as a CUDA graph for batches shaped like (x, y).  Runs ``warmup`` real steps first.

        ``double_buffer``: record the step twice, over two sets of static input buffers that share one memory pool;
        ``prefetch`` then copies a host batch straight into the set the step after next will read, with no staging copy
        on the device."""
        self._sbuf = [(x.clone(), y.clone()) for _ in range(2 if double_buffer else 1)]
        self._graphs, self._next_buf = [], 0
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._eager_step(*self._sbuf[0])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.check_status(wait=True)
        pool = None
        for sx, sy in self._sbuf:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=pool):
                loss = self._eager_step(sx, sy)
            pool = graph.pool()
            self._graphs.append((graph, loss))

    def prefetch(self, hx, hy):
        """Start the host-to-device copy of a (pinned) host batch on a copy stream of its own and return a handle for
        ``step_prefetched``; the copy of batch n + 1 overlaps step n.  After ``capture(..., double_buffer=True)`` the
        batch lands directly in the static buffers of the graph that will consume it; otherwise two device staging
        slots alternate."""
        if not hasattr(self, '_copy_stream'):
            self._copy_stream = torch.cuda.Stream()
            self._slots = [None, None]
            self._slot = 0
        direct = len(self._graphs) == 2 and hx.shape == self._sbuf[0][0].shape and hy.shape == self._sbuf[0][1].shape
        if direct:
            j = self._next_buf
            self._next_buf ^= 1
            dx, dy = self._sbuf[j]
        else:
            j = self._slot
            self._slot ^= 1
            dev = self.state.params.device
            if self._slots[j] is None or self._slots[j][0].shape != hx.shape or self._slots[j][1].shape != hy.shape:
                self._slots[j] = (torch.empty(hx.shape, dtype=hx.dtype, device=dev), torch.empty(hy.shape, dtype=hy.dtype, device=dev))
            dx, dy = self._slots[j]
        # everything queued so far has consumed the buffer's previous batch (two steps back; the step that overlaps this
        # copy is launched after this call and reads the other buffer)
        self._copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._copy_stream):
            dx.copy_(hx, non_blocking=True)
            dy.copy_(hy, non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        return dx, dy, done, (j if direct else None)

    def step_prefetched(self, handle):
        """``step`` on a batch started with ``prefetch``."""
        dx, dy, done, buf = handle
        torch.cuda.current_stream().wait_event(done)
        if buf is not None:
            self.check_status()
            return self._replay(buf)
        return self.step(dx, dy)

    def step(self, x, y):
        """One QAT step on a device batch; returns the loss (a device scalar, valid until the next step)."""
        self.check_status()
        if self._graphs and x.shape == self._sbuf[0][0].shape and y.shape == self._sbuf[0][1].shape:
            sx, sy = self._sbuf[0]
            if x.data_ptr() != sx.data_ptr():
                sx.copy_(x, non_blocking=True)
            if y.data_ptr() != sy.data_ptr():
                sy.copy_(y, non_blocking=True)
            return self._replay(0)
        return self._eager_step(x, y)

    def _replay(self, buf: int):
        graph, loss = self._graphs[buf]
        graph.replay()
        self._status_event = torch.cuda.Event()  # behind the replay, whose last node is the status read-back
        self._status_event.record()
        return loss

    @property
    def static_inputs(self):
        """The static (x, y) buffers of the captured step: a caller that writes its batch there itself (and passes these
        very tensors to ``step``) saves the device-to-device copy."""
        return self._sbuf[0] if self._sbuf else None
