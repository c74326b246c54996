#!/usr/bin/env python
"""Benchmark of the HGQ2 quantizer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the standalone fixed-point quantizer sweep -- 2^28 fp32 elements drawn from N(0, 4^2),
per-element integer parameters k in {0,1}, i in [-2,6], f in [0,8], all six combinations of
{RND,TRN} x {WRAP,SAT,SAT_SYM}, forward plus surrogate backward with an N(0,1) upstream
gradient.  One step = one full sweep (6 forward + 6 backward passes over this rank's share of the
element range).  With N > 1 (torchrun, one rank per GPU) the 2^28 elements are split contiguously
over the ranks and no data crosses between them.

Metric: achieved algorithmic bandwidth in GB/s.  Bytes per element: forward reads x,i,f fp32 + k uint8
(13 B) and writes y (4 B) = 17 B; SAT / SAT_SYM backward reads g,x,i,f,k (17 B) and writes dx,di,df (12 B)
= 29 B; WRAP backward needs neither k nor i and its di is identically zero, so it reads g,x,f (12 B) and
writes dx,df (8 B) = 20 B.  A full sweep is 2 x (17+20) + 4 x (17+29) = 258 B per element.

`--impl reference` times the reference's CPU formulation of the same sweep (the eager fp32 op
sequence of oracle/fixed_point_ops.py on the host cores) on a bounded sample.

Prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

TOTAL_ELEMS = 1 << 28
BYTES_FWD, BYTES_BWD = 17, 29
BYTES_BWD_WRAP = 20
MODES = [(rm, om) for rm in ('RND', 'TRN') for om in ('WRAP', 'SAT', 'SAT_SYM')]
BYTES_PER_ELEM_SWEEP = sum(BYTES_FWD + (BYTES_BWD_WRAP if om == 'WRAP' else BYTES_BWD) for _, om in MODES)  # 258
METRIC = 'quantizer_sweep_hbm_bandwidth'
UNIT = 'GB/s'
# DRAM bytes per element per launch (read + write) measured by ncu on a 2^25-element case of the
# same kernels (profiles/quantize_full_layout_sweep.md); traffic grows in proportion to the element count.
NCU_TRAFFIC_BYTES_PER_ELEM = {'k_bwd_full': 27.56, 'k_fwd_full': 16.16}


def measured_peaks():
    p = ROOT / 'MEASURED_PEAKS.json'
    if p.exists():
        d = json.loads(p.read_text())
        return float(d['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with NVML while a timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get('CUDA_VISIBLE_DEVICES')
            phys = int(visible.split(',')[index]) if visible and visible.split(',')[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            'hw_slowdown': nv.nvmlClocksThrottleReasonHwSlowdown,
            'hw_thermal_slowdown': nv.nvmlClocksThrottleReasonHwThermalSlowdown,
            'sw_thermal_slowdown': nv.nvmlClocksThrottleReasonSwThermalSlowdown,
            'sw_power_cap': nv.nvmlClocksThrottleReasonSwPowerCap,
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': self.max_mhz, 'reasons': ['nvml unavailable']}
        return {'sm_mhz': float(np.median(self.samples)), 'sm_max_mhz': self.max_mhz, 'reasons': sorted(self.reasons),
                'samples': len(self.samples)}


def make_inputs_np(n: int, seed: int):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n, dtype=np.float32) * np.float32(4.0)
    k = rng.integers(0, 2, n, dtype=np.uint8)
    i = rng.integers(-2, 7, n).astype(np.float32)
    f = rng.integers(0, 9, n).astype(np.float32)
    g = rng.standard_normal(n, dtype=np.float32)
    return x, k, i, f, g


# ------------------------------------------------------------------------------------------------
def cpu_sweep(sample: int, threads: int, steps: int, warmup: int):
    """The reference formulation on the host: eager fp32 torch ops, materialised parameters."""
    from oracle import fixed_point_ops as O

    torch.set_num_threads(threads)
    x, k, i, f, g = (torch.from_numpy(a) for a in make_inputs_np(sample, 1))
    kf = k.float()

    def one_step():
        for rm, om in MODES:
            O.quantize_fwd(x, kf, i, f, rm, om, training=False)
            O.quantize_bwd(g, x, kf, i, f, rm, om)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    gbs = BYTES_PER_ELEM_SWEEP * sample / dt / 1e9
    return gbs, dt


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample = 1 << 24
    gbs, dt = cpu_sweep(sample, threads, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': round(gbs, 3), 'unit': UNIT, 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': round(dt * 1e3, 3), 'higher_is_better': True,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': dict(workload_config(args.gpus), elements_timed_per_pass=sample,
                       note='the CPU arm times a 2^24-element sample of the 2^28-element workload; GB/s is per byte, so the '
                            'figures compare'),
        'cpu_baseline': {'value': round(gbs, 3), 'unit': UNIT, 'cores': threads, 'kind': 'port',
                         'sample': f'{sample} elements per pass (2^24 of the 2^28), 6 modes x (fwd+bwd) per step, '
                                   'eager fp32 torch-CPU op sequence of the oracle'},
        'e2e': {'value': round(gbs, 3), 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int):
    return {
        'workload': 'standalone fixed-point quantizer sweep: 2^28 fp32 elements N(0,16), per-element k/i/f, '
                    '{RND,TRN}x{WRAP,SAT,SAT_SYM}, forward + surrogate backward',
        'elements_total': TOTAL_ELEMS, 'elements_per_gpu': TOTAL_ELEMS // n_gpus,
        'bytes_per_element': {'fwd': BYTES_FWD, 'bwd_sat': BYTES_BWD, 'bwd_wrap': BYTES_BWD_WRAP, 'sweep': BYTES_PER_ELEM_SWEEP},
        'sharding': f'contiguous element range / {n_gpus}, no collective',
        'l2': 'inputs larger than L2 (>= 1.5 GB touched per launch vs 126 MB L2)',
    }


# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch.distributed as dist

    from hgq2_b200 import kernels

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the product path has no CPU fallback')
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    n = TOTAL_ELEMS // world

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- inputs resident in HBM -----------------------------------------------------------------
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn(n, device=dev, generator=gen) * 4.0
    g = torch.randn(n, device=dev, generator=gen)
    k = torch.randint(0, 2, (n,), device=dev, generator=gen, dtype=torch.uint8)
    i = torch.randint(-2, 7, (n,), device=dev, generator=gen).float()
    f = torch.randint(0, 9, (n,), device=dev, generator=gen).float()
    y, dx, di, df = (torch.empty(n, device=dev) for _ in range(4))
    L = kernels._lib.lib()
    P = kernels.ptr
    RM, OM = kernels._lib.ROUND_MODES, kernels._lib.OVERFLOW_MODES
    st = torch.cuda.current_stream().cuda_stream

    def fwd(rm, om):
        kernels.check(L.hgq_quantize_fwd(P(x), P(k), P(i), P(f), P(y), None, n, n, RM[rm], OM[om], 0, st), 'fwd')

    def bwd(rm, om):
        di_p = None if om == 'WRAP' else P(di)  # WRAP has no integer-bit gradient
        kernels.check(L.hgq_quantize_bwd(P(g), P(x), P(k), P(i), P(f), P(dx), di_p, P(df), n, n, RM[rm], OM[om], 0,
                                         None, 0, st), 'bwd')

    def step():
        for rm, om in MODES:
            fwd(rm, om)
            bwd(rm, om)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    launches0 = kernels.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    launches = kernels.launch_count() - launches0
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    bytes_per_step_total = BYTES_PER_ELEM_SWEEP * TOTAL_ELEMS
    value = bytes_per_step_total / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel (backward, full layout), timed alone -------------------
    def time_kernel(fn, reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    reps = max(6, args.steps)
    t_bwd = time_kernel(lambda: bwd('RND', 'SAT'), reps)
    t_fwd = time_kernel(lambda: fwd('RND', 'SAT'), reps)
    peak, peak_kind = measured_peaks()
    ach = BYTES_BWD * n / (t_bwd * 1e-3) / 1e9
    tr = NCU_TRAFFIC_BYTES_PER_ELEM['k_bwd_full']
    roofline = {
        'bound': 'hbm', 'kernel': 'k_bwd_full (surrogate backward, full layout)', 'achieved': round(ach, 1),
        'peak': peak, 'peak_source': f'{peak_kind} copy bandwidth (burst)', 'unit': 'GB/s', 'frac': round(ach / peak, 4),
        'frac_of_8TBs_nominal': round(ach / 8000.0, 4),
        'traffic': (tr * n if tr is not None else None),
        'launch_ms': round(t_bwd, 4),
        'fwd_kernel': {'achieved': round(BYTES_FWD * n / (t_fwd * 1e-3) / 1e9, 1), 'launch_ms': round(t_fwd, 4),
                       'frac': round(BYTES_FWD * n / (t_fwd * 1e-3) / 1e9 / peak, 4)},
    }

    # ---- end to end through the host-buffer C-ABI entry ----------------------------------------
    e2e = None
    if not args.no_e2e:
        try:
            e2e = run_e2e(args, kernels, n, dev, world, rank)
        except Exception as exc:  # report, do not hide
            e2e = {'value': None, 'unit': UNIT, 'error': repr(exc)[:300]}

    # ---- CPU baseline on rank 0 at N = 1 --------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        sample = 1 << 24
        gbs, dt = cpu_sweep(sample, threads, 3, 1)
        cpu = {'value': round(gbs, 3), 'unit': UNIT, 'cores': threads, 'kind': 'port',
               'sample': f'{sample} elements per pass (2^24 of 2^28), 6 modes x (fwd+bwd), 3 steps; eager fp32 '
                         'torch-CPU op sequence of the oracle'}

    # free the sweep's device arrays before the training workloads
    del x, g, k, i, f, y, dx, di, df
    torch.cuda.empty_cache()
    qat = None if args.no_qat else run_qat(args, dev, world, rank, peak)

    if rank == 0:
        line = {
            'metric': METRIC, 'value': round(value, 2), 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
            'warmup': max(3, args.warmup), 'ms_per_step': round(ms_per_step, 4), 'higher_is_better': True,
            'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'config': workload_config(world), 'roofline': roofline, 'cpu_baseline': cpu, 'e2e': e2e,
            'gpu_launches': int(launches), 'clocks': clocks.summary(), 'qat_step': qat,
            'frac_of_measured_copy_peak': round(value / world / peak, 4),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# reduced batches for the CPU leg of the QAT step (the oracle's eager torch-CPU formulation), sized for a few seconds each
QAT_CPU_BATCH = {'jet_tagger_mlp': 16384, 'particle_tagger': 512, 'small_cnn': 128, 'transformer_block': 64}


def cpu_qat_step(name, builder_model, make_x, classes):
    """samples/s of one QAT step (forward, backward, Adam, constraints) of the oracle twin on the host cores."""
    import torch.nn.functional as F

    from oracle import train as OT

    batch = QAT_CPU_BATCH[name]
    torch.set_num_threads(os.cpu_count() or 1)
    twin, pairs = OT.mirror_model(builder_model)
    opt = OT.OracleAdam(pairs)
    x = torch.from_numpy(make_x(np.random.default_rng(1), batch))
    y = torch.from_numpy(np.random.default_rng(2).integers(0, classes, batch))
    OT.train_step(twin, opt, x, y, F.cross_entropy)  # warm-up
    t0 = time.perf_counter()
    n = 0
    while n < 3 or (time.perf_counter() - t0 < 2.0 and n < 50):
        OT.train_step(twin, opt, x, y, F.cross_entropy)
        n += 1
    dt = (time.perf_counter() - t0) / n
    return {'samples_per_s': round(batch / dt, 1), 'batch': batch, 'steps': n, 'cores': os.cpu_count() or 1, 'kind': 'port'}


QAT_CONFIGS = {
    # name: (builder, global batch, input maker, classes, modelled HBM bytes per sample for one QAT step)
    'jet_tagger_mlp': ('jet_tagger_mlp', 16384, lambda rng, b: rng.standard_normal((b, 16), dtype=np.float32), 5, 3324),
    'particle_tagger': ('particle_tagger', 65536, lambda rng, b: rng.standard_normal((b, 64, 16), dtype=np.float32), 5, 162108),
    'small_cnn': ('small_cnn', 4096, lambda rng, b: rng.random((b, 32, 32, 3), dtype=np.float32), 10, 657144),
    'transformer_block': ('transformer_block', 8192, lambda rng, b: rng.standard_normal((b, 64, 64), dtype=np.float32), 5,
                          1721916),
}


def run_qat_single(args):
    """Eager (no CUDA graph) QAT steps of one benchmark model, for kernel-level profiling of a training step."""
    import torch.nn.functional as F

    from hgq2_b200 import workloads
    from hgq2_b200.train import Trainer, sparse_categorical_crossentropy

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    builder, batch, make_x, classes, _ = QAT_CONFIGS[args.model]
    batch = args.batch or batch
    model = workloads.build(getattr(workloads, builder)(), device=dev)
    tr = Trainer(model, sparse_categorical_crossentropy)
    x = torch.from_numpy(make_x(np.random.default_rng(1), batch)).to(dev)
    y = torch.from_numpy(np.random.default_rng(2).integers(0, classes, batch)).to(dev)
    for _ in range(max(1, args.warmup)):
        tr.step(x, y)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        loss = tr.step(x, y)
    b.record()
    torch.cuda.synchronize()
    print(json.dumps({'model': args.model, 'batch': batch, 'eager_ms_per_step': round(a.elapsed_time(b) / args.steps, 3),
                      'loss': float(loss)}), flush=True)


def progress(msg: str) -> None:
    """Phase marker on stderr (rank 0): tells where a run stopped if it does not reach its JSON line."""
    if int(os.environ.get('RANK', '0')) == 0:
        print(f'[bench {time.strftime("%H:%M:%S")}] {msg}', file=sys.stderr, flush=True)


def run_qat(args, dev, world, rank, peak):
    """Full QAT steps (forward, backward, gradient all-reduce, fused Adam) of the benchmark models; the global batch is
    fixed and sharded over the ranks.  Reported beside the sweep: samples/s with the batch resident on the device, the
    same with the batch copied from pinned host memory and the loss read back every step, and the fraction of the HBM
    roofline under the model 'every layer-boundary activation crosses HBM once per use' (bytes per sample above)."""
    import torch.distributed as dist
    import torch.nn.functional as F

    from hgq2_b200 import routes, workloads
    from hgq2_b200.train import DataParallel, Trainer, shard_batch, sparse_categorical_crossentropy

    out = []
    dp = DataParallel() if world > 1 else None
    only = [m for m in args.qat_models.split(',') if m]
    for name, (builder, batch, make_x, classes, bytes_per_sample) in QAT_CONFIGS.items():
        if only and name not in only:
            continue
        try:
            progress(f'qat {name}: build')
            model = workloads.build(getattr(workloads, builder)(), device=dev)
            cpu = None
            if rank == 0 and world == 1 and not args.no_cpu:
                cpu = cpu_qat_step(name, model, make_x, classes)  # twin of the freshly built model, before any step
            tr = Trainer(model, sparse_categorical_crossentropy, dp=dp)
            sl = shard_batch(batch, rank, world)
            hx = torch.from_numpy(make_x(np.random.default_rng(1), batch)[sl]).pin_memory()
            hy = torch.from_numpy(np.random.default_rng(2).integers(0, classes, batch)[sl]).pin_memory()
            x, y = hx.to(dev), hy.to(dev)
            steps = max(3, args.steps)
            progress(f'qat {name}: capture')
            routes.reset()
            # the whole step as one CUDA graph, recorded over two sets of static input buffers so that a host batch can be
            # copied straight into the set the step after next reads
            tr.capture(x, y, warmup=3, double_buffer=True)
            fallbacks = routes.fallbacks()  # library routines a layer fell back to while the step was recorded (none expected)
            x, y = tr.static_inputs  # the batch is resident where the captured step reads it
            progress(f'qat {name}: timed steps')
            for _ in range(3):
                tr.step(x, y)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                tr.step(x, y)
            b.record()
            torch.cuda.synchronize()
            ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
            # end to end: host batch in, loss out, every step
            # every step copies its batch from pinned host memory and reads its loss back; the copy of batch n + 1 is
            # started before step n is launched, so it overlaps the step (it lands in the other set of static buffers)
            progress(f'qat {name}: end-to-end steps')
            for _ in range(2):  # untimed warm-up of the copy stream
                tr.step_prefetched(tr.prefetch(hx, hy))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            nxt = tr.prefetch(hx, hy)
            for s_i in range(steps):
                cur = nxt
                if s_i + 1 < steps:
                    nxt = tr.prefetch(hx, hy)
                loss = tr.step_prefetched(cur)
                loss_host = float(loss.item())
            e2e_ms = torch.tensor([(time.perf_counter() - t0) / steps * 1e3], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
            sps = batch / (float(ms.item()) * 1e-3)
            from hgq2_b200 import kernels as _k

            _k.check_status(dev)  # a bounded tensor-core wait that gave up would have left its mark here
            out.append({
                'model': name, 'global_batch': batch, 'ms_per_step': round(float(ms.item()), 4),
                'samples_per_s': round(sps, 1), 'e2e_samples_per_s': round(batch / (float(e2e_ms.item()) * 1e-3), 1),
                'h2d_bytes_per_step': int(hx.numel() * 4 + hy.numel() * 8), 'd2h_bytes_per_step': 4,
                'hbm_roofline_frac': round(sps * bytes_per_sample / world / (peak * 1e9), 4),
                'modelled_bytes_per_sample': bytes_per_sample, 'loss': round(loss_host, 5), 'cuda_graph': True,
                'library_fallbacks': fallbacks, 'cpu_baseline': cpu,
            })
            progress(f'qat {name}: done')
            del model, tr, x, y, hx, hy
            torch.cuda.empty_cache()
        except Exception as exc:
            out.append({'model': name, 'error': repr(exc)[:300]})
    return out


def run_e2e(args, kernels, n, dev, world, rank):
    import torch.distributed as dist

    chunk = 1 << 24
    ws = torch.empty(kernels.quantize_host_workspace(chunk), dtype=torch.uint8, device=dev)
    xs = make_inputs_np(n, 100 + rank)
    hx, hk, hi, hf, hg = (torch.from_numpy(a).pin_memory() for a in xs)
    hy, hdx, hdi, hdf = (torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(4))
    steps = max(1, min(args.steps, 2))

    def step():
        for rm, om in MODES:
            kernels.quantize_fwd_bwd_host(hx, hk, hi, hf, hg, hy, hdx, None if om == 'WRAP' else hdi, hdf, rm, om, False,
                                          ws, chunk)

    kernels.quantize_fwd_bwd_host(hx, hk, hi, hf, hg, hy, hdx, hdi, hdf, 'RND', 'SAT', False, ws, chunk)  # warm-up
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    t = torch.tensor([dt], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item()) / steps
    total = BYTES_PER_ELEM_SWEEP * TOTAL_ELEMS
    return {
        'value': round(total / dt / 1e9, 2), 'unit': UNIT, 'ms_per_step': round(dt * 1e3, 2), 'steps': steps,
        'h2d_bytes_per_step': len(MODES) * 17 * n, 'd2h_bytes_per_step': (4 * 16 + 2 * 12) * n,
        'api': 'hgq_quantize_fwd_bwd_host: pinned host buffers, 3-stream chunked pipeline, synchronous return',
    }


def run_qdense(args):
    """Kernel-level benchmark of the fused dense forward (quantise -> tcgen05 GEMM -> bias/ReLU) on the per-particle
    layer shape of the particle tagger: M = batch x 64 rows, K = N = 64, input bitwidths [64, 64].  Algorithmic bytes
    per row: 4 (K + N)."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    M, K, N, rp = args.rows, args.k, args.n, args.rows_period
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, device=dev, generator=gen)
    f = torch.full((rp, K), 6.0, device=dev)
    w = (torch.randint(-128, 128, (K, N), device=dev, generator=gen).float() / 64.0)
    b = torch.zeros(N, device=dev)
    # --pool-rows P: the kernel also sums y over groups of P consecutive rows (the particle tagger's sum over particles)
    fn = lambda: kernels.qdense_fwd(x, None, None, f, rp, 'RND', 'WRAP', True, False, w, b, 'relu', True, pool_rows=args.pool_rows)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    kernels.check_status(dev)
    a, bb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        fn()
    bb.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(bb) / args.steps
    peak, kind = measured_peaks()
    gbs = 4.0 * (K + N) * M / (ms * 1e-3) / 1e9
    print(json.dumps({'kernel': 'k_qdense_fwd', 'M': M, 'K': K, 'N': N, 'rows_period': rp, 'pool_rows': args.pool_rows, 'ms': round(ms, 4),
                      'achieved_GBs': round(gbs, 1), 'peak_GBs': peak, 'frac': round(gbs / peak, 4), 'peak_source': kind,
                      'tflops': round(2.0 * M * K * N / (ms * 1e-3) / 1e12, 2)}), flush=True)


def run_qdense_bwd(args):
    """Kernel-level benchmark of the fused dense backward (dX, dWq, dbq, df in one pass) on the particle-tagger layer
    shape.  Algorithmic bytes per row: 4 (2 N + 2 K): dY, y and x in, dX out."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    M, K, N, rp = args.rows, args.k, args.n, args.rows_period
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, device=dev, generator=gen)
    gy = torch.randn(M, N, device=dev, generator=gen)
    y = torch.randn(M, N, device=dev, generator=gen).clamp_min(0)
    f = torch.full((rp, K), 6.0, device=dev)
    w = (torch.randint(-128, 128, (K, N), device=dev, generator=gen).float() / 64.0)
    fn = lambda: kernels.qdense_bwd(gy, y, x, f, rp, 'RND', w, True, True, True)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    kernels.check_status(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    peak, kind = measured_peaks()
    gbs = 4.0 * (2 * K + 2 * N) * M / (ms * 1e-3) / 1e9
    print(json.dumps({'kernel': 'k_qdense_bwd', 'M': M, 'K': K, 'N': N, 'rows_period': rp, 'ms': round(ms, 4),
                      'achieved_GBs': round(gbs, 1), 'peak_GBs': peak, 'frac': round(gbs / peak, 4), 'peak_source': kind}), flush=True)


def run_dense_chain(args):
    """Kernel-level benchmark of the single-launch dense stack (hgq_dense_chain_fwd / _bwd) on the jet-tagger MLP's layers:
    16 -> 64 -> 32 -> 32 -> 5, ReLU on the first three, batch 16384 (--batch).  Activations are L2-resident at this size; the
    figures are microseconds per launch, not bandwidth."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    M = args.batch or 16384
    widths, relus = (16, 64, 32, 32, 5), (True, True, True, False)
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, widths[0], device=dev, generator=gen) * 2
    specs = []
    for K, N, relu in zip(widths[:-1], widths[1:], relus):
        specs.append(dict(K=K, N=N, relu=relu, round_mode='RND', qf=torch.randint(2, 7, (K,), device=dev, generator=gen).float(),
                          wq=torch.randint(-48, 48, (K, N), device=dev, generator=gen).float() / 32,
                          bq=torch.randint(-16, 16, (N,), device=dev, generator=gen).float() / 16,
                          y=torch.empty(M, N, device=dev), absmax=torch.zeros(K, device=dev), dwq=torch.empty(K, N, device=dev),
                          dbq=torch.empty(N, device=dev), df=torch.empty(K, device=dev)))
    layers = kernels.dense_chain_layers(specs)
    gy = torch.randn(M, widths[-1], device=dev, generator=gen)
    out = {'kernel': 'k_dense_chain', 'widths': list(widths), 'batch': M}
    for name, fn in (('forward', lambda: kernels.dense_chain_fwd(x, layers, len(specs))),
                     ('backward', lambda: kernels.dense_chain_bwd(gy, x, None, layers, len(specs)))):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        out[name] = {'us': round(a.elapsed_time(b) / args.steps * 1e3, 2)}
    print(json.dumps(out), flush=True)


def run_qconv(args):
    """Kernel-level benchmark of the three convolution passes (forward, input gradient, weight gradient) on one layer of
    the small CNN (--layer 1..3: 32x32x4 -> 16, 15x15x16 -> 32, 6x6x32 -> 64 filters, 3x3 'valid', ReLU).
    Algorithmic bytes per output pixel: forward 4 (C' + N) with C' the input bytes per output pixel (H W C / (OH OW));
    input gradient 4 (N + C'); weight gradient 4 (3 N + C') (dY, y in; masked gradient out; image in)."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    B = args.batch or 4096
    H, C, N = {1: (32, 4, 16), 2: (15, 16, 32), 3: (6, 32, 64)}[args.layer]
    OH = H - 2
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randint(0, 32, (B, H, H, C), device=dev, generator=gen).float() / 32.0  # 5-bit activations: exact in bf16
    w = torch.randint(-64, 64, (3, 3, C, N), device=dev, generator=gen).float() / 64.0
    bq = torch.randint(-8, 8, (N,), device=dev, generator=gen).float() / 8.0
    gy = torch.randn(B, OH, OH, N, device=dev, generator=gen)
    wt = w.flip(0, 1).permute(0, 1, 3, 2).reshape(9 * N, C).contiguous()
    y = kernels.qconv2d_fwd(x, w.reshape(-1, N), bq, 'relu', 3, 3, (OH, OH), (1, 1), (1, 1), (0, 0))
    passes = {
        'forward': (lambda: kernels.qconv2d_fwd(x, w.reshape(-1, N), bq, 'relu', 3, 3, (OH, OH), (1, 1), (1, 1), (0, 0)),
                    4.0 * (H * H * C + OH * OH * N)),
        'input_gradient': (lambda: kernels.qconv2d_fwd(gy, wt, None, None, 3, 3, (H, H), (1, 1), (1, 1), (2, 2)),
                           4.0 * (H * H * C + OH * OH * N)),
        'weight_gradient': (lambda: kernels.qconv2d_wgrad(x, gy, y, 3, 3, (1, 1), (1, 1), (0, 0), True),
                            4.0 * (H * H * C + 3 * OH * OH * N)),
    }
    peak, kind = measured_peaks()
    out = {'kernel': 'qconv', 'layer': args.layer, 'batch': B, 'shape': [H, H, C, N], 'peak_GBs': peak, 'peak_source': kind}
    for name, (fn, bytes_per_sample) in passes.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        kernels.check_status(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        gbs = bytes_per_sample * B / (ms * 1e-3) / 1e9
        out[name] = {'ms': round(ms, 4), 'achieved_GBs': round(gbs, 1), 'frac': round(gbs / peak, 4)}
    print(json.dumps(out), flush=True)


def run_attn(args):
    """Kernel-level benchmark of the three per-head attention product kinds on the transformer block's shape:
    [batch, 64, 4 heads, 16] projections, [batch, 4, 64, 64] scores.  Algorithmic bytes per head: 4 (2 L D + L L)."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    B, L, H, D = args.batch or 8192, 64, 4, 16
    gen = torch.Generator(device=dev).manual_seed(0)
    q = torch.randint(-512, 512, (B, L, H, D), device=dev, generator=gen).float() / 64.0   # 10-bit projections
    k = torch.randint(-512, 512, (B, L, H, D), device=dev, generator=gen).float() / 64.0
    p = torch.randint(0, 256, (B, H, L, L), device=dev, generator=gen).float() / 256.0     # 8-bit probabilities
    g = torch.randn(B, H, L, L, device=dev, generator=gen)
    peak, kind = measured_peaks()
    out = {'kernel': 'k_attn_heads', 'batch': B, 'peak_GBs': peak, 'peak_source': kind}
    cases = {'scores (kind 0)': (0, q, k), 'context (kind 1)': (1, p, k), 'context, fp32 lhs (kind 1)': (1, g, k),
             'transposed (kind 2)': (2, g, q)}
    for name, (kd, x, y) in cases.items():
        fn = lambda: kernels.attn_heads_matmul(kd, x, y, B, L, H, D)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        kernels.check_status(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        gbs = 4.0 * (2 * L * D + L * L) * B * H / (ms * 1e-3) / 1e9
        out[name] = {'ms': round(ms, 4), 'achieved_GBs': round(gbs, 1), 'frac': round(gbs / peak, 4)}
    print(json.dumps(out), flush=True)


def run_bcast(args):
    """Kernel-level benchmark of the broadcast-layout quantizer kernels (bitwidths per activation position, shared over
    the batch): x [rows, P] with P = 4096 parameters (64 particles x 64 features), kif WRAP-training (round + abs-max)
    forward and SAT forward / backward.  Algorithmic bytes per element: forward 8, backward 12 (g, x in; dx out)."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    rows, Pn = (args.batch or 65536), 4096
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(rows, Pn, device=dev, generator=gen) * 4
    g = torch.randn(rows, Pn, device=dev, generator=gen)
    k = torch.randint(0, 2, (1, Pn), device=dev, generator=gen).to(torch.uint8)
    i = torch.randint(-2, 7, (1, Pn), device=dev, generator=gen).float()
    f = torch.randint(0, 9, (1, Pn), device=dev, generator=gen).float()
    peak, kind = measured_peaks()
    out = {'kernel': 'k_fwd_bcast / k_bwd_bcast', 'rows': rows, 'params': Pn, 'peak_GBs': peak, 'peak_source': kind}
    cases = {
        'fwd round + abs-max (WRAP training)': (lambda: kernels.quantize_fwd(x, None, None, f, 'RND', 'NONE', training=True, want_absmax=True), 8.0),
        'fwd SAT': (lambda: kernels.quantize_fwd(x, k, i, f, 'RND', 'SAT', training=True), 8.0),
        'bwd round only (dx, df)': (lambda: kernels.quantize_bwd(g, x, None, None, f, 'RND', 'NONE', want_di=False), 12.0),
        'bwd SAT (dx, di, df)': (lambda: kernels.quantize_bwd(g, x, k, i, f, 'RND', 'SAT'), 12.0),
    }
    for name, (fn, bpe) in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        gbs = bpe * rows * Pn / (ms * 1e-3) / 1e9
        out[name] = {'ms': round(ms, 4), 'achieved_GBs': round(gbs, 1), 'frac': round(gbs / peak, 4)}
    print(json.dumps(out), flush=True)


def run_qsoftmax(args):
    """Kernel-level benchmark of the fused quantised softmax (forward and backward) on the attention-score tensor of the
    transformer block: [batch, 4 heads, 64, 64] scores, softmax over the last axis, output bitwidth table [4 * 64, 64].
    Algorithmic bytes per score: 8 forward (s in, y out), 12 backward (s, dL/dy in, ds out)."""
    from hgq2_b200 import kernels

    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    B, L, rp = args.batch or 8192, 64, 256
    gen = torch.Generator(device=dev).manual_seed(0)
    s = torch.randn(B, 4, 64, L, device=dev, generator=gen) * 4
    gy = torch.randn(B, 4, 64, L, device=dev, generator=gen)
    one = lambda v, dt=torch.float32: torch.full((1,), v, dtype=dt, device=dev)
    k0, k1 = one(0, torch.uint8), one(1, torch.uint8)
    # the modes of the transformer block's layer in training: saturating table index, table outputs that saturate and round
    # half-even (what the layer forces them to), the two WRAP quantizers only round
    quants = [(k0, one(4.0), one(6.0), 'RND', 'SAT'), (k0, one(1.0), one(9.0), 'RND_CONV', 'SAT'), (None, None, one(3.0), 'RND', 'NONE'),
              (k0, one(1.0), one(9.0), 'RND_CONV', 'SAT'), (None, None, torch.full((rp * L,), 8.0, device=dev), 'RND', 'NONE')]
    fwd = lambda: kernels.qsoftmax_fwd(s, quants, 0.25, 1e-7, rp, True, True)
    bwd = lambda: kernels.qsoftmax_bwd(gy, s, quants, 0.25, 1e-7, rp, False)
    peak, kind = measured_peaks()
    out = {'kernel': 'k_qsoftmax', 'scores': s.numel(), 'peak_GBs': peak, 'peak_source': kind}
    for name, fn, bpe in (('fwd', fwd, 8), ('bwd', bwd, 12)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        gbs = bpe * s.numel() / (ms * 1e-3) / 1e9
        out[name] = {'ms': round(ms, 4), 'achieved_GBs': round(gbs, 1), 'frac': round(gbs / peak, 4)}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-cpu', action='store_true', help='skip the cpu_baseline leg')
    ap.add_argument('--no-qat', action='store_true', help='skip the QAT-step leg (training workloads)')
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer end-to-end leg')
    ap.add_argument('--qat-models', default='', help='comma-separated subset of the QAT-step models (default: all)')
    ap.add_argument('--elements', type=int, default=1 << 28,
                    help='total elements of the sweep (default 2^28; smaller values are for profiler captures)')
    ap.add_argument('--model', default='particle_tagger', help='model of --workload qat')
    ap.add_argument('--batch', type=int, default=0, help='batch of --workload qat (0 = the benchmark batch)')
    ap.add_argument('--workload', default='sweep', choices=['sweep', 'bcast', 'qdense', 'qdense_bwd', 'qsoftmax', 'qconv', 'attn', 'dense_chain', 'qat'],
                    help="'qdense' times the fused dense forward kernel alone (for profiler captures)")
    ap.add_argument('--layer', type=int, default=1, choices=[1, 2, 3], help='convolution layer of --workload qconv')
    ap.add_argument('--rows', type=int, default=1 << 22)
    ap.add_argument('--k', type=int, default=64)
    ap.add_argument('--n', type=int, default=64)
    ap.add_argument('--rows-period', type=int, default=64)
    ap.add_argument('--pool-rows', type=int, default=0, help="--workload qdense: also produce the sums over groups of this many rows")
    args = ap.parse_args()
    globals()['TOTAL_ELEMS'] = args.elements
    if args.workload == 'qdense':
        return run_qdense(args)
    if args.workload == 'qat':
        return run_qat_single(args)
    if args.workload == 'qdense_bwd':
        return run_qdense_bwd(args)
    if args.workload == 'bcast':
        return run_bcast(args)
    if args.workload == 'dense_chain':
        run_dense_chain(args)
        return
    if args.workload == 'qconv':
        return run_qconv(args)
    if args.workload == 'attn':
        return run_attn(args)
    if args.workload == 'qsoftmax':
        return run_qsoftmax(args)
    if args.impl == 'reference':
        run_reference(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
