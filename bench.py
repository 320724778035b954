"""Benchmark of the B200 MicroAdam step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama3_8b|gpt2_flat|sweep] [--impl ours|reference]

One "step" is one MicroAdam optimizer step over the whole synthetic model with that step's
gradients already resident in HBM.  The default workload is the Llama-3-8B-shaped bf16 parameter
list (290 tensors, 8 030 257 152 parameters; m=10, k_init=0.01, quant_block_size=64,
weight_decay=0.1) on one GPU.  With N > 1 (launched by torch.distributed.run, one rank per GPU) the
same model is sharded over the N GPUs (strong scaling); by default (`--exchange rows`) the error
feedback and the top-k selection are sharded, the ranks all-gather the window row the step produced
and every rank applies the update to all parameters; `--exchange params` shards both kernels ZeRO-1
style and all-gathers the updated parameters instead.  Rank 0 prints one JSON line.  At N = 1 the line
also carries a `configs.gpt2_flat` record (the fp32 single-GPU configuration) and a
`configs.llama3_8b_quant_block_100000` record (the list with the reference README's quant_block_size), at N > 1 a
`params_mode` record (the same model with the parameter all-gather) and the time of the gradient
reduce-scatter of the shard plan; `param_checksum` is a checksum of all parameters that is equal for
every N exactly when the N-GPU run is bit-identical to the 1-GPU run.  `e2e` is the same step with its
gradients coming from pinned host memory (the copy of the next step's gradients overlaps the current step,
both inside the timed region) and a checksum of all parameters read back every step.

`--workload sweep` times one fp32 flat tensor over the grid d x k_init x m x quant_block_size and
prints per-kernel and per-step GB/s for every point.

`--impl reference` times the CPU oracle (the restatement of the reference's torch-level step, all
host threads) on a bounded sample of the same workload instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, 'ista-daslab-optimizers_b200')):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HYPER = dict(m=10, lr=1e-3, k_init=0.01, quant_block_size=64, betas=(0.9, 0.999), eps=1e-8, alpha=0)
FALLBACK_HBM_GBS = 6650.0      # copy bandwidth assumed when no measured peak file is present
METRIC = 'microadam_step_throughput'
UNIT = 'Gparams/s'

# DRAM bytes per parameter and launch (ncu: dram__bytes_read.sum + dram__bytes_write.sum) captured on a
# 134 217 728-element (bf16) / 67 108 864-element (fp32) flat tensor and scaled to the workload by its
# parameter count (traffic grows in proportion to the elements a launch covers).  None = not captured.
NCU_TRAFFIC_BYTES_PER_PARAM = {
    ('ef_topk_quant', 'bf16'): 3.06, ('window_adam', 'bf16'): 4.14,
    ('ef_topk_quant', 'f32'): 5.03, ('window_adam', 'f32'): 6.49,
}


def workload_spec(name: str):
    from ista_daslab_optimizers_b200 import synthetic as S
    if name == 'llama3_8b':
        return dict(shapes=S.llama3_8b_shapes(), dtype=torch.bfloat16, weight_decay=0.1, grad_sigma=1e-4,
                    label='Llama-3-8B-shaped bf16 parameter list, 290 tensors, weight_decay=0.1')
    if name == 'gpt2_flat':
        return dict(shapes=[(124439808,)], dtype=torch.float32, weight_decay=0.0, grad_sigma=1e-3,
                    label='one fp32 flat parameter of 124,439,808 elements (GPT-2-small size)')
    if name.startswith('flat_'):
        # flat_<bf16|f32>_<numel>: one flat tensor, for ncu captures on a case a few times larger than L2
        _, dt, numel = name.split('_')
        dtype = torch.bfloat16 if dt == 'bf16' else torch.float32
        return dict(shapes=[(int(numel),)], dtype=dtype, weight_decay=0.1 if dtype == torch.bfloat16 else 0.0,
                    grad_sigma=1e-4 if dtype == torch.bfloat16 else 1e-3, label=f'one flat {dt} parameter of {int(numel)} elements')
    raise SystemExit(f'unknown workload {name}')


def algorithmic_bytes_per_param(dtype, rows: float, k_init: float = None, qbs: int = None):
    """HBM bytes per parameter the step cannot avoid, split by kernel: gradient read, one nibble
    of error feedback in and out, bf16 min+max in and out, one (index, value) row out;
    then `rows` window rows in, parameter in and out."""
    e = 2 if dtype == torch.bfloat16 else 4
    qbs = HYPER['quant_block_size'] if qbs is None else qbs
    k = HYPER['k_init'] if k_init is None else k_init
    a = e + 1.0 + 8.0 / qbs + 4.0 * k
    b = 4.0 * rows * k + 2.0 * e
    return a, b


def measured_hbm_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return FALLBACK_HBM_GBS, 'fallback'


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""
    REASONS = {0x1: 'gpu_idle', 0x2: 'applications_clocks_setting', 0x4: 'sw_power_cap', 0x8: 'hw_slowdown',
               0x10: 'sync_boost', 0x20: 'sw_thermal_slowdown', 0x40: 'hw_thermal_slowdown',
               0x80: 'hw_power_brake_slowdown', 0x100: 'display_clock_setting'}

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_flag = threading.Event()
        self.error = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get('CUDA_VISIBLE_DEVICES')
            idx = self.index
            if visible:
                ids = [v for v in visible.split(',') if v.strip()]
                if self.index < len(ids) and ids[self.index].strip().isdigit():
                    idx = int(ids[self.index])
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop_flag.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in self.REASONS.items():
                    if mask & bit and name != 'gpu_idle':
                        self.reasons.add(name)
                time.sleep(self.period)
        except Exception as e:  # NVML missing or refused: report it, the bench itself goes on
            self.error = repr(e)

    def stop(self):
        self._stop_flag.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        out = {'sm_mhz': s[len(s) // 2] if s else None, 'sm_max_mhz': self.max_mhz, 'reasons': sorted(self.reasons)}
        if self.error:
            out['error'] = self.error
        return out


# ----------------------------------------------------------------------------------- CPU oracle arm

def cpu_oracle_rate(spec, steps: int, warmup: int):
    """Gparams/s of the CPU oracle on a bounded sample of the workload: the first transformer
    layer's attention projections and norm for the Llama list, a 16 Mi slice for the flat tensor."""
    from oracle.microadam_oracle import MicroAdamOracle
    from ista_daslab_optimizers_b200 import synthetic as S
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    if len(spec['shapes']) > 1:
        shapes = spec['shapes'][1:5] + spec['shapes'][8:9]
        sample = 'layer 0 of the list: q [4096,4096], k, v [1024,4096], o [4096,4096], one RMSNorm [4096]'
    else:
        shapes = [(16 * 1024 * 1024,)]
        sample = 'a 16 Mi-element slice of the flat tensor'
    params = [S.normal_tensor(0, 100 + i, int(torch.Size(s).numel()), 0.02, spec['dtype']).view(s) for i, s in enumerate(shapes)]
    grads = [S.normal_tensor(1, 100 + i, p.numel(), spec['grad_sigma'], spec['dtype']).view(p.shape) for i, p in enumerate(params)]
    opt = MicroAdamOracle(params, m=HYPER['m'], lr=HYPER['lr'], quant_block_size=HYPER['quant_block_size'],
                          k_init=HYPER['k_init'], alpha=HYPER['alpha'], betas=HYPER['betas'],
                          weight_decay=spec['weight_decay'], eps=HYPER['eps'])
    n = sum(p.numel() for p in params)
    times = []
    for t in range(warmup + steps):
        gs = [g.clone() for g in grads]
        t0 = time.perf_counter()
        opt.step(gs)
        dt = time.perf_counter() - t0
        if t >= warmup:
            times.append(dt)
    med = sorted(times)[len(times) // 2]                      # median step
    return n / med / 1e9, threads, sample, med * 1e3, n


def headline_config(spec, n_params, world, exchange, grad_sets):
    """The `config` object of the JSON line (the same for both arms)."""
    return {'workload': spec['label'], 'params': n_params, 'parallelism': parallelism_label(world, exchange),
            'l2_policy': 'inputs larger than L2 (GBs per step vs 126 MB)', 'grad_sets': grad_sets,
            'arithmetic': 'fp32 on bf16/fp32 storage, 4-bit codes', **{k: v for k, v in HYPER.items() if k != 'betas'},
            'weight_decay': spec['weight_decay']}


def reference_arm(args, spec):
    """The reference's CPU path (the oracle port: the reference's own step needs native modules that are not part
    of its tree) on all host threads; every step is one step over a bounded sample of the workload."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    steps = min(max(1, args.steps), 200)
    warmup = max(3, args.warmup)
    rate, threads, sample, ms, n = cpu_oracle_rate(spec, steps, warmup)
    world = args.gpus
    exchange = args.exchange if (world > 1 and HYPER['alpha'] == 0) else 'params'
    n_params = sum(int(torch.Size(s).numel()) for s in spec['shapes'])
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': rate, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': steps,
        'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': 'bf16' if spec['dtype'] == torch.bfloat16 else 'f32', 'data': 'synthetic',
        'config': headline_config(spec, n_params, world, exchange, max(1, args.grad_sets)),
        'cpu_baseline': {'value': rate, 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': sample, 'sample_params': n,
                         'timing': f'median of {steps} steps after {warmup} warm-up steps, each over the sample'},
        'e2e': {'value': rate, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------- roofline sweep

def sweep(args):
    """One fp32 flat tensor over d x k_init x m x quant_block_size; gradients ~N(0, 1e-3), seed 1; timed at steady
    state (after m + 2 steps, so that the window is full); GB/s per kernel and per step from CUDA events."""
    from ista_daslab_optimizers_b200 import MicroAdam
    assert torch.cuda.is_available(), 'the sweep needs a CUDA device'
    device = torch.device('cuda', 0)
    torch.cuda.set_device(device)
    peak, peak_kind = measured_hbm_peak()
    points = []
    gen = torch.Generator(device=device)
    for log2d in (20, 24, 28, 31):
        if log2d > args.sweep_max_log2:
            continue
        d = 1 << log2d
        gen.manual_seed(1)
        grads = [torch.empty(d, device=device).normal_(0, 1e-3, generator=gen) for _ in range(2)]
        for qbs in (32, 64, 100000):
            for m in (5, 10, 20):
                for k_init in (0.005, 0.01, 0.05):
                    gen.manual_seed(2)
                    p = torch.nn.Parameter(torch.empty(d, device=device).normal_(0, 0.02, generator=gen), requires_grad=False)
                    opt = MicroAdam([p], m=m, lr=1e-3, quant_block_size=qbs, k_init=k_init, alpha=0, weight_decay=0.0)
                    warm = m + 2
                    timed = 3 if log2d >= 28 else 10
                    for t in range(warm):
                        p.grad = grads[t % 2].clone() if qbs == 100000 else grads[t % 2]
                        opt.step()
                    fused = all(e.fused for e in opt._entries)
                    opt.kernel_events = [] if fused else None
                    # the operator-level path and the fused path for loose quantisation blocks overwrite p.grad
                    scratch = [grads[t % 2].clone() for t in range(timed)] if (not fused or qbs == 100000) else None
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for t in range(timed):
                        p.grad = scratch[t] if scratch is not None else grads[t % 2]
                        opt.step()
                    e1.record()
                    torch.cuda.synchronize()
                    ms = e0.elapsed_time(e1) / timed
                    ba, bb = algorithmic_bytes_per_param(torch.float32, m, k_init, qbs)
                    rec = {'d': d, 'log2_d': log2d, 'k_init': k_init, 'm': m, 'quant_block_size': qbs,
                           'path': ('fused' if qbs != 100000 else 'fused, kernel A in two parts') if fused else 'operators', 'ms_per_step': ms,
                           'step_gbs': d * (ba + bb) / (ms * 1e-3) / 1e9, 'step_frac': d * (ba + bb) / (ms * 1e-3) / 1e9 / peak}
                    if fused:
                        ev = [e for e in opt.kernel_events if isinstance(e, list)]
                        ta = sum(e[0].elapsed_time(e[1]) for e in ev) / timed
                        tb = sum(e[1].elapsed_time(e[2]) for e in ev) / timed
                        rec['kernels'] = [{'kernel': 'ef_topk_quant', 'ms': ta, 'gbs': d * ba / (ta * 1e-3) / 1e9, 'frac': d * ba / (ta * 1e-3) / 1e9 / peak},
                                          {'kernel': 'window_adam', 'ms': tb, 'gbs': d * bb / (tb * 1e-3) / 1e9, 'frac': d * bb / (tb * 1e-3) / 1e9 / peak}]
                    points.append(rec)
                    del opt, p, scratch
        del grads
        torch.cuda.empty_cache()
    print(json.dumps({'metric': 'microadam_step_hbm_sweep', 'unit': 'GB/s', 'peak': peak, 'peak_kind': f'of {peak_kind}', 'dtype': 'f32',
                      'data': 'synthetic', 'config': {'workload': 'one fp32 flat tensor: d x k_init x m x quant_block_size, weight_decay=0, alpha=0'},
                      'points': points}))


# ----------------------------------------------------------------------------------- GPU arm

def make_flat_model(spec, device, seed):
    """Parameters as views of one flat buffer (each view 256-byte aligned), filled ~N(0, 0.02)."""
    es = torch.tensor([], dtype=spec['dtype']).element_size()
    align = 256 // es
    offsets, total = [], 0
    for s in spec['shapes']:
        offsets.append(total)
        total += -(-int(torch.Size(s).numel()) // align) * align
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    flat = torch.empty(total, dtype=spec['dtype'], device=device)
    flat.normal_(0.0, 0.02, generator=gen)
    params = [torch.nn.Parameter(flat[o:o + int(torch.Size(s).numel())].view(s), requires_grad=False)
              for o, s in zip(offsets, spec['shapes'])]
    return flat, params, offsets


def make_flat_grads(spec, offsets, total, device, seed):
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    flat = torch.empty(total, dtype=spec['dtype'], device=device)
    flat.normal_(0.0, spec['grad_sigma'], generator=gen)
    return flat, [flat[o:o + int(torch.Size(s).numel())].view(s) for o, s in zip(offsets, spec['shapes'])]


def build_optimizer(spec, params, world, exchange):
    from ista_daslab_optimizers_b200 import MicroAdam
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam
    kw = dict(m=HYPER['m'], lr=HYPER['lr'], quant_block_size=HYPER['quant_block_size'], k_init=HYPER['k_init'],
              alpha=HYPER['alpha'], betas=HYPER['betas'], weight_decay=spec['weight_decay'], eps=HYPER['eps'])
    return ShardedMicroAdam(params, exchange=exchange, **kw) if world > 1 else MicroAdam(params, **kw)


def parallelism_label(world, exchange):
    if world == 1:
        return 'single'
    if exchange == 'rows':
        return f'shard{world}: kernel A sharded, window rows all-gathered, kernel B replicated'
    return f'zero1-shard{world}: both kernels sharded, updated parameters all-gathered'


def whole_buffer_checksum(flat_p):
    """Wrapping 64-bit sum of the parameter buffer's bit patterns: exact, order-independent, equal on every rank and
    for every world size exactly when the parameters are bit-identical."""
    words = flat_p.view(torch.int16) if flat_p.element_size() == 2 else flat_p.view(torch.int32)
    return int(words.sum(dtype=torch.int64).item())


def run_workload(spec, args, world, rank, local_rank, exchange, steps, warmup, e2e_steps, plain_tail_steps=0):
    """Builds the synthetic model, runs warm-up + timed steps + the end-to-end steps and returns the measurements
    (max over ranks) as a dictionary.  `plain_tail_steps` more steps on the end-to-end steps' gradients (already
    on the device) follow, so that a run without end-to-end steps ends on the same step count and parameters."""
    import torch.distributed as dist
    from ista_daslab_optimizers_b200 import _native
    device = torch.device('cuda', local_rank)
    flat_p, params, offsets = make_flat_model(spec, device, args.seed)
    grad_sets = [make_flat_grads(spec, offsets, flat_p.numel(), device, args.seed + 1 + i) for i in range(max(1, args.grad_sets))]
    n_params = sum(p.numel() for p in params)
    opt = build_optimizer(spec, params, world, exchange)

    def set_grads(t):
        for p, g in zip(params, grad_sets[t % len(grad_sets)][1]):
            p.grad = g

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for t in range(warmup):
        set_grads(t)
        opt.step()
    barrier()

    # ---- timed region: K steps, inputs resident in HBM ------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    opt.kernel_events = []
    launches0 = _native.kernel_launch_count()
    rows_per_step = [min(opt.steps + 1 + i, HYPER['m']) for i in range(steps)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for t in range(steps):
        set_grads(warmup + t)
        opt.step()
    end.record()
    barrier()
    clocks = sampler.stop()
    launches = _native.kernel_launch_count() - launches0
    elapsed_ms = start.elapsed_time(end)
    events, opt.kernel_events = opt.kernel_events, None
    calls = [ev for ev in events if isinstance(ev, list)]            # one per fused call (several per step when overlapped)
    t_a = sum(ev[0].elapsed_time(ev[1]) for ev in calls) / steps
    t_b = sum(ev[1].elapsed_time(ev[2]) for ev in calls) / steps
    rows_calls = [ev[1] for ev in events if isinstance(ev, tuple) and ev[0] == 'rows']   # [start, after A, after exchange, after B]
    t_a += sum(ev[0].elapsed_time(ev[1]) for ev in rows_calls) / steps
    t_b += sum(ev[2].elapsed_time(ev[3]) for ev in rows_calls) / steps
    # exchange time that is not hidden behind the kernels: step time minus kernel time
    t_gather = max(0.0, elapsed_ms / steps - t_a - t_b) if world > 1 else 0.0
    stats = torch.tensor([elapsed_ms, t_a, t_b, t_gather], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    elapsed_ms, t_a, t_b, t_gather = stats.tolist()

    # ---- the gradient side of the shard plan (N > 1): every range summed into its owner, timed on its own -----------
    reduce_ms = None
    if world > 1 and args.time_grad_reduce:
        scratch = torch.zeros_like(grad_sets[0][0])
        views = [scratch[o:o + p.numel()].view(p.shape) for o, p in zip(offsets, params)]
        from ista_daslab_optimizers_b200.sharding import reduce_to_owners
        for _ in range(2):
            reduce_to_owners(opt.plan, views, opt.rank, world, None, average=True)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(3):
            reduce_to_owners(opt.plan, views, opt.rank, world, None, average=True)
        r1.record()
        barrier()
        red = torch.tensor([r0.elapsed_time(r1) / 3], dtype=torch.float64, device=device)
        dist.all_reduce(red, op=dist.ReduceOp.MAX)
        reduce_ms = red.item()
        del scratch, views

    # ---- end to end: gradients start in pinned host memory, a checksum of all parameters comes back ---------------
    my_lo, my_hi = 0, flat_p.numel()
    if world > 1:
        mine = [(offsets[pc.index] + pc.lo, offsets[pc.index] + pc.hi) for pc in opt.plan if pc.rank == opt.rank]
        my_lo, my_hi = min(a for a, _ in mine), max(b for _, b in mine)
    gflat = grad_sets[0][0]
    try:
        host = torch.empty(my_hi - my_lo, dtype=spec['dtype'], pin_memory=True)
        host.copy_(gflat[my_lo:my_hi])
        chunked = False
    except RuntimeError:
        host = torch.empty(min(my_hi - my_lo, 1 << 29), dtype=spec['dtype'], pin_memory=True)
        host.copy_(gflat[my_lo:my_lo + host.numel()])
        chunked = True
    set_grads(0)
    h2d_bytes = (my_hi - my_lo) * gflat.element_size()
    # The copy of step t + 1's gradients runs on its own stream while step t computes (two device buffers, the
    # second gradient set's storage): every step's copy lies inside the timed region, the first one exposed.
    pipelined = len(grad_sets) >= 2
    copy_stream = torch.cuda.Stream(device=device) if pipelined else None
    compute = torch.cuda.current_stream(device)

    def copy_in(dst):
        if not chunked:
            dst[my_lo:my_hi].copy_(host, non_blocking=True)
        else:
            for o in range(my_lo, my_hi, host.numel()):
                n = min(host.numel(), my_hi - o)
                dst[o:o + n].copy_(host[:n], non_blocking=True)

    def copy_in_async(dst, after):
        """Enqueues the copy on the copy stream once `after` (the last step that read `dst`) has passed."""
        with torch.cuda.stream(copy_stream):
            if after is not None:
                copy_stream.wait_event(after)
            copy_in(dst)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return ev

    barrier()
    t0 = time.perf_counter()
    checksum = None
    if pipelined:
        read_done = [None, None]                       # per buffer: the event after the last step that read it
        ready = copy_in_async(grad_sets[0][0], None)
        for t in range(e2e_steps):
            cur = t % 2
            compute.wait_event(ready)
            set_grads(cur)
            if t + 1 < e2e_steps:
                ready = copy_in_async(grad_sets[1 - cur][0], read_done[1 - cur])
            opt.step()
            read_done[cur] = torch.cuda.Event()
            read_done[cur].record(compute)
            checksum = whole_buffer_checksum(flat_p)                   # 8-byte device-to-host read, synchronises
        set_grads(0)
    else:
        for t in range(e2e_steps):
            copy_in(gflat)
            opt.step()
            checksum = whole_buffer_checksum(flat_p)                   # 8-byte device-to-host read, synchronises
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    for _ in range(plain_tail_steps):
        opt.step()
        checksum = None
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    if checksum is None:
        checksum = whole_buffer_checksum(flat_p)
    if world > 1:
        # every rank must hold the same parameters: a mismatch is a correctness failure, not a number to report
        lohi = torch.tensor([checksum, -checksum], dtype=torch.int64, device=device)
        dist.all_reduce(lohi, op=dist.ReduceOp.MIN)
        if lohi[0].item() != -lohi[1].item():
            raise SystemExit(f'rank {rank}: parameter checksums differ between the ranks ({lohi[0].item()} .. {-lohi[1].item()})')
    out = dict(n_params=n_params, steps=steps, elapsed_ms=elapsed_ms, t_a=t_a, t_b=t_b, t_gather=t_gather, launches=launches,
               clocks=clocks, rows_avg=sum(rows_per_step) / len(rows_per_step), reduce_ms=reduce_ms,
               e2e_value=(n_params * e2e_steps / e2e_s.item() / 1e9 if e2e_steps else None), e2e_steps=e2e_steps,
               h2d_bytes=h2d_bytes, checksum=checksum, optimizer_steps=opt.steps, exchange=exchange,
               device_error=_native.device_error())
    del opt, params, grad_sets, flat_p, gflat, host
    torch.cuda.empty_cache()
    return out


def loose_blocks_record(spec, args, local_rank, steps, qbs=100000):
    """The same workload with the quant_block_size of the reference's README (100000): quantisation blocks then
    ignore the borders of the top-k blocks and kernel A runs in two parts, which leave the residual in the gradient
    buffers.  Every step therefore starts from a device-to-device copy of the gradients, which is outside the
    kernel times reported here (`ms_per_step` is the sum of the step's kernels)."""
    from ista_daslab_optimizers_b200 import MicroAdam
    device = torch.device('cuda', local_rank)
    flat_p, params, offsets = make_flat_model(spec, device, args.seed)
    gflat, gviews = make_flat_grads(spec, offsets, flat_p.numel(), device, args.seed + 1)
    pristine = gflat.clone()
    opt = MicroAdam(params, m=HYPER['m'], lr=HYPER['lr'], quant_block_size=qbs, k_init=HYPER['k_init'], alpha=HYPER['alpha'],
                    betas=HYPER['betas'], weight_decay=spec['weight_decay'], eps=HYPER['eps'])
    for p, g in zip(params, gviews):
        p.grad = g
    for _ in range(HYPER['m'] + 2):
        gflat.copy_(pristine)
        opt.step()
    torch.cuda.synchronize()
    opt.kernel_events = []
    for _ in range(steps):
        gflat.copy_(pristine)
        opt.step()
    torch.cuda.synchronize()
    ev = [e for e in opt.kernel_events if isinstance(e, list)]
    t_a = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    t_b = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    n = sum(p.numel() for p in params)
    es = 2 if spec['dtype'] == torch.bfloat16 else 4
    peak, kind = measured_hbm_peak()
    ba = 3.0 * es + 1.0 + 4.0 * HYPER['k_init']          # gradient in, residual out and in again, one nibble in and out, one row out
    bb = 4.0 * HYPER['m'] * HYPER['k_init'] + 2.0 * es
    return {'workload': spec['label'], 'quant_block_size': qbs, 'path': 'fused' if all(e.fused for e in opt._entries) else 'operators',
            'value': n / ((t_a + t_b) * 1e-3) / 1e9, 'unit': UNIT, 'ms_per_step': t_a + t_b, 'timing': 'sum of the kernels of a step',
            'kernels': [{'kernel': 'ef_topk_quant (two launches: selection + residual, statistics + codes)', 'ms': t_a,
                         'algorithmic_bytes_per_param': ba, 'gbs': n * ba / (t_a * 1e-3) / 1e9, 'frac': n * ba / (t_a * 1e-3) / 1e9 / peak},
                        {'kernel': 'window_adam', 'ms': t_b, 'algorithmic_bytes_per_param': bb,
                         'gbs': n * bb / (t_b * 1e-3) / 1e9, 'frac': n * bb / (t_b * 1e-3) / 1e9 / peak}],
            'peak_kind': f'of {kind}', 'steps': steps}


def kernel_records(spec, r, world):
    """Per-kernel roofline figures from a run_workload result."""
    peak, _ = measured_hbm_peak()
    ba, bb = algorithmic_bytes_per_param(spec['dtype'], r['rows_avg'])
    per_rank = r['n_params'] / world
    # parameters one rank's launch of each kernel covers: kernel B runs over all of them when window rows are exchanged
    params_a, params_b = per_rank, (r['n_params'] if (world > 1 and r['exchange'] == 'rows') else per_rank)
    dt = 'bf16' if spec['dtype'] == torch.bfloat16 else 'f32'
    kernels = []
    for name, b, ms, np_k in (('ef_topk_quant', ba, r['t_a'], params_a), ('window_adam', bb, r['t_b'], params_b)):
        gbs = np_k * b / (ms * 1e-3) / 1e9
        tr = NCU_TRAFFIC_BYTES_PER_PARAM.get((name, dt))
        kernels.append({'kernel': name, 'ms': ms, 'algorithmic_bytes': np_k * b, 'achieved_gbs': gbs,
                        'frac': gbs / peak, 'traffic': None if tr is None else tr * np_k})
    step_gbs = (params_a * ba + params_b * bb) / ((r['t_a'] + r['t_b']) * 1e-3) / 1e9
    step = {'achieved_gbs': step_gbs, 'frac': step_gbs / peak, 'frac_of_8tbs_nominal': step_gbs / 8000.0,
            'algorithmic_bytes_per_param': ba + bb, 'kernel_ms': r['t_a'] + r['t_b'], 'exposed_exchange_ms': r['t_gather']}
    return kernels, step


def roofline_record(kernels):
    peak, peak_kind = measured_hbm_peak()
    dom = max(kernels, key=lambda k: k['ms'])
    return {'bound': 'hbm', 'kernel': dom['kernel'], 'achieved': dom['achieved_gbs'], 'peak': peak, 'unit': 'GB/s',
            'frac': dom['frac'], 'traffic': dom['traffic'], 'peak_kind': f'of {peak_kind}',
            'frac_of_8tbs_nominal': dom['achieved_gbs'] / 8000.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='llama3_8b', help='llama3_8b | gpt2_flat | flat_<bf16|f32>_<numel> | loose_<one of those> | sweep')
    ap.add_argument('--grad-sets', type=int, default=2, help='distinct pre-generated gradient sets cycled over the steps')
    ap.add_argument('--e2e-steps', type=int, default=5)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extra', action='store_true',
                    help='only the headline workload: no GPT-2-flat sub-record (N = 1), no parameter-exchange sub-record (N > 1)')
    ap.add_argument('--no-grad-reduce', dest='time_grad_reduce', action='store_false',
                    help='N > 1: do not time the gradient reduce-scatter of the shard plan')
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--exchange', default='rows', choices=['rows', 'params'],
                    help='N > 1: what the ranks exchange (window rows, or updated parameters)')
    ap.add_argument('--sweep-max-log2', type=int, default=31, help='sweep: largest tensor is 2^this elements')
    ap.add_argument('--quant-block-size', type=int, default=None,
                    help='quant_block_size of the headline workload (default 64).  Values that are no power of two in [8, 128] '
                         'take the path that leaves the residual in the gradient buffers: later steps then see those as gradients, '
                         'which is fine for timing and profiling a kernel, not for the parameter checksum')
    args = ap.parse_args()
    if args.quant_block_size is not None:
        HYPER['quant_block_size'] = args.quant_block_size
    if args.workload == 'sweep':
        sweep(args)
        return
    if args.workload.startswith('loose_'):
        # loose_<workload>: the kernels for quantisation blocks that ignore top-k block borders (quant_block_size
        # 100000 unless --quant-block-size says otherwise), every step on freshly restored gradients; one GPU
        assert torch.cuda.is_available(), 'bench.py needs a CUDA device'
        torch.cuda.set_device(0)
        rec = loose_blocks_record(workload_spec(args.workload[len('loose_'):]), args, 0, max(1, args.steps),
                                  qbs=args.quant_block_size or 100000)
        print(json.dumps({'metric': METRIC, 'unit': UNIT, 'data': 'synthetic', **rec}))
        return
    spec = workload_spec(args.workload)
    if args.impl == 'reference':
        reference_arm(args, spec)
        return

    import torch.distributed as dist

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 with torch.distributed.run')
    assert torch.cuda.is_available(), 'bench.py needs a CUDA device: there is no CPU implementation to time'
    device = torch.device('cuda', local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    e2e_steps = max(0, min(args.e2e_steps, steps))
    exchange = args.exchange if (world > 1 and HYPER['alpha'] == 0) else 'params'

    r = run_workload(spec, args, world, rank, local_rank, exchange, steps, warmup, e2e_steps)
    extra = {}
    if not args.no_extra and args.workload == 'llama3_8b':
        if world == 1:
            # the single-GPU fp32 configuration (GPT-2-small-sized flat tensor), with its own roofline
            spec2 = workload_spec('gpt2_flat')
            r2 = run_workload(spec2, args, 1, rank, local_rank, 'params', steps, warmup, 0)
            k2, step2 = kernel_records(spec2, r2, 1)
            extra['configs'] = {'gpt2_flat': {
                'workload': spec2['label'], 'value': r2['n_params'] * steps / (r2['elapsed_ms'] * 1e-3) / 1e9, 'unit': UNIT,
                'ms_per_step': r2['elapsed_ms'] / steps, 'dtype': 'f32', 'kernels': k2, 'step_hbm': step2,
                'roofline': roofline_record(k2), 'gpu_launches': r2['launches'], 'checksum': r2['checksum']}}
            del r2
            torch.cuda.empty_cache()
            # the headline list with the quant_block_size of the reference's README
            extra['configs']['llama3_8b_quant_block_100000'] = loose_blocks_record(spec, args, local_rank, min(steps, 10))
        elif exchange == 'rows':
            # the dense alternative: both kernels sharded ZeRO-1 style, updated parameters all-gathered
            r2 = run_workload(spec, args, world, rank, local_rank, 'params', steps, warmup, 0, plain_tail_steps=e2e_steps)
            k2, step2 = kernel_records(spec, r2, world)
            extra['params_mode'] = {
                'parallelism': parallelism_label(world, 'params'), 'value': r2['n_params'] * steps / (r2['elapsed_ms'] * 1e-3) / 1e9,
                'unit': UNIT, 'ms_per_step': r2['elapsed_ms'] / steps, 'kernels': k2, 'step_hbm': step2,
                'param_checksum': {'value': r2['checksum'], 'optimizer_steps': r2['optimizer_steps']}}
            if r2['checksum'] != r['checksum']:
                raise SystemExit(f"rank {rank}: the two exchange modes ended with different parameters "
                                 f"({r['checksum']} vs {r2['checksum']})")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel and the whole step ---------------------------------------------
    n_params = r['n_params']
    value = n_params * steps / (r['elapsed_ms'] * 1e-3) / 1e9
    kernels, step_hbm = kernel_records(spec, r, world)
    dt = 'bf16' if spec['dtype'] == torch.bfloat16 else 'f32'
    line = {
        'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': r['elapsed_ms'] / steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': dt, 'data': 'synthetic',
        'config': headline_config(spec, n_params, world, exchange, max(1, args.grad_sets)),
        'roofline': roofline_record(kernels),
        'kernels': kernels,
        'step_hbm': step_hbm,
        'e2e': {'value': r['e2e_value'], 'unit': UNIT, 'h2d_bytes_per_step': r['h2d_bytes'], 'd2h_bytes_per_step': 8,
                'steps': e2e_steps,
                'copies': 'step t + 1 copied from pinned host memory on a second stream while step t computes; all inside the timed region'},
        # wrapping 64-bit sum of all parameter bit patterns after `optimizer_steps` steps: identical on every rank
        # (checked) and for every N exactly when the N-GPU parameters equal the 1-GPU ones bit for bit
        'param_checksum': {'value': r['checksum'], 'optimizer_steps': r['optimizer_steps']},
        'gpu_launches': r['launches'],
        'device_error': r['device_error'],
        'clocks': r['clocks'],
    }
    if r['reduce_ms'] is not None:
        grad_bytes = n_params * (2 if spec['dtype'] == torch.bfloat16 else 4)
        line['grad_reduce_scatter'] = {'ms': r['reduce_ms'], 'bytes_per_rank_in': grad_bytes * (world - 1) / world,
                                       'note': 'gradient side of the shard plan, timed on its own, not part of value'}
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        rate, threads, sample, ms, n = cpu_oracle_rate(spec, steps=10, warmup=2)
        line['cpu_baseline'] = {'value': rate, 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': sample,
                                'ms_per_step': ms, 'sample_params': n, 'timing': 'median of 10 steps after 2 warm-up steps'}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
