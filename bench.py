"""Benchmark of the B200 MicroAdam step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llama3_8b|gpt2_flat] [--impl ours|reference]

One "step" is one MicroAdam optimizer step over the whole synthetic model with that step's
gradients already resident in HBM.  The default workload is the Llama-3-8B-shaped bf16 parameter
list (290 tensors, 8 030 257 152 parameters; m=10, k_init=0.01, quant_block_size=64,
weight_decay=0.1) on one GPU; with N > 1 (launched by torch.distributed.run, one rank per GPU) the
same model is sharded ZeRO-1 style over the N GPUs and the updated parameters are all-gathered
after every step (strong scaling).  Rank 0 prints one JSON line.

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
FALLBACK_HBM_GBS = 6650.0      # earlier measurement on this pool, used when MEASURED_PEAKS.json is absent
METRIC = 'microadam_step_throughput'
UNIT = 'Gparams/s'

# DRAM bytes per parameter and launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum)
# on a smaller case of the same kernel and scaled by the parameter count; see profiles/.  None = not captured.
NCU_TRAFFIC_BYTES_PER_PARAM = {
    ('ef_topk_quant', 'bf16'): 3.06, ('window_adam', 'bf16'): 4.14,
    ('ef_topk_quant', 'f32'): 5.03, ('window_adam', 'f32'): 6.49,
}


def workload_spec(name: str):
    from ista_daslab_optimizers_b200 import synthetic as S
    if name == 'llama3_8b':
        return dict(shapes=S.llama3_8b_shapes(), dtype=torch.bfloat16, weight_decay=0.1, grad_sigma=1e-4,
                    label='Llama-3-8B-shaped bf16 parameter list, 290 tensors, weight_decay=0.1 (BASELINE config 3)')
    if name == 'gpt2_flat':
        return dict(shapes=[(124439808,)], dtype=torch.float32, weight_decay=0.0, grad_sigma=1e-3,
                    label='one fp32 flat parameter of 124,439,808 elements (BASELINE config 2)')
    if name.startswith('flat_'):
        # flat_<bf16|f32>_<numel>: one flat tensor, for ncu captures on a case a few times larger than L2
        _, dt, numel = name.split('_')
        dtype = torch.bfloat16 if dt == 'bf16' else torch.float32
        return dict(shapes=[(int(numel),)], dtype=dtype, weight_decay=0.1 if dtype == torch.bfloat16 else 0.0,
                    grad_sigma=1e-4 if dtype == torch.bfloat16 else 1e-3, label=f'one flat {dt} parameter of {int(numel)} elements')
    raise SystemExit(f'unknown workload {name}')


def algorithmic_bytes_per_param(dtype, rows: int):
    """HBM bytes per parameter the step cannot avoid, split by kernel: gradient read, one nibble
    of error feedback in and out, bf16 min+max in and out, one (index, value) row out;
    then `rows` window rows in, parameter in and out."""
    e = 2 if dtype == torch.bfloat16 else 4
    qbs, k = HYPER['quant_block_size'], HYPER['k_init']
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
    total = sum(times)
    return n * len(times) / total / 1e9, threads, sample, total / len(times) * 1e3, n


def reference_arm(args, spec):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    steps = max(1, args.steps)
    warmup = max(0, min(args.warmup, 3))
    if steps > 60:
        steps = 60     # each step is ~0.5-1.5 s of CPU work on the sample; keeps the arm within a few minutes
    rate, threads, sample, ms, n = cpu_oracle_rate(spec, steps, warmup)
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': rate, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': steps,
        'warmup': warmup, 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': 'bf16' if spec['dtype'] == torch.bfloat16 else 'f32', 'data': 'synthetic',
        'config': {'workload': spec['label'], 'sample': sample, 'sample_params': n, **{k: v for k, v in HYPER.items() if k != 'betas'}},
        'cpu_baseline': {'value': rate, 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': sample},
        'e2e': {'value': rate, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='llama3_8b', help='llama3_8b | gpt2_flat | flat_<bf16|f32>_<numel>')
    ap.add_argument('--grad-sets', type=int, default=2, help='distinct pre-generated gradient sets cycled over the steps')
    ap.add_argument('--e2e-steps', type=int, default=3)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--exchange', default='rows', choices=['rows', 'params'],
                    help='N > 1: what the ranks exchange (window rows, or updated parameters)')
    args = ap.parse_args()
    spec = workload_spec(args.workload)
    if args.impl == 'reference':
        reference_arm(args, spec)
        return

    import torch.distributed as dist
    from ista_daslab_optimizers_b200 import MicroAdam, _native
    from ista_daslab_optimizers_b200.sharding import ShardedMicroAdam

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

    flat_p, params, offsets = make_flat_model(spec, device, args.seed)
    grad_sets = [make_flat_grads(spec, offsets, flat_p.numel(), device, args.seed + 1 + i) for i in range(max(1, args.grad_sets))]
    n_params = sum(p.numel() for p in params)
    kw = dict(m=HYPER['m'], lr=HYPER['lr'], quant_block_size=HYPER['quant_block_size'], k_init=HYPER['k_init'],
              alpha=HYPER['alpha'], betas=HYPER['betas'], weight_decay=spec['weight_decay'], eps=HYPER['eps'])
    exchange = args.exchange if (world > 1 and HYPER['alpha'] == 0) else 'params'
    opt = ShardedMicroAdam(params, exchange=exchange, **kw) if world > 1 else MicroAdam(params, **kw)

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
    value = n_params * steps / (elapsed_ms * 1e-3) / 1e9

    # ---- end to end: gradients start in pinned host memory, a parameter checksum comes back -----------
    my_lo, my_hi = 0, flat_p.numel()
    if world > 1:
        mine = [(offsets[pc.index] + pc.lo, offsets[pc.index] + pc.hi) for pc in opt.plan if pc.rank == opt.rank]
        my_lo, my_hi = min(a for a, _ in mine), max(b for _, b in mine)
    e2e_steps = max(0, min(args.e2e_steps, steps))
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
    barrier()
    t0 = time.perf_counter()
    checksum = 0.0
    for t in range(max(1, e2e_steps) if e2e_steps else 0):
        if not chunked:
            gflat[my_lo:my_hi].copy_(host, non_blocking=True)
        else:
            for o in range(my_lo, my_hi, host.numel()):
                n = min(host.numel(), my_hi - o)
                gflat[o:o + n].copy_(host[:n], non_blocking=True)
        opt.step()
        checksum = flat_p[my_lo:my_hi:65536].float().sum().item()     # 4-byte device-to-host read, synchronises
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = n_params * e2e_steps / e2e_s.item() / 1e9 if e2e_steps else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel and the whole step ---------------------------------------------
    peak, peak_kind = measured_hbm_peak()
    rows_avg = sum(rows_per_step) / len(rows_per_step)
    ba, bb = algorithmic_bytes_per_param(spec['dtype'], rows_avg)
    per_rank_params = n_params / world
    # parameters one rank's launch of each kernel covers: kernel B runs over all of them when window rows are exchanged
    params_a, params_b = per_rank_params, (n_params if exchange == 'rows' else per_rank_params)
    dt = 'bf16' if spec['dtype'] == torch.bfloat16 else 'f32'
    kernels = []
    for name, b, ms, np_k in (('ef_topk_quant', ba, t_a, params_a), ('window_adam', bb, t_b, params_b)):
        gbs = np_k * b / (ms * 1e-3) / 1e9
        tr = NCU_TRAFFIC_BYTES_PER_PARAM.get((name, dt))
        kernels.append({'kernel': name, 'ms': ms, 'algorithmic_bytes': np_k * b, 'achieved_gbs': gbs,
                        'frac': gbs / peak, 'traffic': None if tr is None else tr * np_k})
    dom = max(kernels, key=lambda k: k['ms'])
    step_gbs = (params_a * ba + params_b * bb) / ((t_a + t_b) * 1e-3) / 1e9

    line = {
        'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': elapsed_ms / steps, 'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': dt, 'data': 'synthetic',
        'config': {'workload': spec['label'], 'params': n_params, 'parallelism': (f'shard{world}: kernel A sharded, window rows exchanged, kernel B replicated' if exchange == 'rows' else f'zero1-shard{world}+allgather') if world > 1 else 'single',
                   'l2_policy': 'inputs larger than L2 (GBs per step vs 126 MB)', 'grad_sets': len(grad_sets),
                   'arithmetic': 'fp32 on bf16/fp32 storage, 4-bit codes', **{k: v for k, v in HYPER.items() if k != 'betas'},
                   'weight_decay': spec['weight_decay']},
        'roofline': {'bound': 'hbm', 'kernel': dom['kernel'], 'achieved': dom['achieved_gbs'], 'peak': peak, 'unit': 'GB/s',
                     'frac': dom['frac'], 'traffic': dom['traffic'], 'peak_kind': f'of {peak_kind}',
                     'frac_of_8tbs_nominal': dom['achieved_gbs'] / 8000.0},
        'kernels': kernels,
        'step_hbm': {'achieved_gbs': step_gbs, 'frac': step_gbs / peak, 'frac_of_8tbs_nominal': step_gbs / 8000.0,
                     'algorithmic_bytes_per_param': ba + bb, 'kernel_ms': t_a + t_b, 'exposed_exchange_ms': t_gather},
        'e2e': {'value': e2e_value, 'unit': UNIT, 'h2d_bytes_per_step': h2d_bytes, 'd2h_bytes_per_step': 4, 'steps': e2e_steps,
                'checksum': checksum},
        'gpu_launches': launches,
        'clocks': clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        rate, threads, sample, ms, n = cpu_oracle_rate(spec, steps=3, warmup=1)
        line['cpu_baseline'] = {'value': rate, 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': sample,
                                'ms_per_step': ms, 'sample_params': n}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
