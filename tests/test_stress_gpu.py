"""The stress configuration at its stated size: 300 mixed-shape fp32 tensors with row / column counts
drawn from {64, ..., 8192} (every 10th a conv-like [256, 256, 3, 3]), heavy-tailed Student-t gradients
rounded to 8 mantissa bits so that exact ties abound, 10 % of the tensors zero-initialised with an
all-zero first gradient, m = 10, k_init = 0.01, alpha = 0.5, 12 steps.

Two checks.  All 300 tensors: the fused kernels against the operator-level kernels (two independent
implementations of the step in this library), state bit for bit, parameters to the fp32 tolerance.  An
unclipped subset of 12 of them (about 250 M elements, what the CPU oracle finishes in a minute): the fused kernels
against the CPU oracle."""
import pytest
import torch

import cases
from ista_daslab_optimizers_b200 import synthetic as S

pytestmark = pytest.mark.gpu

HYPER = dict(m=10, lr=1e-3, quant_block_size=64, k_init=0.01, alpha=0.5, betas=(0.9, 0.999), weight_decay=0.0, eps=1e-8)
STEPS = 12


def student_t3_ties(shape, gen):
    """Student-t (3 degrees of freedom) * 1e-3, rounded to 8 mantissa bits, on the GPU."""
    z = torch.empty(shape, device='cuda').normal_(generator=gen)
    chi = torch.zeros(shape, device='cuda')
    for _ in range(3):
        chi.addcmul_(w := torch.empty(shape, device='cuda').normal_(generator=gen), w)
    return (z / (chi.clamp_min_(1e-12) / 3).sqrt_() * 1e-3).bfloat16().float()


def state_equal(a, b, qbs, numel):
    used = (numel + qbs - 1) // qbs
    return (a['index'] == b['index'] and torch.equal(a['I'], b['I']) and torch.equal(a['V'].view(torch.int16), b['V'].view(torch.int16))
            and torch.equal(a['error'], b['error'])
            and torch.equal(a['min_vals'][:used].view(torch.int16), b['min_vals'][:used].view(torch.int16))
            and torch.equal(a['max_vals'][:used].view(torch.int16), b['max_vals'][:used].view(torch.int16)))


def test_stress_all_300_tensors_fused_equals_operator_level():
    from ista_daslab_optimizers_b200 import MicroAdam, _native
    shapes = S.stress_shapes(0, count=300)
    zero = set(range(0, 300, 10))
    gen = torch.Generator(device='cuda').manual_seed(0)
    init = [torch.zeros(s, device='cuda') if i in zero else torch.empty(s, device='cuda').normal_(0, 0.02, generator=gen)
            for i, s in enumerate(shapes)]
    pa = [torch.nn.Parameter(x.clone()) for x in init]
    pb = [torch.nn.Parameter(x) for x in init]
    fused = MicroAdam(pa, **HYPER)
    plain = MicroAdam(pb, use_fused=False, **HYPER)
    for t in range(STEPS):
        for i, (a, b) in enumerate(zip(pa, pb)):
            g = torch.zeros(shapes[i], device='cuda') if (t == 0 and i in zero) else student_t3_ties(shapes[i], gen)
            a.grad = g
            b.grad = g.clone()                 # the operator-level path uses the gradient as scratch
        fused.step()
        plain.step()
        for a, b in zip(pa, pb):
            b.grad = None
        if t in (0, 1, STEPS - 2, STEPS - 1):  # the first steps (zero tensors, ties) and the wrapped window
            bad = [i for i, (a, b) in enumerate(zip(pa, pb))
                   if not state_equal(fused.state[a], plain.state[b], HYPER['quant_block_size'], a.numel())]
            assert not bad, (t, bad[:10])
    assert all(e.fused for e in fused._entries) and not any(e.fused for e in plain._entries)
    for i, (a, b) in enumerate(zip(pa, pb)):
        rtol, atol = cases.param_tolerances(torch.float32, HYPER['lr'])
        torch.testing.assert_close(a.detach(), b.detach(), rtol=rtol, atol=atol, msg=lambda m: f'tensor {i}: {m}')
    assert _native.device_error() == 0


def test_stress_unclipped_subset_matches_oracle():
    from ista_daslab_optimizers_b200 import MicroAdam
    from oracle.microadam_oracle import MicroAdamOracle
    shapes = S.stress_shapes(0, count=300)[98:110]          # includes one of the conv-like [256, 256, 3, 3] tensors
    zero = {0, 7}
    gen = torch.Generator(device='cuda').manual_seed(1)
    params = [torch.nn.Parameter(torch.zeros(s, device='cuda') if i in zero else torch.empty(s, device='cuda').normal_(0, 0.02, generator=gen))
              for i, s in enumerate(shapes)]
    cpu_params = [p.detach().cpu().clone() for p in params]
    opt = MicroAdam(params, **HYPER)
    ref = MicroAdamOracle(cpu_params, d_block_size=opt.d_block_size, **HYPER)
    qbs = HYPER['quant_block_size']
    for t in range(STEPS):
        grads = [torch.zeros(s, device='cuda') if (t == 0 and i in zero) else student_t3_ties(s, gen) for i, s in enumerate(shapes)]
        for p, g in zip(params, grads):
            p.grad = g
        opt.step()
        ref.step([g.cpu() for g in grads])
        for i, p in enumerate(params):
            a, b = opt.state[p], ref.state[i]
            gpu_state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in a.items() if k in ('I', 'V', 'error', 'min_vals', 'max_vals', 'index')}
            assert state_equal(gpu_state, b, qbs, p.numel()), (t, i)
            rtol, atol = cases.param_tolerances(torch.float32, HYPER['lr'])
            torch.testing.assert_close(p.detach().cpu(), cpu_params[i], rtol=rtol, atol=atol, msg=lambda m: f'step {t}, tensor {i}: {m}')
