"""One transformer layer of the Llama-3-8B-shaped list at its real sizes, against the CPU oracle.

The small parity cases never produce the block geometry of the benchmark's tensors: 577 / 144 / 2020
full top-k blocks followed by a short last block of 11 904 / 10 240 / 27 136 elements, and the norm
vectors that are a single block of 4096.  Here q, k, v, o, gate, up, down and the two norms
(218 112 000 bf16 parameters, weight_decay 0.1) take 12 steps, so the m = 10 window wraps, and after
every step the window row written, the error-feedback codes and the block statistics are compared bit
for bit and every parameter element to the bf16 tolerance.
"""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

SHAPES = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336), (4096,), (4096,)]
HYPER = dict(m=10, lr=1e-3, quant_block_size=64, k_init=0.01, alpha=0, betas=(0.9, 0.999), weight_decay=0.1, eps=1e-8)
STEPS = 12


def test_llama_layer_matches_oracle():
    from ista_daslab_optimizers_b200 import MicroAdam, _native
    from oracle.microadam_oracle import MicroAdamOracle
    gen = torch.Generator(device='cuda').manual_seed(7)
    params = [torch.nn.Parameter(torch.empty(s, dtype=torch.bfloat16, device='cuda').normal_(0, 0.02, generator=gen)) for s in SHAPES]
    cpu_params = [p.detach().cpu().clone() for p in params]
    opt = MicroAdam(params, **HYPER)
    ref = MicroAdamOracle(cpu_params, d_block_size=opt.d_block_size, **HYPER)
    assert opt.d_block_size == 29056
    qbs = HYPER['quant_block_size']
    for t in range(STEPS):
        grads = [torch.empty(s, dtype=torch.bfloat16, device='cuda').normal_(0, 1e-4, generator=gen) for s in SHAPES]
        for p, g in zip(params, grads):
            p.grad = g
        opt.step()
        ref.step([g.cpu() for g in grads])
        assert all(e.fused for e in opt._entries)
        for i, p in enumerate(params):
            a, b = opt.state[p], ref.state[i]
            row = (a['index'] - 1) % HYPER['m']
            assert a['index'] == b['index']
            assert (a['topk_full_blocks_count'], a['k']) == (b['geo'].topk_full_blocks_count, b['geo'].k)
            assert torch.equal(a['I'][row].cpu(), b['I'][row]), (t, i, 'I')
            assert torch.equal(a['V'][row].cpu().view(torch.int16), b['V'][row].view(torch.int16)), (t, i, 'V')
            assert torch.equal(a['error'].cpu(), b['error']), (t, i, 'error')
            used = (p.numel() + qbs - 1) // qbs
            for key in ('min_vals', 'max_vals'):
                assert torch.equal(a[key][:used].cpu().view(torch.int16), b[key][:used].view(torch.int16)), (t, i, key)
            rtol, atol = cases.param_tolerances(torch.bfloat16, HYPER['lr'])
            torch.testing.assert_close(p.detach().cpu().float(), cpu_params[i].float(), rtol=rtol, atol=atol,
                                       msg=lambda m: f'step {t}, tensor {i}: {m}')
    assert _native.device_error() == 0
