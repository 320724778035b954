"""mab_fused_step_static: the fused step whose descriptor table is an array inside the library.

Some hosts of this library cannot give it a device workspace: a trainer whose memory plan has
already handed all of HBM to one arena has nothing left for cudaMalloc, and a runtime that binds
the library through a foreign-function interface may only be able to pass the buffers it tracks
itself (parameters, gradients, optimizer state).  This test drives that entry point through the C
ABI exactly as such a host would - no workspace tensor is created - and checks it against
mab_fused_step on identical inputs, for two steps in a row (the second call reuses the built-in
array, which still holds the first call's table).
"""
import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


def static_step(opt, N):
    """One optimizer step of `opt` through mab_fused_step_static (what MicroAdam.step does, minus the workspace)."""
    opt.steps += 1
    opt._refresh_entries()
    entries = opt._entries
    assert entries and all(e.fused for e in entries)
    descs = (N.MabTensor * len(entries))()
    for d, e in zip(descs, entries):
        opt._fill_static(d, e)
        opt._fill_dynamic(d, e)
        e.st['index'] = (e.st['index'] + 1) % opt.m
    args = opt._step_args()
    device = entries[0].p.device
    with torch.cuda.device(device):
        N.check(N.load().mab_fused_step_static(descs, len(entries), ctypes.byref(args), N.current_stream(device)),
                'mab_fused_step_static')


@pytest.mark.parametrize('name', ['bf16_wd', 'mixed_fp32_alpha'])
def test_static_table_step_equals_workspace_step(name):
    from ista_daslab_optimizers_b200 import _native as N
    case = cases.CASES[name]
    ref = cases.CudaAdapter(case, case.params())          # mab_fused_step with a caller-provided workspace
    new = cases.CudaAdapter(case, case.params())          # mab_fused_step_static
    tol = 1e-5 if case.dtype == torch.float32 else 1e-2   # the tolerance the other parity tests use
    for t in range(2):                                    # two calls in a row
        grads = case.grads(t)
        ref.step(grads)
        for p, g in zip(new.params, grads):
            p.grad = g.cuda()
        static_step(new.opt, N)
        torch.cuda.synchronize()
        for i in range(len(case.shapes)):
            a, b = ref.state(i), new.state(i)
            assert a['index'] == b['index']
            for key in ('I', 'V', 'error', 'min_vals', 'max_vals'):
                assert torch.equal(a[key].view(torch.uint8) if a[key].dtype != torch.uint8 else a[key],
                                   b[key].view(torch.uint8) if b[key].dtype != torch.uint8 else b[key]), (t, i, key)
            torch.testing.assert_close(new.param(i).float(), ref.param(i).float(), rtol=tol, atol=1e-9)
    assert N.device_error() == 0


def _tiny_optimizer(dtypes, numel, seed):
    """An optimizer over len(dtypes) tensors of `numel` elements (tensor i of element type dtypes[i]) with gradients."""
    from ista_daslab_optimizers_b200 import MicroAdam
    gen = torch.Generator(device='cuda').manual_seed(seed)
    params = [torch.nn.Parameter(torch.empty(numel, device='cuda').normal_(0, 0.02, generator=gen).to(dt)) for dt in dtypes]
    grads = [torch.empty(numel, device='cuda').normal_(0, 1e-3, generator=gen).to(dt) for dt in dtypes]
    opt = MicroAdam(params, m=4, lr=1e-3, quant_block_size=64, k_init=0.05, weight_decay=0.1)
    return opt, params, grads


@pytest.mark.parametrize('layout', ['mixed_types', 'many_tensors'])
def test_static_table_splits_a_call_into_runs(layout):
    """One call whose tensors change element type back and forth, and one with more tensors of one type than a
    launch takes (512): the entry point cuts both into several launches per kernel; results equal mab_fused_step's."""
    from ista_daslab_optimizers_b200 import _native as N
    if layout == 'mixed_types':
        dtypes = [torch.float32, torch.float32, torch.bfloat16, torch.float32, torch.bfloat16, torch.bfloat16, torch.float32]
        numel = 70000
    else:
        dtypes = [torch.float32] * 700
        numel = 257
    ref_opt, ref_params, grads = _tiny_optimizer(dtypes, numel, seed=5)
    new_opt, new_params, _ = _tiny_optimizer(dtypes, numel, seed=5)
    for t in range(2):
        for p, q, g in zip(ref_params, new_params, grads):
            p.grad = g
            q.grad = g
        ref_opt.step()
        static_step(new_opt, N)
        torch.cuda.synchronize()
        for i, (p, q) in enumerate(zip(ref_params, new_params)):
            a, b = ref_opt.state[p], new_opt.state[q]
            for key in ('I', 'V', 'error', 'min_vals', 'max_vals'):
                assert torch.equal(a[key].view(torch.uint8) if a[key].dtype != torch.uint8 else a[key],
                                   b[key].view(torch.uint8) if b[key].dtype != torch.uint8 else b[key]), (t, i, key)
            assert torch.equal(p.detach(), q.detach()), (t, i)
    assert N.device_error() == 0


def test_static_table_rejects_more_tensors_than_it_holds():
    from ista_daslab_optimizers_b200 import _native as N
    lib = N.load()
    n = N.MAB_STATIC_MAX_TENSORS + 1
    descs = (N.MabTensor * n)()
    args = N.MabStepArgs()
    args.steps, args.m, args.quant_block_size = 1, 10, 64
    assert lib.mab_fused_step_static(descs, n, ctypes.byref(args), None) == -4
    msg = lib.mab_last_error().decode()
    assert str(N.MAB_STATIC_MAX_TENSORS) in msg and 'split' in msg
