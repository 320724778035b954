"""The unmodified reference micro_adam.py on this library's kernels (ista_daslab_optimizers_b200.compat).

Needs a checkout of the reference ($MICROADAM_REFERENCE_DIR, or a directory `reference` beside this
repository); skipped where there is none."""
import os

import pytest
import torch

import cases
from oracle.reference_harness import DEFAULT_REFERENCE_DIR, reference_available

needs_checkout = pytest.mark.skipif(not reference_available(), reason='no reference checkout on this machine')


@needs_checkout
@pytest.mark.skipif(torch.cuda.is_available(), reason='checks the wiring without a device')
def test_reference_class_reaches_the_native_library_and_fails_loudly_without_a_device():
    """The reference's constructor asks the native module for the SM count (micro_adam.py:40): through the stand-ins
    that is a call into libmicroadam_b200.so, which has no CPU path."""
    from ista_daslab_optimizers_b200 import compat, _native
    Ref = compat.load_reference_microadam(DEFAULT_REFERENCE_DIR)
    assert Ref.__module__ == 'ista_daslab_optimizers.micro_adam.micro_adam'
    import ista_daslab_cuda_tools, ista_daslab_cuda_micro_adam
    assert ista_daslab_cuda_tools.copy_values is _native.copy_values
    assert ista_daslab_cuda_micro_adam.asymm_block_quant is _native.asymm_block_quant
    with pytest.raises(_native.NativeError):
        Ref([torch.nn.Parameter(torch.zeros(8))], m=10, lr=1e-3, quant_block_size=64)


@needs_checkout
@pytest.mark.gpu
@pytest.mark.parametrize('name', ['c1_fp32_1m', 'narrow_m5'])
def test_unmodified_reference_file_runs_on_the_kernels(name):
    """The reference's own step loop (its torch.topk included) on the operator-level kernels against the CPU oracle.
    torch.topk leaves order and ties open, so window rows are compared per block after sorting; the inputs are
    continuous fp32 values, which makes ties at the k-th magnitude improbable (bf16 cases would tie all the time)."""
    from ista_daslab_optimizers_b200 import compat
    Ref = compat.load_reference_microadam(DEFAULT_REFERENCE_DIR)
    case = cases.CASES[name]
    params = [torch.nn.Parameter(p.cuda()) for p in case.params()]
    opt = Ref(params, m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha,
              betas=case.betas, weight_decay=case.weight_decay, eps=case.eps)
    oracle = cases.OracleAdapter(case, case.params())
    rtol, atol = cases.param_tolerances(case.dtype, case.lr)
    for t in range(3):
        grads = case.grads(t)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        oracle.step(grads)
        for i, p in enumerate(params):
            a, b = opt.state[p], oracle.state(i)
            row = (a['index'] - 1) % case.m
            km, nfull = a['k_block_size_many'], a['topk_full_blocks_count']
            got, want = a['I'][row].cpu(), b['I'][row]
            if a['k_index'] > 0:
                assert torch.equal(got[:a['k_index']].view(nfull, km).sort(dim=1).values, want[:a['k_index']].view(nfull, km))
            if a['k_block_size_few'] > 0:
                assert torch.equal(got[a['k_index']:].sort().values, want[a['k_index']:])
            assert torch.equal(a['error'].cpu(), b['error'])
            torch.testing.assert_close(p.detach().cpu().float(), oracle.param(i).float(), rtol=rtol, atol=atol)
