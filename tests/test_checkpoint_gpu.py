"""Checkpoint / resume of the CUDA optimizer: its own `state_dict()`, and one written by the reference class."""
import os

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

STATE_DTYPES = {'I': torch.int16, 'V': torch.bfloat16, 'error': torch.uint8, 'min_vals': torch.bfloat16, 'max_vals': torch.bfloat16}
FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'reference_state_3steps.pt')


def bits(t):
    return t if t.dtype in (torch.uint8, torch.int16) else t.view(torch.int16)


def assert_same_state(a, b):
    assert a['index'] == b['index']
    for key, dt in STATE_DTYPES.items():
        assert a[key].dtype == dt and b[key].dtype == dt, key
        assert torch.equal(bits(a[key]).cpu(), bits(b[key]).cpu()), key


@pytest.mark.parametrize('name', ['bf16_wd', 'mixed_fp32_alpha'])
def test_save_load_continue_equals_uninterrupted(name):
    """4 steps, save, load into a fresh optimizer over copies of the parameters, 3 more steps on both: the state
    stays bit-equal and so do the parameters (same kernels, same inputs).  Every loaded state tensor keeps the
    element type it was saved with (torch's own load_state_dict would cast them to the parameter's)."""
    case = cases.CASES[name]
    first = cases.CudaAdapter(case, case.params())
    for t in range(4):
        first.step(case.grads(t))
    sd = first.opt.state_dict()
    second = cases.CudaAdapter(case, [p.detach().cpu().clone() for p in first.params])
    second.opt.load_state_dict(sd)
    assert second.opt.steps == 4
    for i in range(len(case.shapes)):
        assert_same_state(first.state(i), second.state(i))
        assert second.state(i)['I'].data_ptr() != first.state(i)['I'].data_ptr()      # a copy, not an alias
    for t in range(4, 7):
        first.step(case.grads(t))
        second.step(case.grads(t))
        for i in range(len(case.shapes)):
            assert_same_state(first.state(i), second.state(i))
            assert torch.equal(first.param(i), second.param(i)), (t, i)


def test_reference_written_checkpoint_loads_and_continues():
    """A `state_dict()` written by the unmodified reference class after 3 steps (tests/golden/make_reference_state.py)
    goes into the CUDA optimizer and into the oracle; both continue for 3 steps on the same gradients."""
    from oracle.microadam_oracle import MicroAdamOracle, Geometry
    fx = torch.load(FIXTURE)
    case = cases.CKPT_CASE
    assert fx['case'] == case.name and fx['steps'] == 3
    gpu = cases.CudaAdapter(case, [p.clone() for p in fx['params']])
    gpu.opt.load_state_dict(fx['state_dict'])
    assert gpu.opt.steps == 0          # the reference does not save its step counter: the caller restores it
    gpu.opt.steps = fx['steps']
    cpu_params = [p.clone() for p in fx['params']]
    ref = MicroAdamOracle(cpu_params, m=case.m, lr=case.lr, quant_block_size=case.qbs, k_init=case.k_init, alpha=case.alpha,
                          betas=case.betas, weight_decay=case.weight_decay, eps=case.eps, d_block_size=case.d_block_size)
    ref.steps = fx['steps']
    for i, p in enumerate(cpu_params):
        st = fx['state_dict']['state'][i]
        ref.state[i] = dict(geo=Geometry.make(p.numel(), case.d_block_size, case.k_init, case.qbs), index=st['index'],
                            **{k: st[k].clone() for k in STATE_DTYPES})
    rtol, atol = cases.param_tolerances(case.dtype, case.lr)
    for t in range(3, 6):
        grads = case.grads(t)
        gpu.step(grads)
        ref.step([g.clone() for g in grads])
        for i in range(len(case.shapes)):
            assert_same_state(gpu.state(i), ref.state[i])
            torch.testing.assert_close(gpu.param(i).cpu(), cpu_params[i], rtol=rtol, atol=atol)


def test_indices_saved_in_another_element_type_are_restored():
    """Checkpoint pipelines that cast every state tensor (micro_adam.py:175-178 mentions one) hand `I` back as floats:
    integer-valued indices are accepted and become int16 again."""
    fx = torch.load(FIXTURE)
    case = cases.CKPT_CASE
    sd = fx['state_dict']
    for st in sd['state'].values():
        st['I'] = st['I'].float()
    gpu = cases.CudaAdapter(case, [p.clone() for p in fx['params']])
    gpu.opt.load_state_dict(sd)
    for i in range(len(case.shapes)):
        assert gpu.state(i)['I'].dtype == torch.int16
        assert torch.equal(gpu.state(i)['I'].cpu(), fx['state_dict']['state'][i]['I'].to(torch.int16))


@pytest.mark.parametrize('damage', ['index_beyond_block', 'negative_index', 'wrong_dtype', 'wrong_shape'])
def test_damaged_checkpoint_is_rejected_on_the_host(damage):
    """A window index outside its block would be used as a store offset by the update kernel: load_state_dict
    refuses it (and wrong element types or shapes) before anything reaches the GPU."""
    fx = torch.load(FIXTURE)
    case = cases.CKPT_CASE
    sd = fx['state_dict']
    st = sd['state'][0]
    if damage == 'index_beyond_block':
        st['I'][2, 5] = st['d_block_size']
    elif damage == 'negative_index':
        st['I'][0, 0] = -1
    elif damage == 'wrong_dtype':
        st['error'] = st['error'].float()
    else:
        st['V'] = st['V'][:, :-1]
    gpu = cases.CudaAdapter(case, [p.clone() for p in fx['params']])
    with pytest.raises((ValueError, TypeError)):
        gpu.opt.load_state_dict(sd)


def test_short_block_index_bound():
    """Indices of a tensor's short last block are bounded by that block's length, not by d_block_size."""
    fx = torch.load(FIXTURE)
    case = cases.CKPT_CASE
    sd = fx['state_dict']
    st = sd['state'][0]
    assert st['k_block_size_few'] > 0
    st['I'][1, st['k_index']] = 640                     # the short block holds elements 0..639
    gpu = cases.CudaAdapter(case, [p.clone() for p in fx['params']])
    with pytest.raises(ValueError):
        gpu.opt.load_state_dict(sd)
