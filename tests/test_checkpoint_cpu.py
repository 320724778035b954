"""The host logic of MicroAdam.load_state_dict without a GPU: element types survive, damaged state is refused.

The constructor of the shipped optimizer needs the native library and a device, so a subclass that skips it
stands in here; `load_state_dict` itself is the shipped code."""
import os

import pytest
import torch

from ista_daslab_optimizers_b200.micro_adam import MicroAdam

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'reference_state_3steps.pt')


class HostOnly(MicroAdam):
    def __init__(self, params, m=10):
        torch.optim.Optimizer.__init__(self, params, dict(lr=1e-3, weight_decay=0.1, eps=1e-8, alpha=0))
        self.m, self.steps, self._entries_key = m, 0, None


def load(sd, fx):
    params = [torch.nn.Parameter(p.clone()) for p in fx['params']]
    opt = HostOnly(params)
    opt.load_state_dict(sd)
    return opt, params


def test_element_types_survive_loading():
    fx = torch.load(FIXTURE)
    opt, params = load(fx['state_dict'], fx)
    want = {'I': torch.int16, 'V': torch.bfloat16, 'error': torch.uint8, 'min_vals': torch.bfloat16, 'max_vals': torch.bfloat16}
    for i, p in enumerate(params):
        st = opt.state[p]
        for key, dt in want.items():
            assert st[key].dtype == dt
            assert torch.equal(st[key].view(torch.uint8), fx['state_dict']['state'][i][key].view(torch.uint8))
    sd = opt.state_dict()
    sd['steps'] = 7
    opt2, _ = load(sd, fx)
    assert opt2.steps == 7


def test_bf16_parameters_do_not_round_the_indices():
    """With bf16 parameters torch's own loading would pass `I` through bf16 (29055 -> 29056, one past the block)."""
    fx = torch.load(FIXTURE)
    fx['params'] = [p.bfloat16() for p in fx['params']]
    st0 = fx['state_dict']['state'][0]
    st0['I'][0, 0] = 29055
    opt, params = load(fx['state_dict'], fx)
    assert opt.state[params[0]]['I'].dtype == torch.int16 and int(opt.state[params[0]]['I'][0, 0]) == 29055


@pytest.mark.parametrize('damage', ['index_beyond_block', 'negative_index', 'short_block_index', 'fractional_index',
                                    'wrong_dtype', 'wrong_shape', 'ring_index'])
def test_damaged_state_is_refused(damage):
    fx = torch.load(FIXTURE)
    sd = fx['state_dict']
    st = sd['state'][0]
    if damage == 'index_beyond_block':
        st['I'][2, 5] = st['d_block_size']
    elif damage == 'negative_index':
        st['I'][0, 0] = -1
    elif damage == 'short_block_index':
        st['I'][1, st['k_index']] = st['d'] - st['d_index_topk']
    elif damage == 'fractional_index':
        st['I'] = st['I'].float() + 0.5
    elif damage == 'wrong_dtype':
        st['min_vals'] = st['min_vals'].float()
    elif damage == 'wrong_shape':
        st['error'] = st['error'][:-1]
    else:
        st['index'] = 10
    with pytest.raises((ValueError, TypeError)):
        load(sd, fx)
