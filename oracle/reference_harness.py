"""Runs the UNMODIFIED reference MicroAdam on CPU.  TEST INFRASTRUCTURE ONLY.

The reference file ista_daslab_optimizers/micro_adam/micro_adam.py imports two native modules
that are not part of the reference tree (`ista_daslab_cuda_tools`,
`ista_daslab_cuda_micro_adam`, from the unpinned pip package `ista-daslab-optimizers-cuda`)
and `gpustat`.  This harness registers stand-ins for them whose functions are the CPU
restatements in oracle/microadam_oracle.py, registers a bare parent package so that the heavy
package `__init__` (which imports every other optimizer) is skipped, patches `torch.topk`
inside the reference module with the canonical tie rule, and then imports the reference
class itself from the reference checkout.  The control flow that runs is the reference's own.

It only works where a reference checkout exists (pass its path or set MICROADAM_REFERENCE_DIR);
the golden vectors under tests/golden/ were generated through it and travel instead of it.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import torch

from . import microadam_oracle as O

# a checkout of the reference: $MICROADAM_REFERENCE_DIR, else a directory `reference` beside this repository
DEFAULT_REFERENCE_DIR = os.environ.get('MICROADAM_REFERENCE_DIR') or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..', 'reference'))


def reference_available(reference_dir: str = DEFAULT_REFERENCE_DIR) -> bool:
    return os.path.isfile(os.path.join(reference_dir, 'ista_daslab_optimizers', 'micro_adam', 'micro_adam.py'))


class _CanonicalTopk:
    """Return type compatible with the two attributes micro_adam.py:193-200 reads."""

    def __init__(self, indices):
        self.indices = indices


def _canonical_topk(input, k, sorted=False):  # noqa: A002 - mirrors torch.topk's signature
    keys = input if input.dim() == 2 else input.view(1, -1)
    idx = O.canonical_topk_indices(keys, k)
    return _CanonicalTopk(idx if input.dim() == 2 else idx.view(-1))


class _TorchProxy(types.ModuleType):
    """`torch` as seen by the reference module: everything forwarded, `topk` canonical."""

    def __init__(self):
        super().__init__('torch')

    def __getattr__(self, name):
        if name == 'topk':
            return _canonical_topk
        return getattr(torch, name)


def load_reference_microadam(reference_dir: str = DEFAULT_REFERENCE_DIR, max_floats: int = O.B200_MAX_FLOATS,
                             sm_count: int = 148):
    """Import and return the reference `MicroAdam` class, backed by the CPU stand-ins."""
    if not reference_available(reference_dir):
        raise FileNotFoundError(f'no reference checkout at {reference_dir}')

    tools = types.ModuleType('ista_daslab_cuda_tools')
    tools.get_sm_count = lambda: sm_count
    tools.get_max_floats_for_shared_memory_per_thread_block = lambda: max_floats
    tools.copy_values = O.copy_values
    tools.zerorize_block_components = O.zerorize_block_components

    micro = types.ModuleType('ista_daslab_cuda_micro_adam')
    micro.asymm_block_quant_inv = O.asymm_block_quant_inv
    micro.asymm_block_quant = O.asymm_block_quant
    micro.compute_microadam_update = O.compute_microadam_update

    gpustat = types.ModuleType('gpustat')
    wandb = sys.modules.get('wandb')
    if wandb is None:
        try:
            import wandb  # noqa: F401
        except Exception:
            wandb = types.ModuleType('wandb')
            wandb.log = lambda *a, **k: None
            sys.modules['wandb'] = wandb

    sys.modules['ista_daslab_cuda_tools'] = tools
    sys.modules['ista_daslab_cuda_micro_adam'] = micro
    sys.modules.setdefault('gpustat', gpustat)

    pkg_dir = os.path.join(reference_dir, 'ista_daslab_optimizers')
    parent = types.ModuleType('ista_daslab_optimizers')
    parent.__path__ = [pkg_dir]
    for name in [n for n in sys.modules if n == 'ista_daslab_optimizers' or n.startswith('ista_daslab_optimizers.')]:
        del sys.modules[name]
    sys.modules['ista_daslab_optimizers'] = parent
    mod = importlib.import_module('ista_daslab_optimizers.micro_adam.micro_adam')
    mod.torch = _TorchProxy()
    return mod.MicroAdam
