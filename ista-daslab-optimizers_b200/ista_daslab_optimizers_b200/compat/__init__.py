"""Stand-ins for the two native modules the reference's micro_adam.py imports.

`install()` registers them in sys.modules under the reference's names, so that an unmodified
`ista_daslab_optimizers/micro_adam/micro_adam.py` runs on the B200 kernels:

    from ista_daslab_optimizers_b200 import compat; compat.install()
    from ista_daslab_optimizers import MicroAdam

The reference still calls torch.topk itself (micro_adam.py:193-200); everything else on its step
goes through these modules.

`load_reference_microadam(checkout)` does the same and then imports the reference's MicroAdam class
from a checkout of its repository without running the package `__init__` (which imports every other
optimizer of the package and their dependencies); `gpustat` and `wandb`, which the reference imports
at module level (tools.py:2, micro_adam.py:5), get empty stand-ins when they are not installed.
"""
import importlib
import os
import sys
import types

from . import ista_daslab_cuda_micro_adam, ista_daslab_cuda_tools


def install() -> None:
    sys.modules['ista_daslab_cuda_tools'] = ista_daslab_cuda_tools
    sys.modules['ista_daslab_cuda_micro_adam'] = ista_daslab_cuda_micro_adam


def load_reference_microadam(checkout: str):
    """The reference's own MicroAdam class (file untouched), bound to this library's kernels."""
    pkg_dir = os.path.join(checkout, 'ista_daslab_optimizers')
    if not os.path.isfile(os.path.join(pkg_dir, 'micro_adam', 'micro_adam.py')):
        raise FileNotFoundError(f'no checkout of the reference at {checkout}')
    install()
    for name in ('gpustat', 'wandb'):
        if name not in sys.modules:
            try:
                importlib.import_module(name)
            except Exception:
                stub = types.ModuleType(name)
                stub.log = lambda *a, **k: None       # wandb.log (micro_adam.py:350)
                sys.modules[name] = stub
    for name in [n for n in sys.modules if n == 'ista_daslab_optimizers' or n.startswith('ista_daslab_optimizers.')]:
        del sys.modules[name]
    parent = types.ModuleType('ista_daslab_optimizers')
    parent.__path__ = [pkg_dir]
    sys.modules['ista_daslab_optimizers'] = parent
    return importlib.import_module('ista_daslab_optimizers.micro_adam.micro_adam').MicroAdam
