"""Stand-ins for the two native modules the reference's micro_adam.py imports.

`install()` registers them in sys.modules under the reference's names, so that an unmodified
`ista_daslab_optimizers/micro_adam/micro_adam.py` runs on the B200 kernels:

    from ista_daslab_optimizers_b200 import compat; compat.install()
    from ista_daslab_optimizers import MicroAdam

The reference still calls torch.topk itself (micro_adam.py:193-200); everything else on its step
goes through these modules.
"""
import sys

from . import ista_daslab_cuda_micro_adam, ista_daslab_cuda_tools


def install() -> None:
    sys.modules['ista_daslab_cuda_tools'] = ista_daslab_cuda_tools
    sys.modules['ista_daslab_cuda_micro_adam'] = ista_daslab_cuda_micro_adam
