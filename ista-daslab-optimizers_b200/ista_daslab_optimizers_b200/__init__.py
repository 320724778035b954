"""B200-native MicroAdam optimizer step (drop-in for ista_daslab_optimizers.MicroAdam)."""
from .micro_adam import MicroAdam
from .tools import CopyDirection, block_split, get_first_device

__all__ = ['MicroAdam', 'CopyDirection', 'block_split', 'get_first_device']
