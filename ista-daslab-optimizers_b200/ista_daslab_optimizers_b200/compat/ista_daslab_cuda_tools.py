"""`ista_daslab_cuda_tools` as micro_adam.py uses it (micro_adam.py:40,43,202-209,214)."""
from .._native import (copy_values, get_max_floats_for_shared_memory_per_thread_block, get_sm_count,
                       zerorize_block_components)

__all__ = ['get_sm_count', 'get_max_floats_for_shared_memory_per_thread_block', 'copy_values',
           'zerorize_block_components']
