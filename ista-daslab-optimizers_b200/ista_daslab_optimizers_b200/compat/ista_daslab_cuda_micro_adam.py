"""`ista_daslab_cuda_micro_adam` as micro_adam.py uses it (micro_adam.py:190,231,277-291)."""
from .._native import asymm_block_quant, asymm_block_quant_inv, compute_microadam_update

__all__ = ['asymm_block_quant_inv', 'asymm_block_quant', 'compute_microadam_update']
