"""Host helpers the MicroAdam step uses, with the reference's names and meaning
(ista_daslab_optimizers/tools.py:12-14, 29-34, 85-92)."""
from __future__ import annotations

from enum import Enum

import torch


class CopyDirection(Enum):
    """tools.py:12-14."""
    k2d = 0
    d2k = 1


def get_first_device() -> torch.device:
    """tools.py:29-34: one process per GPU, rank r on cuda:r of a single node."""
    if not torch.cuda.is_available():
        return torch.device('cpu')
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.device(f'cuda:{torch.distributed.get_rank() % torch.cuda.device_count()}')
    return torch.device('cuda:0')


def block_split(model_size: int, block_size: int):
    """tools.py:85-92: (number of full blocks, start of the last, shorter block)."""
    if model_size < block_size:
        return 1, model_size
    blocks_count = int(model_size / block_size)
    start_index_last_block = model_size - model_size % block_size
    return blocks_count, start_index_last_block
