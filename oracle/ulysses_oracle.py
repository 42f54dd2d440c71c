"""CPU restatement of the Ulysses head<->sequence exchange (test infrastructure, not product).

``seq_all_to_all`` evaluates, for all ranks at once, what ``_SeqAllToAll.forward`` (gt_sp/layer.py:
30-45) produces: rank r splits its input into P chunks along ``scatter_idx``, sends chunk r' to rank
r', and concatenates what it receives along ``gather_idx``."""
from __future__ import annotations

from typing import List

import numpy as np


def seq_all_to_all(inputs: List[np.ndarray], scatter_idx: int, gather_idx: int) -> List[np.ndarray]:
    world = len(inputs)
    chunks = [np.array_split(x, world, axis=scatter_idx) for x in inputs]   # tensor_split, :41
    return [np.concatenate([chunks[src][dst] for src in range(world)], axis=gather_idx)   # :44-45
            for dst in range(world)]


def copy_global_token0(x: np.ndarray, global_rows) -> np.ndarray:
    """gt_sp/utils.py:836: rows listed in global_rows take the value of row 0 (per batch entry)."""
    y = x.copy()
    y[:, list(global_rows), :] = x[:, 0:1, :]
    return y
