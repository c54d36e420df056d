"""State pool: what recurrent layers carry from step to step, one slot per live sequence.

A slot is the same number the paged cache hands a sequence (`KVCacheManager.seq_id_to_batch`); slot RESERVED_BATCH
belongs to no sequence (CUDA-graph padding rows point at it and the kernels skip it).  The pool owns, per recurrent
layer, one tensor [slots, *shape] for every entry of the layer's `state_specs()` and sets it as an attribute of the
layer.  Nothing is cleared when a slot changes hands: the kernels start from a zero state whenever a sequence's portion
starts at position 0.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch


class RecurrentStatePool:
    def __init__(self, max_num_batches: int, dtype: torch.dtype, device):
        self.slots = int(max_num_batches) + 1          # + the reserved slot
        self.dtype, self.device = dtype, device
        self.tensors: List[Tuple[torch.nn.Module, str, torch.Tensor]] = []

    def attach(self, layer: torch.nn.Module) -> None:
        for name, (shape, dt) in layer.state_specs(self.dtype).items():
            t = torch.zeros((self.slots, *shape), dtype=dt, device=self.device)
            setattr(layer, name, t)
            self.tensors.append((layer, name, t))

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for _, _, t in self.tensors)

    def bytes_per_slot(self) -> int:
        return self.nbytes // self.slots

    def snapshot(self, slot: int) -> Dict[str, torch.Tensor]:
        """Copies of one slot's state (tests)."""
        return {f"{i}.{name}": t[slot].clone() for i, (_, name, t) in enumerate(self.tensors)}
