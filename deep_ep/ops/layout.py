"""Routing layout without communication (sender half of the dispatch handle)."""
from typing import Tuple

import torch

from .._C_loader import _C


def get_dispatch_layout(topk_idx: torch.Tensor, num_experts: int, num_ranks: int,
                        num_sms: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Return `(dst_buffer_slot_idx [T, k] int32, num_tokens_per_rank [R] int32, num_tokens_per_expert [E] int32)`.

    `dst_buffer_slot_idx[t, j]` is the position token t takes among this rank's tokens sent to the rank that owns
    expert `topk_idx[t, j]`, stored at the last top-k position selecting that rank and -1 elsewhere (duplicates,
    masked entries) — exactly what `EPBuffer.dispatch` records in its handle. On CPU tensors the CPU restatement
    of the same rule is used.
    """
    if not topk_idx.is_cuda:
        from ..sim.ep import sender_slots
        slots, per_rank = sender_slots(topk_idx, num_experts, num_ranks)
        valid = topk_idx[topk_idx >= 0]
        return slots, per_rank.to(torch.int32), torch.bincount(valid, minlength=num_experts).to(torch.int32)
    return _C.get_dispatch_layout(topk_idx.contiguous(), num_experts, num_ranks, num_sms)
