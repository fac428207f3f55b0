"""Expert load balancing over redundant expert slots (API of the reference's `deep_ep/buffers/ep.py:594-649`,
whose native side is unimplemented). Redundant slots live in the LB region of an `EPBuffer`, which is part of the
peer-visible allocation, so owners push weights into them and pull gradients out of them directly over NVLink."""
from typing import Sequence, Union

import torch

from ..utils.event import EventOverlap


def _as_list(t: Union[Sequence[torch.Tensor], torch.Tensor]):
    return [t] if isinstance(t, torch.Tensor) else list(t)


def lb_prefetch_weights(buffer, redundant_expert_weights, expert_weights, redundancy_mapping: torch.Tensor,
                        num_sms: int = 0, previous_event=None) -> EventOverlap:
    redundant, local = _as_list(redundant_expert_weights), _as_list(expert_weights)
    assert redundant and len(redundant) == len(local) and all(t is not None for t in redundant + local)
    return EventOverlap(buffer.runtime.lb_prefetch_weights(redundant, local, redundancy_mapping, num_sms, previous_event))


def lb_reduce_grads(buffer, redundant_expert_grads: torch.Tensor, expert_grads: torch.Tensor,
                    redundancy_mapping: torch.Tensor, num_sms: int = 0, previous_event=None) -> EventOverlap:
    return EventOverlap(buffer.runtime.lb_reduce_grads(redundant_expert_grads, expert_grads, redundancy_mapping,
                                                       num_sms, previous_event))
