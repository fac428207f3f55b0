"""Communicator handles and domain-size queries (reference: `deep_ep/comm/handle.py:12-66`).

On NVLink the data path needs no library communicator: a handle is just the identity of the
process group used for bootstrap, either borrowed from PyTorch or created as an independent
("managed") NCCL group.
"""
import time
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils.envs import get_comm_name


class CommHandle:
    """Identity of the bootstrap communicator of a buffer; `managed` ones are destroyed with the handle."""

    def __init__(self, name: str, managed: bool, group: Optional[dist.ProcessGroup] = None):
        self.name = name
        self.managed = managed
        self.group = group

    def get(self) -> str:
        return self.name

    def release(self) -> None:
        if self.managed and self.group is not None:
            try:
                dist.destroy_process_group(self.group)
            except Exception:  # the default group may already be gone at interpreter exit
                pass
            self.group = None


NCCLCommHandle = CommHandle
HCCLCommHandle = CommHandle

_storage: Dict[Any, CommHandle] = {}


def get_comm_handle(group: dist.ProcessGroup, force_new_comm: bool = False) -> CommHandle:
    """Cached handle that borrows `group`, or (`force_new_comm`) an independent group over the same ranks."""
    if not force_new_comm:
        if group not in _storage:
            _storage[group] = CommHandle(get_comm_name(group, group.rank()), False, group)
        return _storage[group]
    ranks = dist.get_process_group_ranks(group)
    new_group = dist.new_group(ranks)            # collective over the default group members listed
    handle = CommHandle(get_comm_name(new_group, new_group.rank()), True, new_group)
    _storage[time.time_ns()] = handle
    return handle


get_hccl_comm_handle = get_comm_handle


def _domain(group_or_buffer: Any) -> Tuple[int, int]:
    context = getattr(group_or_buffer, 'context', None)
    if context is not None:
        return tuple(context.get_physical_domain_size())
    group: dist.ProcessGroup = group_or_buffer
    if torch.cuda.is_available() and group.size() > 1:
        # one NVSwitch domain: every rank of the group must be a peer-accessible GPU of this node
        assert group.size() <= torch.cuda.device_count(), 'all ranks of an EP group must share one NVLink domain'
    return 1, group.size()


def get_physical_domain_size(group_or_buffer: Any) -> Tuple[int, int]:
    """`(scale-out, scale-up)` sizes: one flat NVLink domain, so `(1, num_ranks)`."""
    return _domain(group_or_buffer)


def get_logical_domain_size(group_or_buffer: Any, allow_hybrid_mode: Optional[bool] = None) -> Tuple[int, int]:
    """Logical domain sizes; hybrid mode is accepted and has no effect on a single domain."""
    return _domain(group_or_buffer)


def destroy_all_managed_comm() -> None:
    """Drop cached handles (managed groups are destroyed); live buffers keep working."""
    for handle in _storage.values():
        handle.release()
    _storage.clear()


destroy_all_managed_hccl_comm = destroy_all_managed_comm
