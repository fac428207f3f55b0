"""Lifecycle shared by all communication buffers (reference: `deep_ep/buffers/base.py:4-27`)."""
import os
from abc import ABC, abstractmethod
from typing import List

import torch
import torch.distributed as dist

from .._C_loader import _C


class BufferBase(ABC):
    """Holds the native runtime object and enforces the explicit-destroy contract."""

    def __init__(self, explicitly_destroy: bool = False):
        self.explicitly_destroy = explicitly_destroy
        self.runtime = None

    @property
    def main_context(self):
        """The first communication context, or `None` once destroyed."""
        return None if self.runtime is None else self.runtime.main_context

    def print_memory_usage(self) -> None:
        """Print workspace / buffer / storage bytes of this rank."""
        assert self.runtime is not None
        self.runtime.print_memory_usage()

    @abstractmethod
    def destroy(self) -> None:
        """Collective teardown; only legal for buffers created with `explicitly_destroy=True`."""
        assert self.explicitly_destroy, '`destroy()` requires `explicitly_destroy=True` at construction'
        if self.runtime is not None:
            self.runtime.destroy()
            self.runtime = None


    def abort(self, group: dist.ProcessGroup = None) -> None:
        """Teardown after a failure (a device-side wait that ran out, a peer that is gone): unlike `destroy()` it runs no
        device-side barrier, whose own state may be what broke. This rank stops mapping its peers' memory, meets the other
        ranks of `group` on the host (skip that with `group=None` when they cannot be reached any more) and frees its
        allocation. The buffer is unusable afterwards; the CUDA context is not affected."""
        if self.runtime is None:
            return
        if hasattr(self.runtime, 'close_peer_mappings'):
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.runtime.close_peer_mappings()
            if group is not None and group.size() > 1:
                dist.barrier(group)
            self.runtime.abort()
        elif hasattr(self.runtime, 'destroyed'):
            self.runtime.destroyed = True          # CPU stand-in runtimes hold nothing that needs releasing
        self.runtime = None


def connect_peers(context, group: dist.ProcessGroup) -> None:
    """Exchange the CUDA-IPC handles of a context's symmetric allocation over `group` and map the peers.

    Plays the role of the reference's channel bring-up (`csrc/kernels/comm/hccl.hpp:173-331`): afterwards
    every rank holds a device-usable base address for every peer's allocation.
    """
    if group.size() == 1 or context.peers_ready:
        return
    handles: List[bytes] = [b''] * group.size()
    device = torch.cuda.current_device()
    exchanged = [None] * group.size()
    dist.all_gather_object(exchanged, (context.get_local_handle(), device, os.uname().nodename), group)
    # one NVLink domain: every peer must be another GPU of this node that this GPU can address directly
    for rank, (_, peer_device, node) in enumerate(exchanged):
        assert node == os.uname().nodename, f'rank {rank} runs on another node ({node}); only one NVLink domain is supported'
        if peer_device != device:
            assert _C.check_peer_access(device, peer_device), f'GPU {device} cannot access GPU {peer_device} (rank {rank}) directly'
    handles = [h for h, _, _ in exchanged]
    context.set_peer_handles(handles)
    if context.multicast_pending():
        # NVLS route (EP_NVLS=1): every device has joined the multicast object; binding memory needs all of them in
        dist.barrier(group)
        context.bind_multicast()
        dist.barrier(group)


def sync_group(group: dist.ProcessGroup) -> None:
    """Device sync, process-group barrier, device sync: construction is complete on every rank afterwards."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dist.barrier(group)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
