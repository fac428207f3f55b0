"""`PPBuffer`: buffered send/recv between ring neighbours (reference: `deep_ep/buffers/pp.py:13-86`)."""
from typing import Optional

import os

import torch
import torch.distributed as dist

from .. import comm
from .._C_loader import _C
from ..utils.semantic import nvtx_range
from .base import BufferBase, connect_peers, sync_group


class PPBuffer(BufferBase):
    """Symmetric ring storage for pipeline-parallel activations.

    `send` returns (on the stream) once the payload sits in the neighbour's landing slot; up to
    `num_max_inflight_tensors` sends per direction may run ahead of the matching `recv`. Messages
    between a pair are FIFO and carry no header: sender and receiver agree on sizes by convention.

    Stream usage: every operation runs on the current stream.

    `transport` (keyword, or `EP_PP_TRANSPORT` in the environment): `'nvlink'` (default) is this library's own ring of
    landing slots in peer memory, written and drained by its kernels; `'nccl'` moves the payload with the process group's
    point-to-point calls on the library's streams (`deep_ep/buffers/pp_p2p.py`), with the same buffered semantics.
    """

    barrier = comm.barrier
    get_comm_stream = comm.get_comm_stream

    def __init__(self, group: dist.ProcessGroup, num_max_tensor_bytes: int, num_max_inflight_tensors: int,
                 sl_idx: Optional[int] = None, num_gpu_timeout_secs: int = 100, explicitly_destroy: bool = False,
                 *, use_huge1g_page: bool = True, transport: Optional[str] = None):
        if sl_idx is not None:
            raise NotImplementedError('RDMA service levels do not exist on NVLink')
        assert num_max_tensor_bytes > 0 and num_max_inflight_tensors > 0 and num_gpu_timeout_secs > 0
        transport = transport or os.environ.get('EP_PP_TRANSPORT', 'nvlink')
        assert transport in ('nvlink', 'nccl'), f'unknown PPBuffer transport {transport!r}'
        self.transport = transport
        self.group = group
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.comm_handle = comm.get_comm_handle(group)
        super().__init__(explicitly_destroy)
        self.is_simulated = not torch.cuda.is_available()
        if transport == 'nccl':
            from .pp_p2p import LibraryP2PRuntime
            device = torch.device('cpu') if self.is_simulated else torch.device('cuda', torch.cuda.current_device())
            self.runtime = LibraryP2PRuntime(group, num_max_tensor_bytes, num_max_inflight_tensors, device)
        elif self.is_simulated:
            from ..sim.buffers import SimPPRuntime
            self.runtime = SimPPRuntime(group, num_max_tensor_bytes, num_max_inflight_tensors)
        else:
            self.runtime = _C.PPBuffer(self.rank_idx, self.num_ranks, self.comm_handle.get(), num_max_tensor_bytes,
                                       num_max_inflight_tensors, use_huge1g_page, num_gpu_timeout_secs, explicitly_destroy)
            connect_peers(self.runtime.context, group)
        self.context = self.runtime.context
        self.storage = self.runtime.storage
        sync_group(group)

    @nvtx_range('deep_ep.PPBuffer.send')
    def send(self, x: torch.Tensor, dst_rank_idx: int, num_sms: Optional[int] = None) -> None:
        """Send contiguous `x` (at most `num_max_tensor_bytes`) to the previous or next rank of the ring."""
        self.runtime.send(x, dst_rank_idx, 0 if num_sms is None else num_sms)

    @nvtx_range('deep_ep.PPBuffer.recv')
    def recv(self, x: torch.Tensor, src_rank_idx: int, num_sms: Optional[int] = None) -> None:
        """Receive into contiguous `x` from the previous or next rank of the ring."""
        self.runtime.recv(x, src_rank_idx, 0 if num_sms is None else num_sms)

    def destroy(self) -> None:
        super().destroy()
        self.storage = None
        self.context = None
        self.comm_handle = None
