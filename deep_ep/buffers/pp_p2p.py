"""Second transport of `PPBuffer`: the process group's own point-to-point calls (NCCL on GPUs, gloo on CPU ranks).

The default transport is a ring of landing slots in peer memory written by this library's kernels
(`csrc/buffers/pp.hpp`). This one keeps the buffered semantics of the reference (`deep_ep/buffers/pp.py:13-86` there:
up to `num_max_inflight_tensors` sends may run ahead of the matching receives, FIFO per pair, ring neighbours only) on
top of library send / recv, which by themselves rendezvous:

* every `send` first copies the tensor into a staging slot (a ring of `num_max_inflight_tensors` slots per direction), so
  the caller's tensor is free again as soon as the copy is queued; the library send then reads the slot;
* a slot is reused only after the send that last read it has completed (the only point where the host may wait);
* the two directions of a pair use two different process groups. With one group a rank's send to a peer and its receive
  from the same peer would sit in one queue, and two ranks that both send first would wait for each other for ever.

Transfers run on the library's own streams and overlap the caller's compute; `recv` makes the current stream wait for
the data.
"""
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..sim.buffers import SimContext


class LibraryP2PRuntime:
    """Runtime object of `PPBuffer(transport='nccl')`; same interface as the native and the simulated runtimes."""

    def __init__(self, group: dist.ProcessGroup, num_max_tensor_bytes: int, num_max_inflight_tensors: int,
                 device: torch.device):
        self.group, self.device = group, device
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.num_max_tensor_bytes, self.num_max_inflight = num_max_tensor_bytes, num_max_inflight_tensors
        self.context = self.main_context = SimContext(self.rank_idx, self.num_ranks)
        ranks = [dist.get_global_rank(group, r) for r in range(self.num_ranks)]
        # [0]: messages from a lower to a higher group rank, [1]: from a higher to a lower one
        self.direction_groups = [dist.new_group(ranks, use_local_synchronization=True) for _ in range(2)]
        slot_bytes = (num_max_tensor_bytes + 255) // 256 * 256
        self.slot_bytes = slot_bytes
        # staging slots: [destination: next, previous][slot]
        self.storage = torch.zeros(2 * num_max_inflight_tensors * slot_bytes, dtype=torch.uint8, device=device)
        self._slots = self.storage.view(2, num_max_inflight_tensors, slot_bytes)
        self._pending: Dict[int, List[Tuple[object, int]]] = {0: [], 1: []}      # per direction: (work, slot)
        self._sent = [0, 0]
        self._loopback: List[torch.Tensor] = []      # a ring of one rank: staged messages waiting for their recv
        self.destroyed = False
        self._connect()

    def _connect(self) -> None:
        """Set up every neighbour connection of both direction groups now, with all ranks taking part. The library
        opens a point-to-point connection at the first transfer between two ranks, and both of them have to be inside a
        call on that group for it: two neighbours that each start with a send (on different groups) would otherwise wait
        on the host for each other. One batched exchange per group (send and receive in a single library group call) with
        both neighbours does it."""
        if self.num_ranks == 1:
            return
        nxt, prv = self._neighbours()
        for group in self.direction_groups:
            out = torch.zeros(2, 4, dtype=torch.uint8, device=self.device)
            got = torch.zeros(2, 4, dtype=torch.uint8, device=self.device)
            ops = []
            for i, peer in enumerate((nxt, prv) if nxt != prv else (nxt,)):
                target = dist.get_global_rank(self.group, peer)
                ops.append(dist.P2POp(dist.isend, out[i], target, group=group))
                ops.append(dist.P2POp(dist.irecv, got[i], target, group=group))
            for work in dist.batch_isend_irecv(ops):
                work.wait()
        if self.device.type == 'cuda':
            torch.cuda.synchronize()

    def _neighbours(self) -> Tuple[int, int]:
        return (self.rank_idx + 1) % self.num_ranks, (self.rank_idx - 1) % self.num_ranks

    def _check(self, x: torch.Tensor, peer: int) -> None:
        assert not self.destroyed and x.is_contiguous() and 0 < x.nbytes <= self.num_max_tensor_bytes
        assert x.device.type == self.device.type
        assert peer in self._neighbours(), 'only the previous or the next rank of the ring can be addressed'

    def _group_for(self, src: int, dst: int) -> dist.ProcessGroup:
        return self.direction_groups[0 if src < dst else 1]

    def send(self, x: torch.Tensor, dst: int, num_sms: int) -> None:
        self._check(x, dst)
        direction = 0 if dst == self._neighbours()[0] else 1
        pending = self._pending[direction]
        slot = self._sent[direction] % self.num_max_inflight
        self._sent[direction] += 1
        while pending and (len(pending) >= self.num_max_inflight or any(s == slot for _, s in pending)):
            pending.pop(0)[0].wait()                                  # the send that last read this slot is over
        staged = self._slots[direction, slot, :x.nbytes]
        if self.num_ranks == 1:
            assert len(self._loopback) < self.num_max_inflight, 'more sends in flight than `num_max_inflight_tensors`'
            staged.copy_(x.view(-1).view(torch.uint8))
            self._loopback.append(staged)
            return
        staged.copy_(x.view(-1).view(torch.uint8))
        work = dist.isend(staged, dist.get_global_rank(self.group, dst), group=self._group_for(self.rank_idx, dst))
        pending.append((work, slot))

    def recv(self, x: torch.Tensor, src: int, num_sms: int) -> None:
        self._check(x, src)
        if self.num_ranks == 1:
            assert self._loopback, 'recv without a matching send'
            staged = self._loopback.pop(0)
            assert staged.numel() == x.nbytes, 'send and recv sizes must match'
            x.view(-1).view(torch.uint8).copy_(staged)
            return
        work = dist.irecv(x.view(-1).view(torch.uint8), dist.get_global_rank(self.group, src),
                          group=self._group_for(src, self.rank_idx))
        work.wait()                      # NCCL: the current stream waits; gloo: the host waits

    def print_memory_usage(self) -> None:
        print(f'[deep_ep] rank {self.rank_idx}/{self.num_ranks}: library p2p transport, staging {self.storage.numel()} bytes')

    def destroy(self) -> None:
        assert not self.destroyed
        for pending in self._pending.values():
            for work, _ in pending:
                work.wait()
            pending.clear()
        if self.device.type == 'cuda':
            torch.cuda.synchronize()
        dist.barrier(self.group)
        for g in self.direction_groups:
            dist.destroy_process_group(g)
        self.storage, self._slots, self.destroyed = None, None, True
