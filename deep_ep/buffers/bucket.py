"""`BucketBuffer` and `BucketSession`: batched all-gather over registered storage
(reference: `deep_ep/buffers/bucket.py:19-356`)."""
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .. import comm
from .._C_loader import _C
from ..utils.event import EventOverlap
from ..utils.math import align
from ..utils.semantic import nvtx_range
from .allocator import BufferAllocator
from .base import BufferBase, connect_peers, sync_group


class BucketSession:
    """Context manager under which the buffer's collectives accept tensors that live outside its storage.

    Inside a session a bump allocator (32-byte aligned, restarting at offset 0 on entry) hands out
    registered regions; outputs requested outside the storage are produced in such a region and copied to
    the caller's tensor inside the wait hook, which then returns the caller's tensor. One group per
    session; sessions do not nest; the buffer's methods are restored on exit even after an exception;
    leaving a session adds no barrier.
    """

    _ALIGNMENT = 32

    def __init__(self, buffer: 'BucketBuffer'):
        self.buffer = buffer
        self.offset = 0
        self.group: Optional[dist.ProcessGroup] = None
        self._saved: Dict[str, Any] = {}

    def __enter__(self) -> 'BucketSession':
        assert self.buffer._active_session is None, 'BucketBuffer sessions cannot be nested'
        self.buffer._active_session = self
        self.offset, self.group = 0, None
        for name in ('all_gather', 'reduce_scatter', 'all_reduce'):
            self._saved[name] = getattr(self.buffer, name)
        self.buffer.all_gather = self._all_gather
        self.buffer.reduce_scatter = self._reduce_scatter
        self.buffer.all_reduce = self._all_reduce
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        for name in self._saved:
            if name in self.buffer.__dict__:
                del self.buffer.__dict__[name]
        self._saved.clear()
        self.buffer._active_session = None

    def _bind_group(self, group: Optional[dist.ProcessGroup]) -> dist.ProcessGroup:
        group = self.buffer.groups[self.buffer.get_context_idx(group)]
        assert self.group is None or self.group is group, 'a session is bound to the first group it used'
        self.group = group
        return group

    def _carve(self, num_bytes: int) -> torch.Tensor:
        start = align(self.offset, self._ALIGNMENT)
        assert start + num_bytes <= self.buffer.storage.numel(), 'BucketBuffer storage exhausted in this session'
        self.offset = start + num_bytes
        return self.buffer.storage.narrow(0, start, num_bytes)

    def allocate(self, shape, dtype: torch.dtype, group: Optional[dist.ProcessGroup] = None):
        """Registered tensor(s) of `shape` (or a list of shapes) inside the storage."""
        self._bind_group(group)
        def one(s):
            numel = 1
            for d in (s if isinstance(s, (tuple, list, torch.Size)) else (s,)):
                numel *= d
            return self._carve(numel * dtype.itemsize).view(dtype).view(s)
        if isinstance(shape, (list, tuple)) and shape and isinstance(shape[0], (list, tuple, torch.Size)):
            return [one(s) for s in shape]
        return one(shape)

    def _inside(self, t: torch.Tensor) -> bool:
        base = self.buffer.storage.data_ptr()
        return base <= t.data_ptr() and t.data_ptr() + t.nbytes <= base + self.buffer.storage.numel()

    def _all_gather(self, srcs, dsts=None, group: Optional[dist.ProcessGroup] = None, num_sms: Optional[int] = None):
        group = self._bind_group(group)
        is_packed, srcs, dsts = BucketBuffer._pack_tensors(srcs, dsts)
        size, rank = group.size(), group.rank()
        inner_dsts: List[torch.Tensor] = []
        copy_back: List[Tuple[torch.Tensor, int]] = []
        for i, src in enumerate(srcs):
            user_dst = dsts[i] if dsts else None
            if user_dst is None and self._inside(src):
                # in-place form: src already is this rank's shard of a registered gathered tensor
                offset = src.data_ptr() - self.buffer.storage.data_ptr() - rank * src.nbytes
                inner_dsts.append(self.buffer.storage.narrow(0, offset, size * src.nbytes).view(src.dtype))
            elif user_dst is not None and self._inside(user_dst):
                inner_dsts.append(user_dst)
            else:
                staged = self._carve(size * src.nbytes).view(src.dtype)
                inner_dsts.append(staged)
                if user_dst is not None:
                    assert user_dst.nbytes == size * src.nbytes and user_dst.dtype == src.dtype
                    copy_back.append((user_dst, i))
        handle = self._saved['all_gather'](srcs, inner_dsts, group=group, num_sms=num_sms)
        inner_hook = handle.hook_after_wait
        handle.hook_after_wait = None
        external = {i: t for t, i in copy_back}

        def hook():
            gathered = inner_hook()
            gathered = [gathered] if isinstance(gathered, torch.Tensor) else list(gathered)
            for i, user_dst in external.items():
                user_dst.view(-1).copy_(gathered[i].view(-1))
                gathered[i] = user_dst
            return gathered[0] if is_packed else gathered
        handle.register_hook_after_wait(hook)
        return handle


    def _stage_sources(self, srcs) -> Tuple[List[torch.Tensor], Dict[int, torch.Tensor]]:
        """Registered stand-ins for the sources of a reduction: tensors inside the storage are used as they are, others
        are copied (on the current stream) into a carved region. Every rank must stage the same tensors in the same
        order, so that the regions sit at the same storage offsets everywhere."""
        inner: List[torch.Tensor] = []
        staged: Dict[int, torch.Tensor] = {}
        for i, src in enumerate(srcs):
            if self._inside(src):
                assert src.is_contiguous(), 'a registered source must be contiguous'
                inner.append(src)
                continue
            region = self._carve(src.nbytes).view(src.dtype).view(src.shape)
            region.copy_(src)
            inner.append(region)
            staged[i] = src
        return inner, staged

    def _reduce_scatter(self, srcs, comm_precision: str = 'fp32', scale: float = 1.0,
                        group: Optional[dist.ProcessGroup] = None, num_sms: Optional[int] = None):
        """`BucketBuffer.reduce_scatter` that also takes tensors outside the storage: those are staged in a registered
        region first. The handle returns this rank's reduced shards, which for staged tensors are views of the region
        (valid until the storage is reused), as in the reference's session (`deep_ep/buffers/bucket.py:103-181`)."""
        group = self._bind_group(group)
        is_packed, srcs = BucketBuffer._pack_tensors(srcs)
        inner, _ = self._stage_sources(srcs)
        handle = self._saved['reduce_scatter'](inner, comm_precision=comm_precision, scale=scale, group=group, num_sms=num_sms)
        inner_hook = handle.hook_after_wait
        handle.hook_after_wait = None

        def hook():
            shards = inner_hook()
            shards = [shards] if isinstance(shards, torch.Tensor) else list(shards)
            return shards[0] if is_packed else shards
        handle.register_hook_after_wait(hook)
        return handle

    def _all_reduce(self, srcs, scale: float = 1.0, group: Optional[dist.ProcessGroup] = None, num_sms: Optional[int] = None):
        """`BucketBuffer.all_reduce` that also takes tensors outside the storage: those are staged in a registered region,
        reduced there, and copied back into the caller's tensor inside the wait hook, so the call stays in place for
        the caller. The handle returns the caller's tensors."""
        group = self._bind_group(group)
        is_packed, srcs = BucketBuffer._pack_tensors(srcs)
        inner, staged = self._stage_sources(srcs)
        handle = self._saved['all_reduce'](inner, scale=scale, group=group, num_sms=num_sms)
        inner_hook = handle.hook_after_wait
        handle.hook_after_wait = None

        def hook():
            reduced = inner_hook()
            reduced = [reduced] if isinstance(reduced, torch.Tensor) else list(reduced)
            for i, user in staged.items():
                user.copy_(reduced[i].view(user.shape))
                reduced[i] = user
            return reduced[0] if is_packed else reduced
        handle.register_hook_after_wait(hook)
        return handle


class BucketBuffer(BufferBase):
    """Contiguous symmetric storage registered with one to eight process groups.

    Stream usage: communication runs on the communication stream; epilogues run on the current stream.
    """

    get_comm_stream = comm.get_comm_stream

    @staticmethod
    def _pack_tensors(*tensors):
        """Normalise `tensor | sequence | None` arguments to lists; report whether a bare tensor was given."""
        is_packed = isinstance(tensors[0], torch.Tensor)
        lists = tuple([] if t is None else [t] if isinstance(t, torch.Tensor) else list(t) for t in tensors)
        assert all(len(item) in (0, len(lists[0])) for item in lists)
        return is_packed, *lists

    def __init__(self, group: Union[dist.ProcessGroup, Sequence[dist.ProcessGroup]],
                 allocation_plan_or_num_bytes: Union[BufferAllocator, int], sl_idx: Optional[int] = None,
                 num_gpu_timeout_secs: int = 100, explicitly_destroy: bool = False, *, use_huge1g_page: bool = True):
        plan = allocation_plan_or_num_bytes if isinstance(allocation_plan_or_num_bytes, BufferAllocator) else None
        num_bytes = allocation_plan_or_num_bytes if plan is None else plan.num_bytes
        if plan is not None:
            assert not plan.materialized
        assert isinstance(num_bytes, int) and num_bytes > 0 and num_gpu_timeout_secs > 0
        self.groups = [group] if isinstance(group, dist.ProcessGroup) else list(group)
        assert self.groups and len(self.groups) <= _C.MAX_CONTEXTS
        assert len(set(self.groups)) == len(self.groups), 'Duplicate communication groups'
        assert num_bytes % _C.get_num_allocation_alignment() == 0
        if sl_idx is not None:
            raise NotImplementedError('RDMA service levels do not exist on NVLink')
        self.comm_handles = [comm.get_comm_handle(g) for g in self.groups]
        for context_idx, g in enumerate(self.groups):
            seen = [None] * g.size()
            dist.all_gather_object(seen, context_idx, g)
            assert all(i == context_idx for i in seen), 'All ranks must use the same context index within a group'
        self.num_bytes = num_bytes
        self._active_session: Optional[BucketSession] = None
        super().__init__(explicitly_destroy)
        self.is_simulated = not torch.cuda.is_available()
        if self.is_simulated:
            # CPU process groups (gloo): same Python layer over `deep_ep.sim.buffers.SimBucketRuntime`
            from ..sim.buffers import SimBucketRuntime
            self.runtime = SimBucketRuntime(self.groups, num_bytes)
        else:
            self.runtime = _C.BucketBuffer([g.rank() for g in self.groups], [g.size() for g in self.groups],
                                           [h.get() for h in self.comm_handles], num_bytes, use_huge1g_page,
                                           num_gpu_timeout_secs, explicitly_destroy)
        self.contexts = self.runtime.contexts
        if not self.is_simulated:
            for context, g in zip(self.contexts, self.groups):
                connect_peers(context, g)
        self.storage = self.runtime.storage
        for g in self.groups:
            sync_group(g)
        if plan is not None:
            plan.materialize(self.storage)

    @property
    def context(self):
        return self.contexts[0] if self.contexts else None

    def get_theoretical_num_sms(self, op: str, group: Optional[dist.ProcessGroup] = None) -> int:
        self.get_context_idx(group)
        if op == 'all_gather':
            return 0
        if op in ('reduce_scatter', 'all_reduce'):
            return _C.get_num_sms()
        raise NotImplementedError(op)

    def get_context_idx(self, group: Optional[dist.ProcessGroup]) -> int:
        assert len(self.groups) == 1 or group is not None, '`group` is required when the buffer has multiple groups'
        return 0 if group is None else self.groups.index(group)

    def session(self) -> BucketSession:
        """Open a session in which collectives accept unregistered tensors."""
        return BucketSession(self)

    def barrier(self, wait_comm_stream: bool = True, with_cpu_sync: bool = False, sequential: bool = True,
                group: Optional[dist.ProcessGroup] = None) -> None:
        """Device barrier over the selected group."""
        comm.barrier(self, wait_comm_stream, with_cpu_sync, sequential, self.get_context_idx(group))

    def _reduce(self, srcs, scale: float, group: Optional[dist.ProcessGroup], num_sms: Optional[int], all_reduce: bool) -> EventOverlap:
        is_packed, srcs = self._pack_tensors(srcs)
        context_idx = self.get_context_idx(group)
        assert num_sms in (None, 0) or num_sms > 0
        results, event, used_sms = self.runtime.reduce(srcs, context_idx, 0 if num_sms is None else num_sms, float(scale), all_reduce)
        handle = EventOverlap(event, extra_tensors=tuple(srcs) + (self.storage,))
        handle.register_hook_after_wait(lambda: results[0] if is_packed else results)
        setattr(handle, 'num_sms', used_sms)
        return handle

    @nvtx_range('deep_ep.BucketBuffer.reduce_scatter')
    def reduce_scatter(self, srcs, comm_precision: str = 'fp32', scale: float = 1.0,
                       group: Optional[dist.ProcessGroup] = None, num_sms: Optional[int] = None) -> EventOverlap:
        """Launch a batched in-place reduce-scatter of up to 64 registered tensors on the communication stream.

        Every rank passes tensors at the same storage offsets (bf16, fp16 or fp32); tensor i is cut into `group.size()`
        equal shards and this rank's shard receives `scale * sum over ranks`, accumulated in fp32 in rank order.
        `handle.wait()` returns this rank's reduced shards (1-D views into `srcs`); the other shards of `srcs` keep
        their contents. `comm_precision` names the accumulation precision and must be 'fp32': shards cross NVLink in
        the tensors' own dtype because the owner pulls them straight from its peers' memory.
        (The reference declares this method without a kernel behind it, `deep_ep/buffers/bucket.py:266-285`.)
        """
        assert comm_precision == 'fp32', 'sums are accumulated in fp32; other precisions are not offered'
        return self._reduce(srcs, scale, group, num_sms, all_reduce=False)

    @nvtx_range('deep_ep.BucketBuffer.all_reduce')
    def all_reduce(self, srcs, scale: float = 1.0, group: Optional[dist.ProcessGroup] = None,
                   num_sms: Optional[int] = None) -> EventOverlap:
        """Launch a batched in-place all-reduce of up to 64 registered tensors on the communication stream.

        One kernel: rank r pulls shard r of every tensor from all ranks, sums in fp32, scales, and stores the result to
        every rank, so all ranks end with bitwise identical tensors. `handle.wait()` returns `srcs`.
        (The reference declares this method without a kernel behind it, `deep_ep/buffers/bucket.py:287-305`.)
        """
        return self._reduce(srcs, scale, group, num_sms, all_reduce=True)

    @nvtx_range('deep_ep.BucketBuffer.all_gather')
    def all_gather(self, srcs: Union[torch.Tensor, Sequence[torch.Tensor]],
                   dsts: Optional[Union[torch.Tensor, Sequence[torch.Tensor]]] = None,
                   group: Optional[dist.ProcessGroup] = None, num_sms: Optional[int] = None) -> EventOverlap:
        """Launch a batched all-gather of up to 64 tensors on the communication stream.

        Without `dsts` each `src` must be this rank's shard *inside* the storage and the gather is in place.
        With `dsts`, each `dst` lies in the storage with `dst.nbytes == group.size() * src.nbytes` and `src` may be
        any contiguous device tensor of the same dtype. All ranks pass equal shard sizes.
        `handle.wait()` is where completion is guaranteed; it returns flat 1-D views of the gathered tensors
        (a single tensor if a single tensor was passed).
        """
        is_packed, srcs, dsts = self._pack_tensors(srcs, dsts)
        context_idx = self.get_context_idx(group)
        assert num_sms in (None, 0) or num_sms > 0
        event, epilogue, used_sms = self.runtime.all_gather(srcs, dsts, context_idx, 0 if num_sms is None else num_sms)
        handle = EventOverlap(event, extra_tensors=tuple(srcs) + tuple(dsts) + (self.storage,))
        handle.register_hook_after_wait(lambda: epilogue()[0] if is_packed else epilogue())
        setattr(handle, 'num_sms', 0 if num_sms is None else num_sms)
        return handle

    def destroy(self) -> None:
        super().destroy()
        self.contexts = None
        self.storage = None
        self.comm_handles = None
