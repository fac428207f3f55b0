"""`EPBuffer` / `EPHandle`: expert-parallel dispatch and combine in the expanded layout.

Public contract of the reference's `deep_ep/buffers/ep.py:21-649` (argument order, handle fields,
cached replays, deferred epilogues), implemented over NVLink peer memory on B200. Extensions that
the reference does not have are keyword-only: `fused_fp8_quant` (BF16 in, e4m3 + 1x128 scales on
the wire, quantised inside the dispatch kernel).
"""
import functools
import os
from typing import Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .. import comm
from .._C_loader import _C
from ..utils.event import EventHandle, EventOverlap
from ..utils.semantic import nvtx_range, value_or
from .allocator import BufferAllocator
from .base import BufferBase, connect_peers, sync_group


class EPHandle:
    """Routing state returned by `EPBuffer.dispatch`; reusable as a cached handle and required by `combine`.

    Attributes:
        do_expand: always True (one output row per selected local expert).
        num_experts, expert_alignment, num_max_tokens_per_rank, num_sms: the dispatch configuration.
        topk_idx: `[num_tokens, num_topk]` int64, held by reference; it must not change while the
            handle is alive (ordinary in-place edits are caught through the tensor version counter).
        num_recv_tokens / num_expanded_tokens: row counts of `recv_src_metadata` / `recv_x`
            (worst-case capacities when dispatch ran without host sync).
        num_recv_tokens_per_expert_list: aligned per-expert counts on the host (empty without host sync).
        psum_num_recv_tokens_per_rank: `[num_ranks]` int32 inclusive prefix of rank-deduplicated receive counts.
        psum_num_recv_tokens_per_expert: `[num_local_experts]` int32; entry i = aligned counts of experts
            before i plus the exact count of expert i (region starts are aligned, ends are not).
        num_unaligned_recv_tokens_per_expert: `[num_local_experts]` int32 exact counts.
        recv_src_metadata: `[num_recv_tokens, num_topk + 2]` int32 rows
            `[expanded slot per top-k position or -1 ..., src_token_global_idx, master_topk_idx]`.
        dst_buffer_slot_idx: `[num_tokens, num_topk]` int32 slot inside the destination rank's per-source
            region, stored at the master position of that rank, -1 elsewhere.
        dst_gsge_idx: `[num_tokens, num_topk]` int32, all -1 (scatter-gather bookkeeping of the reference's
            transport; kept for API shape).
    """

    def __init__(self, do_expand: bool, num_experts: int, expert_alignment: int, num_max_tokens_per_rank: int,
                 num_sms: int, topk_idx: torch.Tensor, num_recv_tokens: int, num_expanded_tokens: int,
                 num_recv_tokens_per_expert_list: list, psum_num_recv_tokens_per_rank: torch.Tensor,
                 psum_num_recv_tokens_per_expert: torch.Tensor, num_unaligned_recv_tokens_per_expert: torch.Tensor,
                 recv_src_metadata: torch.Tensor, dst_buffer_slot_idx: torch.Tensor, dst_gsge_idx: torch.Tensor):
        assert topk_idx is not None
        self.do_expand = do_expand
        self.num_experts = num_experts
        self.expert_alignment = expert_alignment
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_sms = num_sms
        self.num_recv_tokens = num_recv_tokens
        self.num_expanded_tokens = num_expanded_tokens
        self.num_recv_tokens_per_expert_list = num_recv_tokens_per_expert_list
        self.psum_num_recv_tokens_per_rank = psum_num_recv_tokens_per_rank
        self.psum_num_recv_tokens_per_expert = psum_num_recv_tokens_per_expert
        self.num_unaligned_recv_tokens_per_expert = num_unaligned_recv_tokens_per_expert
        self.recv_src_metadata = recv_src_metadata
        self.dst_buffer_slot_idx = dst_buffer_slot_idx
        self.dst_gsge_idx = dst_gsge_idx
        self.cached_recv_src_metadata_before_sort = None
        self._topk_idx = topk_idx
        self._topk_idx_version = None if topk_idx.is_inference() else topk_idx._version

    def __setstate__(self, state: dict) -> None:
        # A handle is plain data and may be pickled (for instance into a checkpoint). The tensor version counter is not
        # part of a tensor's value: a restored `topk_idx` starts counting again, so the guard is re-armed on it.
        self.__dict__.update(state)
        restored = self._topk_idx
        self._topk_idx_version = None if restored.is_inference() else restored._version

    @property
    def topk_idx(self) -> torch.Tensor:
        assert self._topk_idx_version is None or self._topk_idx._version == self._topk_idx_version, \
            '`topk_idx` must not be modified while the EP handle is in use'
        return self._topk_idx

    def deterministic_sort(self, do_cpu_sync: bool, is_cached_dispatch: bool, recv_x: torch.Tensor,
                           recv_sf: Optional[torch.Tensor], recv_topk_weights: Optional[torch.Tensor]) -> None:
        """Make the expanded layout a pure function of the inputs.

        The B200 dispatch assigns expanded rows in (source rank, source token) order with a two-pass
        count/assign scheme, which already equals the order of `src_token_global_idx` inside every
        expert. The rows therefore are where a sort would put them; this method only records the
        metadata snapshot that the reference keeps for cached replays
        (`deep_ep/buffers/ep.py:100-160`) and verifies the order when `EP_CHECK_DETERMINISTIC=1`.
        """
        if not is_cached_dispatch:
            self.cached_recv_src_metadata_before_sort = self.recv_src_metadata
        assert self.cached_recv_src_metadata_before_sort is not None
        if is_cached_dispatch or os.environ.get('EP_CHECK_DETERMINISTIC', '0') != '1':
            return
        num_recv = int(self.psum_num_recv_tokens_per_rank[-1])
        meta = self.recv_src_metadata[:num_recv]
        slots, src = meta[:, :-2], meta[:, -2]
        starts = (self.psum_num_recv_tokens_per_expert - self.num_unaligned_recv_tokens_per_expert).long()
        valid = slots >= 0
        expert_of_slot = torch.bucketize(slots[valid].long(), starts[1:].contiguous(), right=True)
        keys = expert_of_slot * (1 << 32) + src.unsqueeze(1).expand_as(slots)[valid].long()
        order = torch.argsort(slots[valid].long())
        assert bool((keys[order][1:] >= keys[order][:-1]).all()), 'expanded rows are not in source-token order'


class EPBuffer(BufferBase):
    """Expert-parallel dispatch/combine over one NVLink domain, expanded layout.

    Stream usage: every operation runs on the current stream.
    """

    barrier = comm.barrier
    get_comm_stream = comm.get_comm_stream
    get_physical_domain_size = comm.get_physical_domain_size
    get_logical_domain_size = comm.get_logical_domain_size

    def __init__(self, group: dist.ProcessGroup, num_bytes: Optional[int] = None,
                 num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 0,
                 use_fp8_dispatch: bool = False,
                 lb_allocation_plan_or_num_bytes: Union[BufferAllocator, int] = 0,
                 deterministic: bool = False, allow_hybrid_mode: bool = True,
                 allow_multiple_reduction: bool = True, prefer_overlap_with_compute: bool = True,
                 sl_idx: Optional[int] = None, num_allocated_qps: int = 0,
                 num_cpu_timeout_secs: int = 300, num_gpu_timeout_secs: int = 100,
                 explicitly_destroy: bool = False, *, use_huge1g_page: bool = True):
        """Create the buffer (collective over `group`).

        `num_bytes` excludes the workspace and must be 2 MiB aligned; when `None` it is derived from
        `num_max_tokens_per_rank`, `hidden`, `num_topk` and `use_fp8_dispatch`. Hybrid mode and the
        overlap preference are accepted for compatibility; service levels and explicit queue-pair
        counts do not exist on NVLink and are rejected.
        """
        lb_plan = lb_allocation_plan_or_num_bytes if isinstance(lb_allocation_plan_or_num_bytes, BufferAllocator) else None
        num_lb_bytes = lb_allocation_plan_or_num_bytes if lb_plan is None else lb_plan.num_bytes
        if lb_plan is not None:
            assert not lb_plan.materialized
        alignment = _C.get_num_allocation_alignment()
        assert isinstance(num_lb_bytes, int) and num_lb_bytes >= 0 and num_lb_bytes % alignment == 0
        if sl_idx is not None or num_allocated_qps != 0:
            raise NotImplementedError('RDMA service levels and QP configuration do not exist on NVLink')
        assert allow_multiple_reduction, 'per-rank pre-reduction is the only combine mode'
        assert num_cpu_timeout_secs > 0 and num_gpu_timeout_secs > 0

        self.group = group
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.allow_hybrid_mode = allow_hybrid_mode
        self.allow_multiple_reduction = allow_multiple_reduction
        self.prefer_overlap_with_compute = prefer_overlap_with_compute
        self.deterministic = deterministic
        self.use_fp8_dispatch = use_fp8_dispatch
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_allocated_qps = 0
        self.num_lb_bytes = num_lb_bytes
        if num_bytes is None:
            num_bytes = self.get_buffer_size_hint(group, num_max_tokens_per_rank, hidden, num_topk, use_fp8_dispatch,
                                                  allow_hybrid_mode, allow_multiple_reduction)
        assert num_bytes >= 0 and num_bytes % alignment == 0
        self.num_bytes = num_bytes
        if os.environ.get('EP_BUFFER_DEBUG', 0):
            print(f'Initializing EP buffer with {num_bytes} bytes at rank EP {self.rank_idx}/{self.num_ranks}')

        # every rank must build the same buffer: a mismatch would corrupt peers' receive regions later
        configs = [None] * self.num_ranks
        dist.all_gather_object(configs, (num_bytes, num_lb_bytes, num_max_tokens_per_rank), group)
        assert all(c == configs[0] for c in configs), f'EPBuffer arguments differ across ranks: {configs}'

        self.comm_handle = comm.get_comm_handle(group)
        super().__init__(explicitly_destroy)
        self.is_simulated = not torch.cuda.is_available()
        if self.is_simulated:
            from ..sim.ep import SimEPRuntime
            self.runtime = SimEPRuntime(group, num_bytes, num_lb_bytes)
        else:
            self.runtime = _C.EPBuffer(self.rank_idx, self.num_ranks, self.comm_handle.get(), num_bytes, num_lb_bytes,
                                       use_huge1g_page, num_cpu_timeout_secs, num_gpu_timeout_secs, explicitly_destroy)
            connect_peers(self.runtime.context, group)
        self.context = self.runtime.context
        if lb_plan is not None:
            lb_plan.materialize(self.runtime.lb_storage)
        self.num_scaleout_ranks, self.num_scaleup_ranks = self.get_logical_domain_size()
        self.scaleout_rank_idx = self.rank_idx // self.num_scaleup_ranks
        self.scaleup_rank_idx = self.rank_idx % self.num_scaleup_ranks
        self.num_rdma_ranks, self.num_nvlink_ranks = self.get_physical_domain_size()
        sync_group(group)

    def destroy(self) -> None:
        super().destroy()
        self.context = None
        self.comm_handle = None

    @staticmethod
    def get_buffer_size_hint(group: dist.ProcessGroup, num_max_tokens_per_rank: int, hidden: int,
                             num_topk: int = 0, use_fp8_dispatch: bool = False,
                             allow_hybrid_mode: bool = True, allow_multiple_reduction: bool = True) -> int:
        """Recommended `num_bytes` (2 MiB aligned): max of the dispatch and combine landing areas."""
        assert allow_multiple_reduction
        return _C.calculate_ep_buffer_size(group.size(), num_max_tokens_per_rank, hidden, num_topk, use_fp8_dispatch)

    @staticmethod
    def capture() -> EventHandle:
        """Record an event on the current stream."""
        return EventHandle()

    def get_theoretical_num_sms(self, num_experts: int, num_topk: int, num_scaleout_topk: int = 0,
                                rdma_gbs: float = 0, nvlink_gbs: float = 0,
                                sm_read_gbs: float = 0, sm_write_gbs: float = 0) -> int:
        """Default SM budget of one dispatch/combine kernel."""
        return _C.get_num_sms()

    def get_theoretical_num_qps(self, num_sms: int) -> int:
        return 0

    # ------------------------------------------------------------------------------------------
    @nvtx_range('deep_ep.EPBuffer.dispatch')
    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]],
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                 cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                 num_experts: Optional[int] = None, num_max_tokens_per_rank: Optional[int] = None,
                 expert_alignment: Optional[int] = None, num_sms: int = 0, num_qps: int = 0,
                 previous_event: Optional[EventHandle] = None, async_with_compute_stream: bool = False,
                 allocate_on_comm_stream: bool = False, handle: Optional[EPHandle] = None,
                 do_handle_copy: bool = False, do_cpu_sync: Optional[bool] = None, do_expand: bool = False,
                 do_zero_padding: bool = False, use_tma_aligned_col_major_sf: bool = False,
                 defer_epilogue: bool = False, *, fused_fp8_quant: Union[bool, str] = False):
        """Send every token to the ranks that own its selected experts.

        Arguments:
            x: `[num_tokens, hidden]` bf16, or `(x_fp8 [num_tokens, hidden] e4m3, sf [num_tokens, num_sf_packs])`
                with 2-byte scale-factor packs, row- or column-major.
            topk_idx: `[num_tokens, num_topk]` int64, -1 = no selection. Must be `None` with `handle`.
            topk_weights: `[num_tokens, num_topk]` fp32 or `None`; may be given with a cached handle.
            cumulative_local_expert_recv_stats: `[num_local_experts]` int32 counter that the kernel increments.
            num_experts, num_max_tokens_per_rank, expert_alignment: layout parameters (taken from `handle` if cached).
            num_sms: SMs to use (0 = default). Cached dispatch always uses `handle.num_sms`.
            previous_event: the current stream waits for it before the kernel starts.
            async_with_compute_stream: also return an event recorded after the enqueued work.
            handle: cached `EPHandle`; routing layout is reused and only payloads move.
            do_cpu_sync: wait on the host for exact receive counts and size the outputs exactly
                (default True, False with `handle`). Without it outputs have worst-case capacity and nothing
                blocks the host, which is the CUDA-graph friendly mode.
            do_expand: must be True.
            do_zero_padding: zero the alignment padding rows of x, SF and weights.
            use_tma_aligned_col_major_sf: return SF with strides `(1, num_expanded_tokens)`.
            defer_epilogue: return only an `EventOverlap`; `current_stream_wait()` then runs the host count
                wait and the expand kernel and returns `(recv_x, None, recv_topk_weights, handle)`.
            fused_fp8_quant: `x` is bf16 and is quantised to e4m3 with fp32 1x128 scales inside the kernel;
                the result is `(recv_x_fp8, recv_sf_fp32 [rows, hidden / 128])`. `'ue8m0'` rounds every scale up to a
                power of two (`2^ceil(log2(amax / 448))`, still delivered as fp32): the form that the hardware-scaled
                FP8 GEMM (`deep_ep.ops.grouped_gemm`) consumes directly.

        Returns `(recv_x | (recv_x, recv_sf), None, recv_topk_weights, handle, event)` or, deferred, the event.
        """
        if num_qps not in (None, 0):
            raise NotImplementedError('Explicit QP counts do not exist on NVLink')
        assert not do_handle_copy, '`do_handle_copy` must be False; handle copying is not supported'
        x, sf = x if isinstance(x, tuple) else (x, None)
        assert fused_fp8_quant in (False, True, 'ue8m0'), "`fused_fp8_quant` is False, True or 'ue8m0'"
        quant_mode = 2 if fused_fp8_quant == 'ue8m0' else int(bool(fused_fp8_quant))
        assert do_expand, 'only the expanded layout (`do_expand=True`) is implemented'

        if handle is not None:
            assert topk_idx is None
            assert handle.do_expand == do_expand
            assert do_cpu_sync is None or not do_cpu_sync, 'Cannot do CPU sync with cached handle'
            topk_idx = handle.topk_idx
            num_max_tokens_per_rank = value_or(num_max_tokens_per_rank, handle.num_max_tokens_per_rank)
            num_experts = value_or(num_experts, handle.num_experts)
            expert_alignment = value_or(expert_alignment, handle.expert_alignment)
            num_sms = handle.num_sms
            do_cpu_sync = False
            assert (num_experts, expert_alignment, num_max_tokens_per_rank) == \
                   (handle.num_experts, handle.expert_alignment, handle.num_max_tokens_per_rank)
            cached = (handle.num_recv_tokens, handle.num_expanded_tokens, handle.num_recv_tokens_per_expert_list,
                      handle.psum_num_recv_tokens_per_rank, handle.psum_num_recv_tokens_per_expert,
                      handle.num_unaligned_recv_tokens_per_expert, handle.dst_buffer_slot_idx, handle.dst_gsge_idx,
                      handle.recv_src_metadata)
        else:
            assert topk_idx is not None and num_experts is not None
            if num_sms == 0:
                num_sms = self.get_theoretical_num_sms(num_experts, topk_idx.size(1))
            cached = (None,) * 9
        num_max_tokens_per_rank = value_or(num_max_tokens_per_rank, self.num_max_tokens_per_rank)
        expert_alignment = value_or(expert_alignment, 1)
        do_cpu_sync = value_or(do_cpu_sync, True)

        result, event, deferred_epilogue = self.runtime.dispatch(
            x, sf, topk_idx, topk_weights, cumulative_local_expert_recv_stats, *cached,
            num_max_tokens_per_rank, num_experts, expert_alignment, num_sms, previous_event,
            async_with_compute_stream, allocate_on_comm_stream, do_handle_copy, do_cpu_sync, do_expand,
            do_zero_padding, use_tma_aligned_col_major_sf, defer_epilogue, quant_mode)
        event_overlap = EventOverlap(event)

        def finalize(dispatch_result: tuple, deterministic_by_hook: bool):
            nonlocal handle
            (recv_x, recv_sf, recv_topk_weights, num_recv_tokens, num_expanded_tokens, per_expert_list,
             psum_rank, psum_expert, num_unaligned, recv_src_metadata, dst_buffer_slot_idx, dst_gsge_idx) = dispatch_result
            is_cached = handle is not None
            if not is_cached:
                handle = EPHandle(do_expand, num_experts, expert_alignment, num_max_tokens_per_rank, num_sms, topk_idx,
                                  num_recv_tokens, num_expanded_tokens, per_expert_list, psum_rank, psum_expert,
                                  num_unaligned, recv_src_metadata, dst_buffer_slot_idx, dst_gsge_idx)
            if fused_fp8_quant and recv_sf is not None:
                recv_sf = recv_sf.view(torch.float32) if recv_sf.stride(1) == 1 else recv_sf
            if self.deterministic:
                det = functools.partial(handle.deterministic_sort, do_cpu_sync, is_cached, recv_x, recv_sf, recv_topk_weights)
                if deterministic_by_hook:
                    event_overlap.register_hook_after_wait(det)
                else:
                    det()
            out_x = (recv_x, recv_sf) if recv_sf is not None else recv_x
            return out_x, None, recv_topk_weights, handle

        if deferred_epilogue is not None:
            event_overlap.register_hook_after_wait(lambda: finalize(deferred_epilogue(), False))
            return event_overlap
        assert result is not None
        return *finalize(result, async_with_compute_stream), event_overlap

    # ------------------------------------------------------------------------------------------
    @nvtx_range('deep_ep.EPBuffer.combine')
    def combine(self, x: torch.Tensor, handle: EPHandle, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[None, torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = None,
                num_sms: int = 0, num_qps: int = 0, previous_event: Optional[EventHandle] = None,
                async_with_compute_stream: bool = False, allocate_on_comm_stream: bool = False,
                defer_epilogue: bool = False, *, fused_single_rows: bool = False, apply_weights: bool = False):
        """Reduce expert outputs back to the ranks that own the tokens.

        Arguments:
            x: `[num_expanded_tokens, hidden]` bf16 expert outputs in the expanded layout.
            handle: the handle of the matching dispatch.
            topk_weights: `[num_expanded_tokens]` fp32 or `None`; routed back positionally, never multiplied in.
            bias: `None`, one tensor or a tuple of two `[num_tokens, hidden]` bf16 tensors added before the partials.
            num_sms: ignored, combine uses `handle.num_sms`.
            apply_weights: multiply every expanded row by its entry of `topk_weights` inside the kernel, before the
                fp32 sum (the reference never multiplies weights in; off by default). The weights are still routed back.
            fused_single_rows: the rows of `x` that are their token's only row on this rank were not written to `x`
                but stored by the producing GEMM straight into the owners' landing slots (`build_combine_route`);
                combine then sends only the routed weights for them.
            defer_epilogue: return only the event; `current_stream_wait()` runs the reduction and returns
                `(combined_x, combined_topk_weights)`.

        Returns `(combined_x, combined_topk_weights | None, event)` or, deferred, the event. The sum of one
        token is `bf16(fp32(bias_0) + fp32(bias_1) + sum over destination ranks, in top-k slot order, of
        bf16(fp32 sum of that rank's rows in top-k order))`.
        """
        if num_qps not in (None, 0):
            raise NotImplementedError('Explicit QP counts do not exist on NVLink')
        assert handle.recv_src_metadata is not None
        if isinstance(bias, torch.Tensor):
            bias_0, bias_1 = bias, None
        elif bias is None:
            bias_0 = bias_1 = None
        else:
            assert len(bias) == 2
            bias_0, bias_1 = bias
        result, event, deferred_epilogue = self.runtime.combine(
            x, topk_weights, bias_0, bias_1, handle.recv_src_metadata, handle.topk_idx,
            handle.psum_num_recv_tokens_per_rank, handle.num_experts, handle.num_max_tokens_per_rank,
            handle.num_sms, previous_event, async_with_compute_stream, allocate_on_comm_stream, defer_epilogue,
            fused_single_rows, apply_weights)
        event_overlap = EventOverlap(event)
        if deferred_epilogue is not None:
            event_overlap.register_hook_after_wait(deferred_epilogue)
            return event_overlap
        assert result is not None
        combined_x, combined_topk_weights = result
        return combined_x, combined_topk_weights, event_overlap

    # ------------------------------------------------------------------------------------------
    def build_combine_route(self, handle: EPHandle, hidden: int) -> torch.Tensor:
        """Destination table for a GEMM that produces the `x` of the next `combine` with this handle.

        `route[r]` (`hidden` = columns of the rows to come; int64 device addresses, 0 = none) tells the GEMM epilogue (`route=` of
        `deep_ep.ops.grouped_gemm.grouped_gemm_forward` / `grouped_gemm_dgrad`) to store expanded row r directly into
        the combine landing slot of its token's owner, local or over NVLink, instead of its output tensor. That is
        possible for tokens with exactly one row on this rank, whose combine message is the row itself; the transfer
        then overlaps the GEMM tile by tile. Afterwards call `combine(x, handle, ..., fused_single_rows=True)`.
        Call `barrier()` on this buffer between the dispatch that produced `handle` and the GEMM that uses the table.
        """
        assert not self.is_simulated, 'GEMM epilogues that store into landing slots exist on CUDA only'
        return self.runtime.build_combine_route(handle.recv_src_metadata, handle.psum_num_recv_tokens_per_rank,
                                                int(handle.num_expanded_tokens), handle.num_max_tokens_per_rank, hidden)

    # ------------------------------------------------------------------------------------------ diagnostics
    _TRACE_PHASES = {
        'dispatch': ('count', 'entry_barrier', 'grid_sync', 'count_exchange', 'push', 'stores_complete', 'flags_and_tail'),
        'expand': ('wait_arrival', 'layout', 'copy'),
        'combine': ('entry_barrier', 'grid_sync', 'push', 'stores_complete', 'flags_and_tail'),
        'reduce': ('wait_arrival', 'reduce'),
    }

    def enable_phase_trace(self) -> None:
        """From now on the four EP kernels record time stamps at their phase boundaries (a few stores per kernel)."""
        assert not self.is_simulated, 'the phase trace exists for the CUDA kernels only'
        self._phase_trace = self.runtime.enable_phase_trace()

    def disable_phase_trace(self) -> None:
        self.runtime.disable_phase_trace()
        self._phase_trace = None

    def read_phase_trace(self) -> dict:
        """Durations in microseconds of the phases of the most recent dispatch / expand / combine / reduce kernels, as
        seen by CTA 0 (`flags_and_tail` ends when the last CTA has released the completion flags). Synchronises."""
        assert getattr(self, '_phase_trace', None) is not None, 'call enable_phase_trace() first'
        torch.cuda.synchronize()
        stamps = self._phase_trace.cpu().tolist()
        out = {}
        for row, (kernel, phases) in zip(stamps, self._TRACE_PHASES.items()):
            out[kernel] = {name: (row[i + 1] - row[i]) / 1e3 for i, name in enumerate(phases) if row[i] and row[i + 1]}
            last = max(row)
            if row[0] and last:
                out[kernel]['total'] = (last - row[0]) / 1e3
        order = [(name, stamps[i][0]) for i, name in enumerate(self._TRACE_PHASES) if stamps[i][0]]
        for (a, ta), (b, tb) in zip(order, order[1:]):
            out[f'{a}_start_to_{b}_start'] = (tb - ta) / 1e3
        return out

    def lb_get_theoretical_num_sms(self) -> int:
        return _C.get_num_sms()

    def lb_prefetch_weights(self, redundant_expert_weights: Union[Sequence[torch.Tensor], torch.Tensor],
                            expert_weights: Union[Sequence[torch.Tensor], torch.Tensor],
                            redundancy_mapping: torch.Tensor, num_sms: int = 0,
                            previous_event: Optional[EventHandle] = None) -> EventOverlap:
        """Push local expert weights into the redundant-expert slots that peers requested (collective).

        `redundant_expert_weights[i]` is `[num_redundant_experts, *shape]` inside this buffer's LB region,
        `expert_weights[i]` is `[num_local_experts, *shape]`, `redundancy_mapping [num_ranks, num_redundant]`
        int32 holds the global expert id wanted in each slot (-1 = empty) and is identical on all ranks.
        """
        as_list = lambda t: [t] if isinstance(t, torch.Tensor) else list(t)
        redundant, local = as_list(redundant_expert_weights), as_list(expert_weights)
        assert redundant and len(redundant) == len(local) and all(t is not None for t in redundant + local)
        return EventOverlap(self.runtime.lb_prefetch_weights(redundant, local, redundancy_mapping, num_sms, previous_event))

    def lb_reduce_grads(self, redundant_expert_grads: torch.Tensor, expert_grads: torch.Tensor,
                        redundancy_mapping: torch.Tensor, num_sms: int = 0,
                        previous_event: Optional[EventHandle] = None) -> EventOverlap:
        """Add the gradients of redundant expert copies held by peers into this rank's `expert_grads` (collective)."""
        return EventOverlap(self.runtime.lb_reduce_grads(redundant_expert_grads, expert_grads, redundancy_mapping, num_sms,
                                                         previous_event))
