"""CPU restatement of the expert-parallel dispatch/combine semantics.

Two uses: (1) the oracle the GPU tests compare the sm_100a kernels against, and (2) the runtime
behind `EPBuffer` when the process group is a CPU (gloo) group, so that the public API can be
exercised end to end without a GPU. It is never selected for CUDA tensors.

The layout rules it implements are the ones documented for `EPHandle`
(reference: `deep_ep/buffers/ep.py:27-51`, `impls/ep/dispatch.hpp:167-292`,
`impls/ep/dispatch_copy_epilogue.hpp:450-545`, `impls/ep/combine_reduce_epilogue.hpp:100-140`):
a token travels once per destination rank; received rows are ordered by (source rank, source
token); each received token is expanded into one row per local expert it selected, expert regions
are padded to `expert_alignment`; the master top-k position of a rank is the last position that
selects it; combine sums in fp32 in top-k order with one rounding to bf16 per rank partial and one
for the final result.
"""
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils.math import align


@dataclass
class RankInput:
    x: torch.Tensor                       # [T, hidden] (bf16 / fp8 viewed as uint8 / any dtype on CPU)
    sf: Optional[torch.Tensor]            # [T, packs] or None
    topk_idx: torch.Tensor                # [T, k] int64
    topk_weights: Optional[torch.Tensor]  # [T, k] fp32 or None


@dataclass
class DispatchLayout:
    """Everything rank `rank` knows after a dispatch (handle fields + outputs)."""
    recv_rows_src: torch.Tensor           # [N] source rank of each received row
    recv_rows_token: torch.Tensor         # [N] source-local token index of each received row
    psum_num_recv_tokens_per_rank: torch.Tensor
    psum_num_recv_tokens_per_expert: torch.Tensor
    num_unaligned_recv_tokens_per_expert: torch.Tensor
    recv_src_metadata: torch.Tensor       # [N, k + 2]
    num_expanded_tokens: int


def rank_of_expert(topk_idx: torch.Tensor, num_local_experts: int) -> torch.Tensor:
    """Destination rank per top-k entry, -1 for masked entries."""
    return torch.where(topk_idx >= 0, topk_idx // num_local_experts, torch.full_like(topk_idx, -1))


def master_mask(topk_rank: torch.Tensor) -> torch.Tensor:
    """True where a top-k position is the LAST one that selects its destination rank."""
    num_topk = topk_rank.size(1)
    is_master = topk_rank >= 0
    for j in range(num_topk):
        for j2 in range(j + 1, num_topk):
            is_master[:, j] &= topk_rank[:, j] != topk_rank[:, j2]
    return is_master


def sender_slots(topk_idx: torch.Tensor, num_experts: int, num_ranks: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """`dst_buffer_slot_idx [T, k]` and per-destination send counts for one source rank.

    The slot of (token, destination rank) is the number of earlier tokens of this source that also
    go to that rank; it is stored at the master position, all other positions hold -1.
    """
    num_local_experts = num_experts // num_ranks
    topk_rank = rank_of_expert(topk_idx, num_local_experts)
    is_master = master_mask(topk_rank)
    slots = torch.full_like(topk_idx, -1, dtype=torch.int32)
    counts = torch.zeros(num_ranks, dtype=torch.int64)
    for r in range(num_ranks):
        hit = (is_master & (topk_rank == r))                  # [T, k], at most one True per row
        token_hits = hit.any(dim=1)
        order = torch.cumsum(token_hits.to(torch.int64), 0) - 1
        rows, cols = hit.nonzero(as_tuple=True)
        slots[rows, cols] = order[rows].to(torch.int32)
        counts[r] = int(token_hits.sum())
    return slots, counts


def receiver_layout(all_topk_idx: List[torch.Tensor], rank: int, num_experts: int, expert_alignment: int,
                    num_max_tokens_per_rank: int) -> DispatchLayout:
    """Layout on the receiving side of `rank`, from every source's `topk_idx`."""
    num_ranks = len(all_topk_idx)
    num_local_experts = num_experts // num_ranks
    num_topk = all_topk_idx[0].size(1)
    lo = rank * num_local_experts

    src_list, tok_list, local_idx_list = [], [], []
    per_rank_counts = []
    for s, idx in enumerate(all_topk_idx):
        local = torch.where((idx >= lo) & (idx < lo + num_local_experts), idx - lo, torch.full_like(idx, -1))
        hit = (local >= 0).any(dim=1)
        tokens = hit.nonzero(as_tuple=True)[0]
        src_list.append(torch.full_like(tokens, s))
        tok_list.append(tokens)
        local_idx_list.append(local[tokens])
        per_rank_counts.append(tokens.numel())
    rows_src = torch.cat(src_list) if src_list else torch.zeros(0, dtype=torch.int64)
    rows_tok = torch.cat(tok_list)
    local_idx = torch.cat(local_idx_list)                    # [N, k] local expert or -1
    num_recv = rows_src.numel()

    counts = torch.zeros(num_local_experts, dtype=torch.int64)
    if num_recv:
        valid = local_idx[local_idx >= 0]
        counts = torch.bincount(valid, minlength=num_local_experts)
    aligned = (counts + expert_alignment - 1) // expert_alignment * expert_alignment
    starts = torch.cumsum(aligned, 0) - aligned
    psum_expert = (starts + counts).to(torch.int32)

    # expanded slot of every (row, position): rows of an expert keep the stream order
    slots = torch.full((num_recv, num_topk), -1, dtype=torch.int32)
    running = starts.clone()
    for e in range(num_local_experts):
        rows, cols = (local_idx == e).nonzero(as_tuple=True)   # row-major order == stream order
        slots[rows, cols] = (running[e] + torch.arange(rows.numel())).to(torch.int32)
    positions = torch.arange(num_topk).view(1, -1).expand(num_recv, -1)
    master = torch.where(local_idx >= 0, positions, torch.full_like(positions, -1)).max(dim=1).values \
        if num_recv else torch.zeros(0, dtype=torch.int64)
    metadata = torch.empty((num_recv, num_topk + 2), dtype=torch.int32)
    metadata[:, :num_topk] = slots
    metadata[:, num_topk] = (rows_src * num_max_tokens_per_rank + rows_tok).to(torch.int32)
    metadata[:, num_topk + 1] = master.to(torch.int32)

    return DispatchLayout(
        recv_rows_src=rows_src, recv_rows_token=rows_tok,
        psum_num_recv_tokens_per_rank=torch.cumsum(torch.tensor(per_rank_counts, dtype=torch.int64), 0).to(torch.int32),
        psum_num_recv_tokens_per_expert=psum_expert,
        num_unaligned_recv_tokens_per_expert=counts.to(torch.int32),
        recv_src_metadata=metadata,
        num_expanded_tokens=int(aligned.sum()))


def expand(layout: DispatchLayout, inputs: List[RankInput], num_expanded_rows: int, zero_padding: bool,
           sf_col_major: bool = False):
    """Materialise `recv_x`, `recv_sf`, `recv_topk_weights` of the expanded layout."""
    ref = inputs[0]
    num_topk = ref.topk_idx.size(1)
    hidden = ref.x.size(1)
    make = torch.zeros if zero_padding else torch.empty
    recv_x = make((num_expanded_rows, hidden), dtype=ref.x.dtype)
    recv_sf = None
    if ref.sf is not None:
        packs = ref.sf.size(1)
        recv_sf = torch.zeros((num_expanded_rows, packs), dtype=ref.sf.dtype) if zero_padding else \
            torch.empty((num_expanded_rows, packs), dtype=ref.sf.dtype)
        if sf_col_major:
            recv_sf = torch.empty_strided((num_expanded_rows, packs), (1, num_expanded_rows), dtype=ref.sf.dtype).copy_(recv_sf)
    recv_w = None if ref.topk_weights is None else make((num_expanded_rows,), dtype=torch.float32)
    meta = layout.recv_src_metadata
    for row in range(meta.size(0)):
        s, t = int(layout.recv_rows_src[row]), int(layout.recv_rows_token[row])
        for j in range(num_topk):
            slot = int(meta[row, j])
            if slot < 0:
                continue
            recv_x[slot] = inputs[s].x[t]
            if recv_sf is not None:
                recv_sf[slot] = inputs[s].sf[t]
            if recv_w is not None:
                recv_w[slot] = inputs[s].topk_weights[t, j]
    return recv_x, recv_sf, recv_w


class _EpilogueTicket:
    """Marks a deferred epilogue as outstanding until it is run or dropped; the CUDA runtime refuses a second dispatch
    (or combine) while one is outstanding (`csrc/buffers/ep.hpp`), and so does this one."""

    def __init__(self, owner, kind: str):
        self.owner, self.kind, self.released = owner, kind, False
        owner._pending[kind] += 1

    def release(self) -> None:
        if not self.released:
            self.released = True
            self.owner._pending[self.kind] -= 1

    def __del__(self):
        self.release()


def combine_partials(x: torch.Tensor, topk_weights: Optional[torch.Tensor], metadata: torch.Tensor, num_topk: int,
                     apply_weights: bool = False):
    """Per received row: fp32 sum of its expanded rows in top-k order -> bf16, and the routed weights. With
    `apply_weights` every row is multiplied by its routing weight (fused multiply-add in fp32) before the sum."""
    slots = metadata[:, :num_topk].long()
    num_rows, hidden = metadata.size(0), x.size(1)
    acc = torch.zeros((num_rows, hidden), dtype=torch.float32)
    weights = torch.zeros((num_rows, num_topk), dtype=torch.float32)
    for j in range(num_topk):
        valid = slots[:, j] >= 0
        rows = valid.nonzero(as_tuple=True)[0]
        if apply_weights:
            acc[rows] = torch.addcmul(acc[rows], x[slots[rows, j]].float(), topk_weights[slots[rows, j]].unsqueeze(1))
        else:
            acc[rows] += x[slots[rows, j]].float()
        if topk_weights is not None:
            weights[rows, j] = topk_weights[slots[rows, j]]
    return acc.to(x.dtype), weights


def combine_reduce(partials_by_rank: List[Optional[torch.Tensor]], weights_by_rank: List[Optional[torch.Tensor]],
                   topk_idx: torch.Tensor, num_experts: int, bias: Tuple[Optional[torch.Tensor], Optional[torch.Tensor]],
                   with_weights: bool):
    """Owner-side reduction. `partials_by_rank[d][t]` is rank d's partial for local token t."""
    num_ranks = len(partials_by_rank)
    num_tokens, num_topk = topk_idx.shape
    hidden = next(p for p in partials_by_rank if p is not None).size(1)
    dtype = next(p for p in partials_by_rank if p is not None).dtype
    topk_rank = rank_of_expert(topk_idx, num_experts // num_ranks)
    is_master = master_mask(topk_rank)
    acc = torch.zeros((num_tokens, hidden), dtype=torch.float32)
    for b in bias:
        if b is not None:
            acc += b.float()
    for j in range(num_topk):
        rows = is_master[:, j].nonzero(as_tuple=True)[0]
        for d in range(num_ranks):
            sel = rows[topk_rank[rows, j] == d]
            if sel.numel():
                acc[sel] += partials_by_rank[d][sel].float()
    combined_weights = None
    if with_weights:
        combined_weights = torch.zeros((num_tokens, num_topk), dtype=torch.float32)
        for j in range(num_topk):
            for d in range(num_ranks):
                sel = (topk_rank[:, j] == d).nonzero(as_tuple=True)[0]
                if sel.numel():
                    combined_weights[sel, j] = weights_by_rank[d][sel, j]
    return acc.to(dtype), combined_weights


class SimEPRuntime:
    """Drop-in for the native `EPBuffer` runtime over a CPU process group (gloo).

    Every call is collective. Inputs are exchanged with `all_gather_object`; each rank then runs the
    functions above for itself. Deferred epilogues, events and handle tuples have the same shape as
    the native runtime's so the Python `EPBuffer` code path is identical.
    """

    class _Context:
        def __init__(self, rank_idx, num_ranks):
            self.rank_idx, self.num_ranks = rank_idx, num_ranks
            self.num_workspace_bytes = self.num_gpu_buffer_bytes = self.num_rdma_storage_bytes = 0

        def get_physical_domain_size(self):
            return 1, self.num_ranks

        def get_logical_domain_size(self):
            return 1, self.num_ranks

    def __init__(self, group: dist.ProcessGroup, num_bytes: int, num_lb_bytes: int):
        self.group = group
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.context = self.main_context = SimEPRuntime._Context(self.rank_idx, self.num_ranks)
        self.lb_storage = torch.zeros(num_lb_bytes, dtype=torch.uint8)
        self.destroyed = False
        self._pending = {'dispatch': 0, 'combine': 0}      # deferred epilogues handed out and not yet run

    def destroy(self):
        dist.barrier(self.group)
        self.destroyed = True

    def print_memory_usage(self):
        print(f'[deep_ep sim] rank {self.rank_idx}/{self.num_ranks}: CPU simulation, no device memory')

    def check_status(self):
        pass

    def _gather(self, obj):
        out = [None] * self.num_ranks
        dist.all_gather_object(out, obj, self.group)
        return out

    # ---- expert load balancing: `redundancy_mapping[r, c]` is the global expert held by redundant slot c of rank r (-1: free)
    def lb_prefetch_weights(self, redundant_expert_weights, expert_weights, redundancy_mapping, num_sms, previous_event):
        """Every redundant slot of this rank receives the weights of the expert the mapping assigns to it."""
        from ..utils.event import EventHandle
        assert not self.destroyed and len(redundant_expert_weights) == len(expert_weights) > 0
        mapping = redundancy_mapping.view(self.num_ranks, -1)
        for dst, src in zip(redundant_expert_weights, expert_weights):
            assert dst.size(0) == mapping.size(1) and dst.shape[1:] == src.shape[1:] and dst.dtype == src.dtype
            everyone = torch.cat([t for t in self._gather(src.detach().clone())])        # [num_ranks * local, ...]
            for c in range(mapping.size(1)):
                e = int(mapping[self.rank_idx, c])
                if e >= 0:
                    dst[c].copy_(everyone[e])
        dist.barrier(self.group)
        return EventHandle()

    def lb_reduce_grads(self, redundant_expert_grads, expert_grads, redundancy_mapping, num_sms, previous_event):
        """The owner of an expert adds the fp32 gradients of all its redundant copies, in slot order."""
        from ..utils.event import EventHandle
        assert not self.destroyed and expert_grads.dtype == torch.float32 and redundant_expert_grads.dtype == torch.float32
        mapping = redundancy_mapping.view(self.num_ranks, -1)
        num_local = expert_grads.size(0)
        assert redundant_expert_grads.shape == (mapping.size(1), expert_grads.size(1))
        everyone = self._gather(redundant_expert_grads.detach().clone())
        for r in range(self.num_ranks):
            for c in range(mapping.size(1)):
                e = int(mapping[r, c])
                if e >= 0 and e // num_local == self.rank_idx:
                    expert_grads[e % num_local] += everyone[r][c]
        dist.barrier(self.group)
        return EventHandle()

    def dispatch(self, x, sf, topk_idx, topk_weights, stats,
                 cached_num_recv_tokens, cached_num_expanded_tokens, cached_list,
                 cached_psum_rank, cached_psum_expert, cached_num_unaligned,
                 cached_dst_buffer_slot_idx, cached_dst_gsge_idx, cached_recv_src_metadata,
                 num_max_tokens_per_rank, num_experts, expert_alignment, num_sms, previous_event,
                 async_with_compute_stream, allocate_on_comm_stream, do_handle_copy, do_cpu_sync, do_expand,
                 do_zero_padding, use_col_major_sf, defer_epilogue, fused_fp8_quant):
        from ..utils.event import EventHandle
        from ..utils.math import per_token_cast_to_fp8
        assert do_expand and not do_handle_copy and not self.destroyed
        assert self._pending['dispatch'] == 0, \
            'the deferred epilogue of the previous dispatch on this buffer has not been run yet'
        cached = cached_recv_src_metadata is not None
        num_tokens, num_topk = topk_idx.shape
        assert num_tokens <= num_max_tokens_per_rank and num_experts % self.num_ranks == 0
        if fused_fp8_quant:
            x, scales = per_token_cast_to_fp8(x, round_scale=int(fused_fp8_quant) == 2)
            sf = scales.contiguous().view(torch.int16)
        x_wire = x.view(torch.uint8) if x.dtype == torch.float8_e4m3fn else x
        inputs = [RankInput(*item) for item in self._gather((x_wire, sf, topk_idx, topk_weights))]
        layout = receiver_layout([i.topk_idx for i in inputs], self.rank_idx, num_experts, expert_alignment,
                                 num_max_tokens_per_rank)
        num_local_experts = num_experts // self.num_ranks
        exact_recv = layout.recv_src_metadata.size(0)
        if cached:
            num_recv_tokens, num_expanded = cached_num_recv_tokens, cached_num_expanded_tokens
            per_expert_list = cached_list
            psum_rank, psum_expert, num_unaligned = cached_psum_rank, cached_psum_expert, cached_num_unaligned
            slot_idx, gsge_idx, metadata = cached_dst_buffer_slot_idx, cached_dst_gsge_idx, cached_recv_src_metadata
            layout.recv_src_metadata = metadata[:exact_recv]
        else:
            psum_rank, psum_expert = layout.psum_num_recv_tokens_per_rank, layout.psum_num_recv_tokens_per_expert
            num_unaligned = layout.num_unaligned_recv_tokens_per_expert
            slot_idx, _ = sender_slots(topk_idx, num_experts, self.num_ranks)
            gsge_idx = torch.full_like(slot_idx, -1)
            if stats is not None:
                stats += num_unaligned
            if do_cpu_sync:
                num_recv_tokens, num_expanded = exact_recv, layout.num_expanded_tokens
                per_expert_list = [align(int(c), expert_alignment) for c in num_unaligned]
                metadata = layout.recv_src_metadata
            else:
                num_recv_tokens = self.num_ranks * num_max_tokens_per_rank
                worst = num_recv_tokens * min(num_topk, num_local_experts) + (expert_alignment - 1) * num_local_experts
                num_expanded = align(worst, expert_alignment)
                per_expert_list = []
                metadata = torch.full((num_recv_tokens, num_topk + 2), -1, dtype=torch.int32)
                metadata[:exact_recv] = layout.recv_src_metadata

        ticket = _EpilogueTicket(self, 'dispatch')

        def epilogue():
            assert not ticket.released, 'this dispatch epilogue has already been run'
            ticket.release()
            recv_x, recv_sf, recv_w = expand(layout, inputs, num_expanded, do_zero_padding, use_col_major_sf)
            if x.dtype == torch.float8_e4m3fn:
                recv_x = recv_x.view(torch.float8_e4m3fn)
            return (recv_x, recv_sf, recv_w, num_recv_tokens, num_expanded, per_expert_list,
                    psum_rank, psum_expert, num_unaligned, metadata, slot_idx, gsge_idx)

        if defer_epilogue:
            assert async_with_compute_stream
            return None, EventHandle(), epilogue
        return epilogue(), (EventHandle() if async_with_compute_stream else None), None

    def combine(self, x, topk_weights, bias_0, bias_1, recv_src_metadata, topk_idx, psum_rank,
                num_experts, num_max_tokens_per_rank, num_sms, previous_event,
                async_with_compute_stream, allocate_on_comm_stream, defer_epilogue, skip_single_rows=False,
                apply_weights=False):
        from ..utils.event import EventHandle
        assert not skip_single_rows, 'GEMM epilogues that store into landing slots exist on CUDA only'
        assert not apply_weights or topk_weights is not None, 'a weighted combine needs `topk_weights`'
        assert self._pending['combine'] == 0, \
            'the deferred epilogue of the previous combine on this buffer has not been run yet'
        num_tokens, num_topk = topk_idx.shape
        num_recv = int(psum_rank[-1])
        metadata = recv_src_metadata[:num_recv]
        partials, weights = combine_partials(x, topk_weights, metadata, num_topk, apply_weights)
        src_global = metadata[:, num_topk].long()
        gathered = self._gather((partials, weights, src_global))

        ticket = _EpilogueTicket(self, 'combine')

        def epilogue():
            assert not ticket.released, 'this combine epilogue has already been run'
            ticket.release()
            partials_by_rank, weights_by_rank = [], []
            for d, (p, w, g) in enumerate(gathered):
                mine = (g // num_max_tokens_per_rank) == self.rank_idx
                tokens = (g[mine] % num_max_tokens_per_rank)
                pd = torch.zeros((num_tokens, x.size(1)), dtype=x.dtype)
                wd = torch.zeros((num_tokens, num_topk), dtype=torch.float32)
                pd[tokens], wd[tokens] = p[mine], w[mine]
                partials_by_rank.append(pd), weights_by_rank.append(wd)
            return combine_reduce(partials_by_rank, weights_by_rank, topk_idx, num_experts, (bias_0, bias_1),
                                  topk_weights is not None)

        if defer_epilogue:
            assert async_with_compute_stream
            return None, EventHandle(), epilogue
        return epilogue(), (EventHandle() if async_with_compute_stream else None), None
