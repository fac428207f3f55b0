"""Oracles built only on `torch.distributed` collectives: a non-expanded dispatch, the deterministic
pre-combine data pattern and the strict-order combine. They run unchanged on a gloo/CPU group and on
NCCL (reference: `deep_ep/utils/refs.py:1-247`); the dispatch oracle doubles as the
`all_to_all_single` baseline that the benchmarks compare against.
"""
import math
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .envs import get_global_seed


def dispatch(x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], topk_idx: torch.Tensor,
             topk_weights: Optional[torch.Tensor], num_max_tokens_per_rank: int, num_experts: int,
             group: Optional[dist.ProcessGroup] = None):
    """Rank-deduplicated token exchange, rows ordered by (source rank, source token).

    Returns `(recv_x | (recv_x, recv_sf), recv_topk_idx (local expert ids, -1 elsewhere), recv_topk_weights,
    recv_src_token_idx (= src_rank * num_max_tokens_per_rank + token), num_recv_tokens_per_rank)`.
    """
    rank, num_ranks = dist.get_rank(group), dist.get_world_size(group)
    assert num_experts % num_ranks == 0
    per_rank = num_experts // num_ranks
    x, sf = x if isinstance(x, tuple) else (x, None)
    num_tokens = x.size(0)
    dev = x.device

    dst_rank = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, -1))
    send_tokens: List[torch.Tensor] = [(dst_rank == r).any(dim=1).nonzero(as_tuple=True)[0] for r in range(num_ranks)]
    order = torch.cat(send_tokens)
    send_counts = [t.numel() for t in send_tokens]
    recv_counts_t = torch.empty(num_ranks, dtype=torch.int64, device=dev)
    dist.all_to_all_single(recv_counts_t, torch.tensor(send_counts, dtype=torch.int64, device=dev), group=group)
    recv_counts = recv_counts_t.tolist()
    total = sum(recv_counts)

    def exchange(t: torch.Tensor) -> torch.Tensor:
        payload = t[order].contiguous()
        out = torch.empty((total, *t.shape[1:]), dtype=t.dtype, device=dev)
        if t.dtype in (torch.int16, torch.float8_e4m3fn) and t.dim() == 2:
            # collective libraries do not know these element types: ship the rows as bytes
            dist.all_to_all_single(out.view(torch.uint8), payload.view(torch.uint8), recv_counts, send_counts, group=group)
        else:
            dist.all_to_all_single(out, payload, recv_counts, send_counts, group=group)
        return out

    recv_x = exchange(x)
    recv_sf = exchange(sf) if sf is not None else None
    recv_idx = exchange(topk_idx)
    recv_w = exchange(topk_weights) if topk_weights is not None else None
    src_idx = torch.arange(num_tokens, device=dev, dtype=torch.int32) + rank * num_max_tokens_per_rank
    recv_src = exchange(src_idx)

    lo = rank * per_rank
    mine = (recv_idx >= lo) & (recv_idx < lo + per_rank)
    recv_idx = torch.where(mine, recv_idx - lo, torch.full_like(recv_idx, -1))
    out_x = (recv_x, recv_sf) if sf is not None else recv_x
    return out_x, recv_idx, recv_w, recv_src, torch.tensor(recv_counts, dtype=torch.int)


def generate_pre_combine_data(src_token_global_idx: torch.Tensor, num_max_tokens_per_rank: int, num_topk: int,
                              hidden: int, num_ranks: Optional[int] = None) -> torch.Tensor:
    """Deterministic bf16 "expert outputs" `[n, num_topk, hidden]` that depend only on (global token, top-k slot).

    `y[i, j, c] = sin(((seed_ij * 131071 mod M) + 1) / M * (c + 1) + sin(global_seed))` with
    `seed_ij = src_token_global_idx[i] * num_topk + j` and `M = num_ranks * num_max_tokens_per_rank * num_topk`.
    """
    num_ranks = num_ranks if num_ranks is not None else dist.get_world_size()
    dev = src_token_global_idx.device
    seeds = src_token_global_idx.long().unsqueeze(1) * num_topk + torch.arange(num_topk, device=dev).unsqueeze(0)
    modulus = num_ranks * num_max_tokens_per_rank * num_topk
    phase = ((seeds * 131071 % modulus).float() + 1) / modulus
    cols = torch.arange(1, hidden + 1, device=dev, dtype=torch.float32).view(1, 1, hidden)
    return torch.sin(phase.unsqueeze(-1) * cols + math.sin(float(get_global_seed()))).to(torch.bfloat16)


def ordered_accumulate(data: torch.Tensor, initial_value: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 sum over dim 1 in index order (after `initial_value`), rounded once to `data.dtype`."""
    acc = torch.zeros((data.shape[0], data.shape[2]), dtype=torch.float32, device=data.device) \
        if initial_value is None else initial_value.clone()
    for j in range(data.shape[1]):
        acc += data[:, j].float()
    return acc.to(data.dtype)


def combine(y: torch.Tensor, topk_idx: torch.Tensor, num_experts: int,
            bias: Union[None, torch.Tensor, Tuple[torch.Tensor, ...]], reduce_in_local: bool,
            num_ranks: Optional[int] = None) -> torch.Tensor:
    """Strict-order combine of `y [num_tokens, num_topk, hidden]`.

    With `reduce_in_local`, the entries of one token that live on the same rank are first summed in fp32
    in top-k order and rounded to bf16; the rounded partial takes the place of the LAST such entry and the
    others become zero. Then bias (fp32) plus all entries are summed in top-k order and rounded once.
    """
    num_ranks = num_ranks if num_ranks is not None else dist.get_world_size()
    num_tokens, num_topk, hidden = y.shape
    per_rank = num_experts // num_ranks
    if reduce_in_local:
        group_id = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, -1))
        reduced = torch.zeros_like(y)
        for r in group_id.unique().tolist():
            member = group_id == r                                         # [T, k]
            acc = torch.zeros((num_tokens, hidden), dtype=torch.float32, device=y.device)
            for j in range(num_topk):
                acc += torch.where(member[:, j:j + 1], y[:, j].float(), torch.zeros_like(acc))
            positions = torch.arange(num_topk, device=y.device).view(1, -1).expand(num_tokens, -1)
            last = torch.where(member, positions, torch.full_like(positions, -1)).max(dim=1).values
            rows = (last >= 0).nonzero(as_tuple=True)[0]
            reduced[rows, last[rows]] = acc[rows].to(y.dtype)
        y = reduced
    bias_sum = None
    for b in (bias if isinstance(bias, tuple) else (bias,)):
        if b is not None:
            bias_sum = b.float() if bias_sum is None else bias_sum + b.float()
    return ordered_accumulate(y, bias_sum)
