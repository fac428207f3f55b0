"""Synthetic gating scores with a controllable rank imbalance (reference: `deep_ep/utils/gate.py:1-180`).

"Imbalance ratio" = how many (rank-deduplicated) tokens rank 0 receives relative to the average of the
other ranks. The *random* generator scales the scores of rank 0's experts by a factor found by bisection;
the *precise* generator first fixes, per token, how many experts go to each rank and then fills in
experts and scores, which hits the ratio within a few percent and keeps the other ranks equal.
"""
from typing import Optional

import torch

from .envs import default_device


def _dev(device: Optional[torch.device]) -> torch.device:
    return device if device is not None else default_device()


def generate_topk_idx(rank_count: torch.Tensor, num_tokens: int, num_experts: int, num_ranks: int,
                      num_topk: int) -> torch.Tensor:
    """Pick, for every token and rank, `rank_count[token, rank]` distinct random experts of that rank."""
    dev = rank_count.device
    assert rank_count.shape == (num_tokens, num_ranks)
    assert bool((rank_count.sum(dim=1) == num_topk).all())
    per_rank = num_experts // num_ranks
    shuffled = torch.rand(num_tokens, num_ranks, per_rank, device=dev).argsort(dim=-1)
    experts = shuffled + (torch.arange(num_ranks, device=dev) * per_rank).view(1, num_ranks, 1)
    keep = torch.arange(per_rank, device=dev).view(1, 1, per_rank) < rank_count.unsqueeze(-1)
    return experts[keep].view(num_tokens, num_topk)


def generate_rank_count(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                        device: Optional[torch.device] = None) -> torch.Tensor:
    """`[num_tokens, num_ranks]` int32: experts per (token, rank); rank 0 is hit by `ratio` x as many tokens."""
    assert ratio >= 1.0, 'ratio must be no less than 1.0'
    dev = _dev(device)
    per_rank = num_experts // num_ranks
    others = num_ranks - 1
    # number of distinct ranks a token touches, drawn from what uniform routing would give
    sample = torch.rand(num_tokens, num_experts, device=dev).topk(num_topk, dim=1).indices // per_rank
    sorted_ranks = sample.sort(dim=1).values
    distinct = (sorted_ranks[:, 1:] != sorted_ranks[:, :-1]).sum(dim=1) + 1
    min_ranks = max(1, -(-num_topk // per_rank))
    max_ranks = min(num_topk, num_ranks, int(others / ratio) + 1)
    distinct = distinct.clamp(min_ranks, max(max_ranks, min_ranks))

    # hits per rank: total = h0 + others * h, with h0 = ratio * h
    total_hits = int(distinct.sum())
    h = total_hits / (others + ratio) if others > 0 else 0
    want_special = min(num_tokens, int(round(ratio * h))) if others > 0 else num_tokens
    must = distinct >= num_ranks                      # tokens that touch every rank necessarily touch rank 0
    want_special = max(want_special, int(must.sum()))
    optional = (~must).nonzero(as_tuple=True)[0]
    chosen = optional[torch.randperm(optional.numel(), device=dev)[:want_special - int(must.sum())]]
    special = must.clone()
    special[chosen] = True

    # the remaining (distinct - special) ranks of every token are dealt round-robin from one long random
    # cycle over ranks 1..n-1, which keeps those ranks equally loaded and distinct within a token
    need = (distinct - special.long()).clamp(min=0, max=others)
    starts = torch.cumsum(need, 0) - need
    hit = torch.zeros(num_tokens, num_ranks, dtype=torch.bool, device=dev)
    hit[:, 0] = special
    if others > 0:
        cycle = torch.randperm(others, device=dev) + 1
        slot = torch.arange(others, device=dev).view(1, -1)
        ranks = cycle[(starts.view(-1, 1) + slot) % others]
        active = slot < need.view(-1, 1)
        rows = torch.arange(num_tokens, device=dev).view(-1, 1).expand_as(ranks)
        hit[rows[active], ranks[active]] = True
    # a token whose only rank would be "none" (need == 0 and not special) falls back to rank 0
    empty = ~hit.any(dim=1)
    hit[empty, 0] = True

    # spread the num_topk experts over the touched ranks: one each, the rest round-robin, capped by per_rank
    count = hit.to(torch.int32)
    remaining = num_topk - count.sum(dim=1)
    touched = hit.sum(dim=1)
    order = torch.rand(num_tokens, num_ranks, device=dev).masked_fill(~hit, 2.0).argsort(dim=1)   # touched ranks first
    for step in range(num_topk):
        if int(remaining.max()) <= 0:
            break
        col = order[torch.arange(num_tokens, device=dev), step % touched.clamp(min=1)]
        can = (remaining > 0) & (count[torch.arange(num_tokens, device=dev), col] < per_rank)
        count[torch.arange(num_tokens, device=dev)[can], col[can]] += 1
        remaining = remaining - can.long()
    while int(remaining.max()) > 0:       # rare: caps hit during the round-robin, fill any touched rank with room
        room = hit & (count < per_rank)
        col = room.float().argmax(dim=1)
        can = (remaining > 0) & room.any(dim=1)
        if not bool(can.any()):
            break
        count[torch.arange(num_tokens, device=dev)[can], col[can]] += 1
        remaining = remaining - can.long()
    return count[torch.randperm(num_tokens, device=dev)]


def get_precise_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                                  device: Optional[torch.device] = None) -> torch.Tensor:
    """Scores whose top-k reproduces a rank-count plan exactly (synthetic; not a realistic score distribution)."""
    dev = _dev(device)
    rank_count = generate_rank_count(num_tokens, num_experts, num_ranks, num_topk, ratio, dev)
    threshold = 0.9
    scores = torch.empty((num_tokens, num_experts), dtype=torch.float32, device=dev).uniform_(0, threshold)
    topk_idx = generate_topk_idx(rank_count, num_tokens, num_experts, num_ranks, num_topk)
    high = torch.empty((num_tokens, num_topk), dtype=torch.float32, device=dev).uniform_(threshold + 1e-6, 1.0)
    scores.scatter_(1, topk_idx, high)
    return scores


def get_scores_by_factor(num_tokens: int, num_experts: int, num_ranks: int, factor: float,
                         device: Optional[torch.device] = None) -> torch.Tensor:
    """Uniform scores, those of rank 0's experts stretched to `[0, factor)`."""
    dev = _dev(device)
    per_rank = num_experts // num_ranks
    scores = torch.rand((num_tokens, num_experts), dtype=torch.float32, device=dev)
    scores[:, :per_rank] *= factor
    return scores


def map_unbalanced_ratio_to_factor(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                                   device: Optional[torch.device] = None) -> float:
    """Bisection on the stretch factor until rank 0 receives about `ratio` x the other ranks' mean."""
    lo, hi = 1.0, 100.0
    per_rank = num_experts // num_ranks
    for _ in range(20):
        mid = (lo + hi) / 2
        idx = get_scores_by_factor(num_tokens, num_experts, num_ranks, mid, device).topk(num_topk, dim=-1).indices
        hits = torch.nn.functional.one_hot(idx // per_rank, num_ranks).any(dim=1).float().sum(dim=0)
        if hits[0].item() > hits[1:].mean().item() * ratio:
            hi = mid
        else:
            lo = mid
    return lo


def get_random_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                                 device: Optional[torch.device] = None) -> torch.Tensor:
    factor = 1.0 if ratio == 1.0 else map_unbalanced_ratio_to_factor(num_tokens, num_experts, num_ranks, num_topk, ratio, device)
    return get_scores_by_factor(num_tokens, num_experts, num_ranks, factor, device)


def get_unbalanced_scores(num_tokens: int, num_experts: int, num_ranks: int, num_topk: int, ratio: float,
                          precise: bool, device: Optional[torch.device] = None) -> torch.Tensor:
    if precise:
        return get_precise_unbalanced_scores(num_tokens, num_experts, num_ranks, num_topk, ratio, device)
    return get_random_unbalanced_scores(num_tokens, num_experts, num_ranks, num_topk, ratio, device)
