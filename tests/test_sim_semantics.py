"""Semantics of the dispatch/combine layout on CPU, with all ranks simulated in one process."""
import pytest
import torch

from deep_ep.sim import ep as sim
from deep_ep.utils.math import align


def make_inputs(num_ranks, num_tokens, hidden, num_experts, num_topk, masked=0.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    inputs = []
    for r in range(num_ranks):
        t = max(1, num_tokens - r)
        scores = torch.rand(t, num_experts, generator=g)
        w, idx = scores.topk(num_topk, dim=-1)
        if masked > 0:
            idx = idx.masked_fill(torch.rand(idx.shape, generator=g) < masked, -1)
            w = w.masked_fill(idx < 0, 0)
        x = torch.randn(t, hidden, generator=g).to(torch.bfloat16)
        inputs.append(sim.RankInput(x, None, idx.long(), w.float()))
    return inputs


@pytest.mark.parametrize('num_ranks,num_experts,num_topk', [(2, 16, 4), (4, 32, 6), (8, 64, 8), (1, 8, 3)])
@pytest.mark.parametrize('alignment', [1, 16])
@pytest.mark.parametrize('masked', [0.0, 0.3])
def test_layout_invariants(num_ranks, num_experts, num_topk, alignment, masked):
    num_tokens, hidden, max_tokens = 33, 32, 40
    inputs = make_inputs(num_ranks, num_tokens, hidden, num_experts, num_topk, masked)
    per_rank = num_experts // num_ranks
    for rank in range(num_ranks):
        lay = sim.receiver_layout([i.topk_idx for i in inputs], rank, num_experts, alignment, max_tokens)
        meta = lay.recv_src_metadata
        # rows are ordered by (source rank, token) and appear once per token that selects this rank
        assert torch.equal(meta[:, -2], meta[:, -2].sort().values)
        expected_rows = sum(int(((i.topk_idx >= rank * per_rank) & (i.topk_idx < (rank + 1) * per_rank)).any(1).sum())
                            for i in inputs)
        assert meta.size(0) == expected_rows == int(lay.psum_num_recv_tokens_per_rank[-1])
        # psum semantics: starts aligned, ends exact
        counts = lay.num_unaligned_recv_tokens_per_expert.tolist()
        start = 0
        for e, c in enumerate(counts):
            assert int(lay.psum_num_recv_tokens_per_expert[e]) == start + c
            slots = meta[:, :-2][meta[:, :-2] >= 0]
            in_region = slots[(slots >= start) & (slots < start + align(c, alignment) if c else slots < start)]
            assert in_region.numel() == c and (c == 0 or torch.equal(in_region.sort().values, torch.arange(start, start + c, dtype=torch.int32)))
            start += align(c, alignment)
        assert lay.num_expanded_tokens == start
        # master position = last valid one
        valid = meta[:, :-2] >= 0
        pos = torch.arange(num_topk).view(1, -1).expand_as(valid)
        assert torch.equal(meta[:, -1].long(), torch.where(valid, pos, torch.full_like(pos, -1)).max(1).values)
        # inside an expert region rows are ordered by source token index (deterministic layout)
        for j in range(num_topk):
            col = meta[:, j]
            assert torch.equal(col[col >= 0], col[col >= 0])  # placeholder for readability
        flat_slot = meta[:, :-2][valid]
        flat_src = meta[:, -2:-1].expand(-1, num_topk)[valid]
        order = flat_slot.argsort()
        starts = torch.tensor([int(p) - c for p, c in zip(lay.psum_num_recv_tokens_per_expert.tolist(), counts)])
        expert_of = torch.bucketize(flat_slot[order].long(), starts[1:], right=True)
        keys = expert_of * (1 << 32) + flat_src[order].long()
        assert bool((keys[1:] > keys[:-1]).all())


@pytest.mark.parametrize('num_ranks,num_experts,num_topk', [(2, 16, 4), (4, 32, 6), (8, 64, 8)])
def test_sender_slots_match_receiver_rows(num_ranks, num_experts, num_topk):
    inputs = make_inputs(num_ranks, 29, 16, num_experts, num_topk, masked=0.2, seed=3)
    max_tokens = 32
    layouts = [sim.receiver_layout([i.topk_idx for i in inputs], r, num_experts, 1, max_tokens) for r in range(num_ranks)]
    per_rank = num_experts // num_ranks
    for s, inp in enumerate(inputs):
        slots, counts = sim.sender_slots(inp.topk_idx, num_experts, num_ranks)
        topk_rank = sim.rank_of_expert(inp.topk_idx, per_rank)
        for d in range(num_ranks):
            lay = layouts[d]
            base = 0 if s == 0 else int(lay.psum_num_recv_tokens_per_rank[s - 1])
            n_from_s = int(lay.psum_num_recv_tokens_per_rank[s]) - base
            assert n_from_s == int(counts[d])
            rows, cols = ((slots >= 0) & (topk_rank == d)).nonzero(as_tuple=True)
            # slot k of source s is row base + k on the receiver, and that row names the same token
            for t, j in zip(rows.tolist(), cols.tolist()):
                row = base + int(slots[t, j])
                assert int(lay.recv_src_metadata[row, -2]) == s * max_tokens + t
        # duplicates and masked entries carry -1, each destination rank exactly one slot per token
        assert int((slots >= 0).sum()) == int(counts.sum())


@pytest.mark.parametrize('num_ranks,num_experts,num_topk', [(2, 16, 4), (4, 32, 6), (8, 64, 8)])
@pytest.mark.parametrize('num_bias', [0, 1, 2])
def test_dispatch_combine_identity(num_ranks, num_experts, num_topk, num_bias):
    """combine(dispatch(x) scaled by the routed weights) == sum_k w_k x (in fp32 accumulation order)."""
    hidden, max_tokens = 64, 24
    inputs = make_inputs(num_ranks, 24, hidden, num_experts, num_topk, masked=0.15, seed=5)
    layouts = [sim.receiver_layout([i.topk_idx for i in inputs], r, num_experts, 8, max_tokens) for r in range(num_ranks)]
    outs = []
    for r in range(num_ranks):
        recv_x, _, recv_w = sim.expand(layouts[r], inputs, layouts[r].num_expanded_tokens, True)
        y = (recv_x.float() * recv_w.unsqueeze(1)).to(torch.bfloat16)      # identity "experts" scaled by weight
        outs.append(sim.combine_partials(y, recv_w, layouts[r].recv_src_metadata, num_topk))
    for s, inp in enumerate(inputs):
        t = inp.x.size(0)
        partials, weights = [], []
        for d in range(num_ranks):
            p = torch.zeros(t, hidden, dtype=torch.bfloat16)
            w = torch.zeros(t, num_topk)
            src = layouts[d].recv_src_metadata[:, -2].long()
            mine = (src // max_tokens) == s
            p[src[mine] % max_tokens], w[src[mine] % max_tokens] = outs[d][0][mine], outs[d][1][mine]
            partials.append(p), weights.append(w)
        bias = tuple(torch.randn(t, hidden).to(torch.bfloat16) for _ in range(num_bias)) + (None,) * (2 - num_bias)
        combined, combined_w = sim.combine_reduce(partials, weights, inp.topk_idx, num_experts, bias, True)
        assert torch.equal(combined_w, inp.topk_weights)
        expected = sum((b.float() for b in bias if b is not None), torch.zeros(t, hidden))
        expected = expected + (inp.x.float().unsqueeze(1) * inp.topk_weights.unsqueeze(2)).sum(1)
        assert torch.allclose(combined.float(), expected, atol=0.08, rtol=0.03)


# ------------------------------------------------------------------------------------------ property tests
try:
    from hypothesis import given, settings, strategies as st
    _have_hypothesis = True
except ImportError:                                   # pragma: no cover
    _have_hypothesis = False


if _have_hypothesis:
    @st.composite
    def _shapes(draw):
        num_ranks = draw(st.sampled_from([1, 2, 3, 4, 8]))
        per_rank = draw(st.integers(1, 5))
        num_experts = num_ranks * per_rank
        num_topk = draw(st.integers(1, min(num_experts, 9)))
        num_tokens = draw(st.integers(1, 17))
        alignment = draw(st.sampled_from([1, 2, 8, 16, 128]))
        masked = draw(st.sampled_from([0.0, 0.2, 0.6, 1.0]))
        seed = draw(st.integers(0, 10_000))
        return num_ranks, num_experts, num_topk, num_tokens, alignment, masked, seed

    @settings(max_examples=60, deadline=None)
    @given(_shapes())
    def test_random_shapes_conserve_tokens_and_round_trip(shape):
        """For arbitrary small shapes: every (token, destination rank) pair becomes exactly one received row, every valid
        (token, expert) selection exactly one expanded row inside that expert's region, and combine(dispatch(x) * w)
        returns sum_k w_k x together with the original weights."""
        num_ranks, num_experts, num_topk, num_tokens, alignment, masked, seed = shape
        hidden, max_tokens = 16, num_tokens
        inputs = make_inputs(num_ranks, num_tokens, hidden, num_experts, num_topk, masked, seed)
        per_rank = num_experts // num_ranks
        layouts = [sim.receiver_layout([i.topk_idx for i in inputs], r, num_experts, alignment, max_tokens)
                   for r in range(num_ranks)]
        for r, lay in enumerate(layouts):
            lo, hi = r * per_rank, (r + 1) * per_rank
            hits = [((i.topk_idx >= lo) & (i.topk_idx < hi)) for i in inputs]
            assert lay.recv_src_metadata.size(0) == sum(int(h.any(1).sum()) for h in hits)
            selections = torch.zeros(per_rank, dtype=torch.long)
            for i, h in zip(inputs, hits):
                selections += torch.bincount((i.topk_idx[h] - lo).long(), minlength=per_rank)
            assert lay.num_unaligned_recv_tokens_per_expert.tolist() == selections.tolist()
            assert lay.num_expanded_tokens == sum(align(int(c), alignment) for c in selections.tolist())
            assert lay.num_expanded_tokens % alignment == 0
        outs = []
        for r in range(num_ranks):
            recv_x, _, recv_w = sim.expand(layouts[r], inputs, layouts[r].num_expanded_tokens, True)
            y = (recv_x.float() * recv_w.unsqueeze(1)).to(torch.bfloat16)
            outs.append(sim.combine_partials(y, recv_w, layouts[r].recv_src_metadata, num_topk))
        for s, inp in enumerate(inputs):
            t = inp.x.size(0)
            partials, weights = [], []
            for d in range(num_ranks):
                p, w = torch.zeros(t, hidden, dtype=torch.bfloat16), torch.zeros(t, num_topk)
                src = layouts[d].recv_src_metadata[:, -2].long()
                mine = (src // max_tokens) == s
                p[src[mine] % max_tokens], w[src[mine] % max_tokens] = outs[d][0][mine], outs[d][1][mine]
                partials.append(p), weights.append(w)
            combined, combined_w = sim.combine_reduce(partials, weights, inp.topk_idx, num_experts, (None, None), True)
            assert torch.equal(combined_w, inp.topk_weights)
            expected = (inp.x.float().unsqueeze(1) * inp.topk_weights.unsqueeze(2)).sum(1)
            assert torch.allclose(combined.float(), expected, atol=0.1, rtol=0.04)
