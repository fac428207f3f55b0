"""Two CPU ranks over gloo: the public `EPBuffer` API against the `torch.distributed` oracles.

Configuration of the semantic baseline: 128 tokens per rank, hidden 256, fp32 tokens ~ N(0, 1), 16 experts
(8 per rank), top-4 from N(0, 1) gating logits with softmax weights over the selected logits.
"""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _worker(rank, world_size, deterministic):
    import deep_ep
    from deep_ep.utils import refs
    from deep_ep.utils.envs import init_seed
    from deep_ep.utils.math import align

    group = dist.group.WORLD
    init_seed(7)
    num_tokens, hidden, num_experts, num_topk, alignment = 128, 256, 16, 4, 8
    max_tokens = num_tokens
    x = torch.randn(num_tokens - rank, hidden)                       # fp32 payload; ranks differ in token count
    logits = torch.randn(x.size(0), num_experts)
    top_logits, topk_idx = logits.topk(num_topk, dim=-1)
    topk_weights = torch.softmax(top_logits, dim=-1)

    buffer = deep_ep.EPBuffer(group, num_max_tokens_per_rank=max_tokens, hidden=hidden, num_topk=num_topk,
                              deterministic=deterministic, explicitly_destroy=True)
    assert buffer.is_simulated and buffer.num_ranks == world_size
    stats = torch.zeros(num_experts // world_size, dtype=torch.int32)

    for defer in (False, True):
        out = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts,
                              cumulative_local_expert_recv_stats=stats if not defer else None,
                              expert_alignment=alignment, do_expand=True, do_zero_padding=True,
                              async_with_compute_stream=True, defer_epilogue=defer)
        if defer:
            recv_x, recv_idx, recv_w, handle = out.current_stream_wait()
        else:
            recv_x, recv_idx, recv_w, handle, event = out
            event.current_stream_wait()
        assert recv_idx is None

        ref_x, ref_idx, ref_w, ref_src, ref_counts = refs.dispatch(x, topk_idx, topk_weights, max_tokens, num_experts)
        meta = handle.recv_src_metadata
        assert handle.num_recv_tokens == ref_x.size(0) == meta.size(0)
        assert torch.equal(meta[:, -2], ref_src)                      # both are ordered by (src rank, token)
        valid = meta[:, :-2] >= 0
        assert torch.equal(valid, ref_idx >= 0)
        slots = meta[:, :-2][valid].long()
        assert torch.equal(recv_x[slots], ref_x.unsqueeze(1).expand(-1, num_topk, -1)[valid])
        assert torch.equal(recv_w[slots], ref_w[valid])
        counts = torch.bincount(ref_idx[ref_idx >= 0], minlength=num_experts // world_size)
        assert torch.equal(handle.num_unaligned_recv_tokens_per_expert.long(), counts)
        assert handle.num_recv_tokens_per_expert_list == [align(int(c), alignment) for c in counts]
        psum = [0] + handle.psum_num_recv_tokens_per_rank.tolist()
        assert [b - a for a, b in zip(psum, psum[1:])] == ref_counts.tolist()
        assert recv_x.size(0) == handle.num_expanded_tokens == sum(handle.num_recv_tokens_per_expert_list)
        if not defer:
            assert torch.equal(stats.long(), counts)

        # identity experts scaled by the routed weight, then combine: sum_k w_k x
        y = recv_x * recv_w.unsqueeze(1)
        combined, combined_w, _ = buffer.combine(y, handle, topk_weights=recv_w)
        assert torch.equal(combined_w, topk_weights)
        expected = (x.unsqueeze(1) * topk_weights.unsqueeze(2)).sum(1)
        assert torch.allclose(combined, expected, atol=1e-5, rtol=1e-5)
        # the same with the weights applied inside combine (opt-in; the reference's combine never multiplies them in)
        combined_in, combined_w_in, _ = buffer.combine(recv_x, handle, topk_weights=recv_w, apply_weights=True)
        assert torch.equal(combined_w_in, topk_weights)
        assert torch.allclose(combined_in, expected, atol=1e-5, rtol=1e-5)
        with pytest.raises(AssertionError):
            buffer.combine(recv_x, handle, apply_weights=True)             # needs the weights

        # cached replay with new payload and new weights keeps the handle and the layout
        x2, w2 = torch.randn_like(x), torch.rand_like(topk_weights)
        saved = [t.clone() for t in (handle.psum_num_recv_tokens_per_rank, handle.recv_src_metadata, handle.dst_buffer_slot_idx)]
        recv_x2, _, recv_w2, handle2, _ = buffer.dispatch(x2, topk_weights=w2, handle=handle, do_expand=True, do_zero_padding=True)
        assert handle2 is handle
        for t, s in zip((handle.psum_num_recv_tokens_per_rank, handle.recv_src_metadata, handle.dst_buffer_slot_idx), saved):
            assert torch.equal(t, s)
        combined2, combined_w2, _ = buffer.combine(recv_x2 * recv_w2.unsqueeze(1), handle, topk_weights=recv_w2)
        assert torch.equal(combined_w2, w2)
        assert torch.allclose(combined2, (x2.unsqueeze(1) * w2.unsqueeze(2)).sum(1), atol=1e-5, rtol=1e-5)
        recv_x3, _, recv_w3, _, _ = buffer.dispatch(x2, handle=handle, do_expand=True)
        assert recv_w3 is None

    # bf16 payload: combine must equal the strict-order oracle bit for bit
    xb = torch.randn(x.size(0), hidden).to(torch.bfloat16)
    recv_x, _, recv_w, handle, _ = buffer.dispatch(xb, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts,
                                                   do_expand=True, do_cpu_sync=False)
    assert handle.num_recv_tokens == world_size * max_tokens and handle.num_recv_tokens_per_expert_list == []
    num_recv = int(handle.psum_num_recv_tokens_per_rank[-1])
    meta = handle.recv_src_metadata[:num_recv]
    local_y = refs.generate_pre_combine_data(meta[:, -2], max_tokens, num_topk, hidden)
    y = torch.zeros(recv_x.size(0) + 1, hidden, dtype=torch.bfloat16)
    y[meta[:, :-2].long().flatten()] = local_y.view(-1, hidden)
    bias = (torch.randn(x.size(0), hidden).to(torch.bfloat16), torch.randn(x.size(0), hidden).to(torch.bfloat16))
    combined, _, _ = buffer.combine(y[:-1], handle, bias=bias)
    ref_y = refs.generate_pre_combine_data(rank * max_tokens + torch.arange(x.size(0)), max_tokens, num_topk, hidden)
    ref = refs.combine(ref_y, topk_idx, num_experts, bias, reduce_in_local=True)
    assert torch.equal(combined, ref)

    with pytest.raises(AssertionError):
        topk_idx.add_(0)
        handle.topk_idx
    buffer.destroy()


@pytest.mark.parametrize('deterministic', [False, True])
def test_ep_api_two_cpu_ranks(master_port, deterministic):
    run_distributed(_worker, 2, master_port, 'gloo', (deterministic,))


def _lb_worker(rank, world):
    """Expert load balancing on CPU ranks: redundant slots receive their experts' weights, owners collect the gradients."""
    import torch.distributed as dist
    import deep_ep
    num_local, num_redundant, hidden = 3, 2, 32
    plan = deep_ep.BufferAllocator()
    red_w = plan.allocate((num_redundant, 4, hidden), torch.bfloat16)
    red_g = plan.allocate((num_redundant, hidden), torch.float32)
    ep = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=8, hidden=hidden, num_topk=2,
                          lb_allocation_plan_or_num_bytes=plan, explicitly_destroy=True)
    assert ep.is_simulated
    torch.manual_seed(0)                                                   # the same mapping on every rank
    mapping = torch.randint(-1, world * num_local, (world, num_redundant), dtype=torch.int32)
    weights = torch.stack([torch.full((4, hidden), float(rank * num_local + e)) for e in range(num_local)]).to(torch.bfloat16)
    red_w.fill_(-5)
    ep.lb_prefetch_weights(red_w, weights, mapping).current_stream_wait()
    for c in range(num_redundant):
        e = int(mapping[rank, c])
        assert torch.all(red_w[c] == (e if e >= 0 else -5)), f'slot {c} expected expert {e}'

    red_g.copy_(torch.arange(num_redundant).view(-1, 1).float() + 10 * rank + 1)
    grads = torch.ones(num_local, hidden)
    ep.lb_reduce_grads(red_g, grads, mapping).current_stream_wait()
    for e in range(num_local):
        expect = 1.0 + sum(c + 10 * r + 1 for r in range(world) for c in range(num_redundant)
                           if int(mapping[r, c]) == rank * num_local + e)
        assert torch.all(grads[e] == expect), f'expert {e}: {grads[e, 0]} vs {expect}'
    ep.destroy()


def test_lb_two_cpu_ranks(master_port):
    run_distributed(_lb_worker, 2, master_port, 'gloo')


def _pending_epilogue_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=16, hidden=32, num_topk=2, explicitly_destroy=True)
    x = torch.randn(16, 32).to(torch.bfloat16)
    idx = torch.rand(16, 4 * world).topk(2, dim=-1).indices
    common = dict(topk_idx=idx, num_experts=4 * world, expert_alignment=1, do_expand=True, async_with_compute_stream=True)
    first = buffer.dispatch(x, defer_epilogue=True, **common)
    # the first dispatch's epilogue is still outstanding: a second dispatch would read the landing area, the epoch and the
    # host counts of the wrong call, so it is refused
    with pytest.raises((AssertionError, deep_ep.EPException)):
        buffer.dispatch(x, defer_epilogue=True, **common)
    recv_x, _, _, handle = first.current_stream_wait()
    second = buffer.dispatch(x, defer_epilogue=True, **common)            # fine once the hook has run
    second.current_stream_wait()
    dropped = buffer.dispatch(x, defer_epilogue=True, **common)           # a hook that is dropped releases its claim
    del dropped
    import gc
    gc.collect()
    combine_a = buffer.combine(recv_x, handle, async_with_compute_stream=True, defer_epilogue=True)
    with pytest.raises((AssertionError, deep_ep.EPException)):
        buffer.combine(recv_x, handle, async_with_compute_stream=True, defer_epilogue=True)
    combine_a.current_stream_wait()
    buffer.destroy()


def test_second_operation_is_refused_while_a_deferred_epilogue_is_pending(master_port):
    run_distributed(_pending_epilogue_worker, 2, master_port, 'gloo', timeout_s=120)


def _abort_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=8, hidden=32, num_topk=2, explicitly_destroy=True)
    buffer.abort(dist.group.WORLD)               # teardown without the collective barrier of destroy()
    assert buffer.runtime is None
    buffer.abort()                               # idempotent
    again = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=8, hidden=32, num_topk=2, explicitly_destroy=True)
    again.destroy()


def test_abort_releases_a_buffer_without_destroy(master_port):
    run_distributed(_abort_worker, 2, master_port, 'gloo', timeout_s=120)


def _handle_pickle_worker(rank, world):
    """A routing handle is plain data (integers, lists, tensors): it survives a pickle round trip and still drives a
    cached dispatch and a combine, which is all a checkpoint of this library's state would have to hold."""
    import pickle
    import torch.distributed as dist
    import deep_ep
    buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=16, hidden=32, num_topk=2, explicitly_destroy=True)
    torch.manual_seed(rank)
    x = torch.randn(16, 32).to(torch.bfloat16)
    idx = torch.rand(16, 4 * world).topk(2, dim=-1).indices
    common = dict(num_experts=4 * world, expert_alignment=1, do_expand=True)
    recv_x, _, _, handle, _ = buffer.dispatch(x, topk_idx=idx, **common)
    restored = pickle.loads(pickle.dumps(handle))
    assert torch.equal(restored.recv_src_metadata, handle.recv_src_metadata) and restored.num_sms == handle.num_sms
    assert torch.equal(restored.topk_idx, idx)
    again, _, _, same, _ = buffer.dispatch(x, handle=restored, do_expand=True)
    assert same is restored and torch.equal(again, recv_x)
    combined, _, _ = buffer.combine(again, restored)
    assert torch.allclose(combined.float(), 2 * x.float(), atol=2e-2, rtol=2e-2)
    buffer.destroy()


def test_handles_survive_a_pickle_round_trip(master_port):
    run_distributed(_handle_pickle_worker, 2, master_port, 'gloo', timeout_s=120)
