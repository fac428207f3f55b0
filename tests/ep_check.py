"""Correctness sweep of `EPBuffer.dispatch/combine` on GPUs against the `torch.distributed` oracles.

Mirrors the checks of the reference's `tests/ep/test_ep.py:47-388`: bitwise expanded payload/SF/weights,
slot uniqueness and ranges, per-rank and per-expert counts, psum semantics, statistics counter, zero
padding, master top-k index, bitwise combine (with 0/1/2 biases, with and without weights), cached
replays with new payloads/weights, and run-to-run determinism of the layout.
"""
import torch

import deep_ep
from deep_ep.utils import refs
from deep_ep.utils.gate import get_unbalanced_scores
from deep_ep.utils.math import align, per_token_cast_to_fp8


def enumerate_modes(quick: bool):
    for expert_alignment in (128, 1):
        for use_fp8 in (True, False):
            for num_bias in ((0, 2) if quick else (0, 1, 2)):
                for col_major in ((False, True) if use_fp8 else (False,)):
                    if quick and col_major and num_bias:
                        continue
                    yield expert_alignment, num_bias, use_fp8, col_major


def launch(buffer, name, defer, **params):
    result = getattr(buffer, name)(defer_epilogue=defer, **params)
    if defer:
        return *result.current_stream_wait(release_handle=True), result
    result[-1].current_stream_wait(release_handle=True)
    return result


def check_dispatch_combine(buffer: deep_ep.EPBuffer, num_tokens_max: int, hidden: int, num_topk: int, num_experts: int,
                           do_cpu_sync: bool = True, defer: bool = True, masked_ratio: float = 0.0,
                           unbalanced_ratio: float = 1.0, quick: bool = True, num_sms: int = 0, log=None):
    rank, num_ranks = buffer.rank_idx, buffer.num_ranks
    num_local_experts = num_experts // num_ranks
    num_tokens = max(1, num_tokens_max - rank)
    dev = torch.device('cuda', torch.cuda.current_device())

    scores = get_unbalanced_scores(num_tokens, num_experts, num_ranks, num_topk, unbalanced_ratio, False, device=dev)
    topk_weights, topk_idx = torch.topk(scores, num_topk, dim=-1, largest=True, sorted=False)
    topk_idx = topk_idx.to(torch.int64)
    if masked_ratio > 0:
        topk_idx.masked_fill_(torch.rand_like(topk_idx, dtype=torch.float) < masked_ratio, -1)
        topk_weights.masked_fill_(topk_idx < 0, 0)

    for expert_alignment, num_bias, use_fp8, col_major in enumerate_modes(quick):
        if log:
            log(f' > {expert_alignment=} {use_fp8=} {col_major=} {num_bias=} {do_cpu_sync=} {defer=}')
        x = torch.randn((num_tokens, hidden), dtype=torch.bfloat16, device=dev)
        if use_fp8:
            x_data, sf = per_token_cast_to_fp8(x)
            sf = sf.view(torch.int16)
            num_sf_packs = sf.size(1)
            if col_major:
                store = torch.empty((num_tokens * num_sf_packs,), dtype=torch.int16, device=dev)
                input_sf = torch.as_strided(store, (num_tokens, num_sf_packs), (1, num_tokens))
                input_sf.copy_(sf)
            else:
                input_sf = sf
            x = (x_data, input_sf)
        bias = None
        if num_bias == 1:
            bias = torch.randn((num_tokens, hidden), dtype=torch.bfloat16, device=dev)
        elif num_bias == 2:
            bias = tuple(torch.randn((num_tokens, hidden), dtype=torch.bfloat16, device=dev) for _ in range(2))

        stats = torch.zeros((num_local_experts,), dtype=torch.int, device=dev)
        dispatch_args = dict(x=x, topk_idx=topk_idx, topk_weights=topk_weights, num_sms=num_sms,
                             num_max_tokens_per_rank=num_tokens_max, num_experts=num_experts,
                             expert_alignment=expert_alignment, async_with_compute_stream=True,
                             do_cpu_sync=do_cpu_sync, do_expand=True, do_zero_padding=True,
                             use_tma_aligned_col_major_sf=col_major)
        ref_x = (x_data.view(torch.uint8), input_sf) if use_fp8 else x
        ref_recv_x, ref_recv_idx, ref_recv_w, ref_src, ref_counts = refs.dispatch(
            ref_x, topk_idx, topk_weights, num_tokens_max, num_experts, group=buffer.group)
        torch.cuda.synchronize()

        recv_x, recv_idx, recv_w, handle, event = launch(buffer, 'dispatch', defer,
                                                         cumulative_local_expert_recv_stats=stats, **dispatch_args)
        torch.cuda.synchronize()
        buffer.runtime.check_status()
        recv_x_data, recv_sf = recv_x if use_fp8 else (recv_x, None)
        check_x = recv_x_data.view(torch.uint8) if use_fp8 else recv_x_data
        if use_fp8:
            assert recv_sf.stride() == ((1, recv_x_data.size(0)) if col_major else (num_sf_packs, 1))

        num_recv = handle.psum_num_recv_tokens_per_rank[-1].item()
        num_expanded = align(handle.psum_num_recv_tokens_per_expert[-1].item(), expert_alignment)
        expected_rows = num_recv if do_cpu_sync else num_ranks * num_tokens_max
        assert handle.num_recv_tokens == expected_rows and handle.recv_src_metadata.size(0) == expected_rows
        assert recv_idx is None and recv_w is not None
        if do_cpu_sync:
            assert recv_x_data.size(0) == num_expanded == handle.num_expanded_tokens
        meta = handle.recv_src_metadata[:num_recv]

        # --- dispatch vs oracle (bitwise, through the metadata)
        ref_recv_x_data, ref_recv_sf = ref_recv_x if use_fp8 else (ref_recv_x, None)
        assert num_recv == ref_recv_x_data.size(0), f'{num_recv=} expected {ref_recv_x_data.size(0)}'
        slots, src = meta[:, :-2], meta[:, -2]
        assert torch.equal(src, ref_src), 'received rows must be ordered by (source rank, token)'
        valid = slots >= 0
        assert torch.equal(valid, ref_recv_idx >= 0)
        flat = slots[valid].long()
        assert flat.numel() == handle.num_unaligned_recv_tokens_per_expert.sum().item()
        if flat.numel():
            assert flat.min().item() >= 0 and flat.max().item() < num_expanded
            assert torch.unique(flat).numel() == flat.numel()
            assert torch.equal(check_x[flat], ref_recv_x_data.unsqueeze(1).expand(-1, num_topk, -1)[valid])
            if ref_recv_sf is not None:
                assert torch.equal(recv_sf[flat], ref_recv_sf.unsqueeze(1).expand(-1, num_topk, -1)[valid])
            assert torch.equal(recv_w[flat], ref_recv_w[valid])
        pos = torch.arange(num_topk, device=dev, dtype=meta.dtype).view(1, -1)
        assert torch.equal(meta[:, -1], torch.where(valid, pos, torch.full_like(slots, -1)).max(dim=1).values)

        psum_rank = [0] + handle.psum_num_recv_tokens_per_rank.tolist()
        assert [b - a for a, b in zip(psum_rank, psum_rank[1:])] == ref_counts.tolist()
        psum_expert = [0] + handle.psum_num_recv_tokens_per_expert.tolist()
        unaligned = handle.num_unaligned_recv_tokens_per_expert.tolist()
        stats_list = stats.tolist()
        for e in range(num_local_experts):
            start, end = align(psum_expert[e], expert_alignment), psum_expert[e + 1]
            ref_count = (ref_recv_idx == e).sum().item()
            assert end - start == ref_count == stats_list[e] == unaligned[e], f'{e=} {end - start=} {ref_count=}'
            if do_cpu_sync:
                assert handle.num_recv_tokens_per_expert_list[e] == align(ref_count, expert_alignment)
            expert_slots = slots[ref_recv_idx == e]
            if ref_count:
                # rows of one expert are in stream order, i.e. sorted by source token index
                assert torch.equal(expert_slots, torch.arange(start, end, device=dev, dtype=slots.dtype))
            pad_end = align(end, expert_alignment)
            assert torch.count_nonzero(recv_x_data[end:pad_end].view(torch.uint8)).item() == 0
            if recv_sf is not None:
                assert torch.count_nonzero(recv_sf[end:pad_end]).item() == 0
            assert torch.count_nonzero(recv_w[end:pad_end]).item() == 0
        own_slots = handle.dst_buffer_slot_idx
        assert own_slots.shape == topk_idx.shape and bool((handle.dst_gsge_idx == -1).all())

        # --- deterministic layout: a second dispatch gives the same rows
        recv_x_2, _, recv_w_2, handle_2, _ = launch(buffer, 'dispatch', defer, **dispatch_args)
        torch.cuda.synchronize()
        x2_data = (recv_x_2[0] if use_fp8 else recv_x_2)
        assert torch.equal((x2_data.view(torch.uint8) if use_fp8 else x2_data)[flat], check_x[flat])
        assert torch.equal(handle_2.recv_src_metadata[:num_recv], meta)
        assert torch.equal(handle_2.dst_buffer_slot_idx, own_slots)

        # --- combine vs oracle (bitwise)
        local_y = refs.generate_pre_combine_data(src, num_tokens_max, num_topk, hidden, num_ranks)
        y = torch.empty((recv_x_data.size(0) + 1, hidden), dtype=torch.bfloat16, device=dev)
        y[slots.long().flatten()] = local_y.view(-1, hidden)
        y = y[:-1]
        combined, combined_w, _ = launch(buffer, 'combine', defer, x=y, handle=handle, topk_weights=recv_w, bias=bias,
                                         async_with_compute_stream=True)
        torch.cuda.synchronize()
        buffer.runtime.check_status()
        ref_y = refs.generate_pre_combine_data(rank * num_tokens_max + torch.arange(num_tokens, device=dev),
                                               num_tokens_max, num_topk, hidden, num_ranks)
        ref_y[topk_idx == -1] = 0
        ref_combined = refs.combine(ref_y, topk_idx, num_experts, bias, True, num_ranks)
        diff = (combined.float() - ref_combined.float()).abs().max().item()
        assert torch.equal(combined, ref_combined), f'combine mismatch, max diff {diff}'
        assert torch.equal(combined_w, topk_weights)
        if num_bias == 0 and not col_major:
            combined_nw, w_nw, _ = launch(buffer, 'combine', defer, x=y, handle=handle, bias=bias, async_with_compute_stream=True)
            torch.cuda.synchronize()
            assert torch.equal(combined_nw, ref_combined) and w_nw is None

        # --- cached replays
        cached_args = dict(dispatch_args, handle=handle, num_sms=0, do_cpu_sync=False)
        del cached_args['topk_idx']
        cached_tensors = (handle.psum_num_recv_tokens_per_rank, handle.psum_num_recv_tokens_per_expert,
                          handle.num_unaligned_recv_tokens_per_expert, handle.recv_src_metadata,
                          handle.dst_buffer_slot_idx, handle.dst_gsge_idx)
        copies = [t.clone() for t in cached_tensors]
        padding_mask = torch.ones(num_expanded, dtype=torch.bool, device=dev)
        padding_mask[flat] = False
        order_meta, order_ref = torch.argsort(src), torch.argsort(ref_src)
        for send_weights in (True, False):
            new_x = torch.randn((num_tokens, hidden), dtype=torch.bfloat16, device=dev) * (8 if send_weights else 0.125)
            if use_fp8:
                new_data, new_sf = per_token_cast_to_fp8(new_x)
                new_sf = new_sf.view(torch.int16)
                if col_major:
                    new_sf = new_sf.t().contiguous().t()
                new_x = (new_data, new_sf)
            new_w = torch.randn_like(topk_weights).masked_fill_(topk_idx < 0, 0)
            ref_in = (new_data.view(torch.uint8), new_sf) if use_fp8 else new_x
            ref_cx, _, ref_cw, _, _ = refs.dispatch(ref_in, topk_idx, new_w, num_tokens_max, num_experts, group=buffer.group)
            cx, cidx, cw, chandle, _ = launch(buffer, 'dispatch', defer,
                                              **dict(cached_args, x=new_x, num_sms=0 if send_weights else handle.num_sms + 1,
                                                     topk_weights=new_w if send_weights else None))
            torch.cuda.synchronize()
            buffer.runtime.check_status()
            assert chandle is handle and cidx is None
            for t, c in zip(cached_tensors, copies):
                assert torch.equal(t, c)
            cx_data, csf = cx if use_fp8 else (cx, None)
            ref_cx_data, ref_csf = ref_cx if use_fp8 else (ref_cx, None)
            ccheck = cx_data.view(torch.uint8) if use_fp8 else cx_data
            assert torch.equal(ccheck[flat], ref_cx_data.unsqueeze(1).expand(-1, num_topk, -1)[valid])
            assert torch.count_nonzero(ccheck[:num_expanded][padding_mask]).item() == 0
            if csf is not None:
                assert torch.equal(csf[flat], ref_csf.unsqueeze(1).expand(-1, num_topk, -1)[valid])
                assert torch.count_nonzero(csf[:num_expanded][padding_mask]).item() == 0
            if send_weights:
                assert torch.equal(cw[flat], ref_cw[valid])
                assert torch.count_nonzero(cw[:num_expanded][padding_mask]).item() == 0
            else:
                assert cw is None
            ccomb, ccomb_w, _ = launch(buffer, 'combine', defer, x=y, handle=chandle, topk_weights=cw, bias=bias,
                                       async_with_compute_stream=True)
            torch.cuda.synchronize()
            assert torch.equal(ccomb, ref_combined)
            assert (torch.equal(ccomb_w, new_w) if send_weights else ccomb_w is None)


def check_fused_quant(buffer: deep_ep.EPBuffer, num_tokens_max: int, hidden: int, num_topk: int, num_experts: int):
    """Dispatch with in-kernel BF16 -> e4m3 quantisation equals quantise-then-dispatch bit for bit."""
    rank, num_ranks = buffer.rank_idx, buffer.num_ranks
    dev = torch.device('cuda', torch.cuda.current_device())
    num_tokens = max(1, num_tokens_max - rank)
    x = torch.randn((num_tokens, hidden), dtype=torch.bfloat16, device=dev) * 3
    x[0, :128] = 0         # an all-zero group exercises the amax clamp
    topk_idx = torch.rand(num_tokens, num_experts, device=dev).topk(num_topk, dim=-1).indices
    common = dict(topk_idx=topk_idx, num_experts=num_experts, num_max_tokens_per_rank=num_tokens_max,
                  expert_alignment=16, do_expand=True, do_zero_padding=True)
    (fx, fsf), _, _, fh, _ = buffer.dispatch(x, fused_fp8_quant=True, **common)
    q, s = per_token_cast_to_fp8(x)
    (rx, rsf), _, _, rh, _ = buffer.dispatch((q, s.view(torch.int16)), **common)
    torch.cuda.synchronize()
    buffer.runtime.check_status()
    assert fsf.dtype == torch.float32 and fsf.shape == (fx.size(0), hidden // 128)
    assert torch.equal(fh.recv_src_metadata, rh.recv_src_metadata)
    slots = fh.recv_src_metadata[:, :-2]
    flat = slots[slots >= 0].long()
    assert torch.equal(fx.view(torch.uint8)[flat], rx.view(torch.uint8)[flat]), 'fused e4m3 payload differs'
    assert torch.equal(fsf.view(torch.int16)[flat], rsf[flat]), 'fused scale factors differ'

    # power-of-two scales: the same comparison against the torch quantiser with `round_scale`
    (px, psf), _, _, ph, _ = buffer.dispatch(x, fused_fp8_quant='ue8m0', **common)
    q2, s2 = per_token_cast_to_fp8(x, round_scale=True)
    (rx2, rsf2), _, _, _, _ = buffer.dispatch((q2, s2.view(torch.int16)), **common)
    torch.cuda.synchronize()
    buffer.runtime.check_status()
    assert torch.equal(px.view(torch.uint8)[flat], rx2.view(torch.uint8)[flat]), 'power-of-two e4m3 payload differs'
    assert torch.equal(psf.view(torch.int16)[flat], rsf2[flat]), 'power-of-two scale factors differ'
    assert torch.equal(torch.log2(psf[flat]), torch.log2(psf[flat]).round()), 'scales are not powers of two'
