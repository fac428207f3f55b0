"""The expert-parallel MoE layer (dispatch -> grouped tcgen05 GEMMs -> combine) against a dense fp32 PyTorch
computation of the same layer, forward and backward, and the FP8 inference path against the BF16 one."""
import os

import pytest
import torch

from dist_utils import run_distributed


def _dense_reference(x, gate, w_gate_up, w_down, num_topk, bf16_gate=True):
    """fp32 MoE FFN with every expert available locally: `sum_k weight_k * FFN_{expert_k}(x)`."""
    import torch.nn.functional as F
    # on a GPU the layer multiplies the bf16 activations by the gate matrix rounded to bf16 (fp32 accumulation), on CPU
    # ranks by the fp32 matrix; the router is part of the graph, so both the gate matrix and x receive a gradient
    # through the routing weights
    scores = torch.softmax(F.linear(x.float(), gate.to(torch.bfloat16).float() if bf16_gate else gate.float()), dim=-1)
    topk_w, topk_idx = scores.topk(num_topk, dim=-1)
    topk_w = topk_w / topk_w.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(w_gate_up.size(0)):
        hit = (topk_idx == e)
        rows = hit.any(dim=1).nonzero().squeeze(1)
        if rows.numel() == 0:
            continue
        weight = (topk_w * hit)[rows].sum(dim=1, keepdim=True)
        g, u = F.linear(x[rows].float(), w_gate_up[e].float()).chunk(2, dim=-1)
        out.index_add_(0, rows, F.linear(F.silu(g) * u, w_down[e].float()) * weight)
    return out


def _moe_worker(rank, world_size, num_tokens, hidden, inter, num_experts, num_topk):
    import torch.distributed as dist
    from deep_ep.models.moe_layer import MoEConfig, MoELayer
    torch.manual_seed(5)                       # same parameters on every rank, sliced per rank below
    dev = torch.device('cuda')
    cfg = MoEConfig(hidden=hidden, intermediate=inter, num_experts=num_experts, num_topk=num_topk,
                    num_max_tokens_per_rank=num_tokens, expert_alignment=128)
    gate = torch.randn(num_experts, hidden) * 0.5
    w1 = (torch.randn(num_experts, 2 * inter, hidden) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(num_experts, hidden, inter) * 0.05).to(torch.bfloat16)
    layer = MoELayer(dist.group.WORLD, cfg).to(dev)
    local = num_experts // world_size
    with torch.no_grad():
        layer.gate.copy_(gate)
        layer.w_gate_up.copy_(w1[rank * local:(rank + 1) * local])
        layer.w_down.copy_(w2[rank * local:(rank + 1) * local])
    torch.manual_seed(100 + rank)
    x = torch.randn(num_tokens, hidden, device=dev, dtype=torch.bfloat16).requires_grad_()
    dy = torch.randn(num_tokens, hidden, device=dev, dtype=torch.bfloat16)

    y = layer(x)
    y.backward(dy)
    torch.cuda.synchronize()

    xr = x.detach().clone().requires_grad_()
    w1r, w2r = w1.to(dev).requires_grad_(), w2.to(dev).requires_grad_()
    gate_r = gate.to(dev).requires_grad_()
    ref = _dense_reference(xr, gate_r, w1r, w2r, num_topk)
    ref.backward(dy.float())
    # router: the gradient of the routing weights comes back through the combine's weight channel
    assert layer.gate.grad is not None and torch.isfinite(layer.gate.grad).all()
    gate_rel = ((layer.gate.grad - gate_r.grad).norm() / gate_r.grad.norm().clamp(min=1e-12)).item()
    assert gate_rel < 0.1, f'gate gradient deviates by {gate_rel}'
    scale = ref.abs().max().item()
    assert torch.allclose(y.float(), ref, atol=2e-2 * scale, rtol=2e-2), f'forward: {(y.float() - ref).abs().max()} of {scale}'
    gscale = xr.grad.abs().max().item()
    assert torch.allclose(x.grad.float(), xr.grad.float(), atol=3e-2 * gscale, rtol=3e-2), 'input gradient'
    # weight gradients: this rank's experts receive contributions from every rank's tokens
    g1, g2 = w1r.grad.float(), w2r.grad.float()
    dist.all_reduce(g1), dist.all_reduce(g2)
    sl = slice(rank * local, (rank + 1) * local)
    assert torch.allclose(layer.w_gate_up.grad.float(), g1[sl], atol=3e-2 * g1[sl].abs().max().item(), rtol=3e-2), 'gate/up gradient'
    assert torch.allclose(layer.w_down.grad.float(), g2[sl], atol=3e-2 * g2[sl].abs().max().item(), rtol=3e-2), 'down gradient'

    # FP8 inference path: e4m3 on the wire and in both GEMMs; compared as a whole-tensor relative difference
    y8 = layer.forward_fp8(x.detach())
    torch.cuda.synchronize()
    a, b = y8.float(), ref.detach()
    diff = 1 - 2 * (a * b).sum() / ((a * a).sum() + (b * b).sum())
    assert diff.item() < 5e-3, f'fp8 forward differs: {diff.item()}'

    # the same with power-of-two scales end to end: the dispatch kernel rounds its scales up to powers of two and the
    # expert GEMMs let the tensor core apply them (UE8M0 block scales)
    if hidden % 512 == 0 and inter % 512 == 0:
        layer.config.fp8_scales = 'ue8m0'
        layer.quantize_weights()
        y8h = layer.forward_fp8(x.detach())
        torch.cuda.synchronize()
        a = y8h.float()
        diff = 1 - 2 * (a * b).sum() / ((a * a).sum() + (b * b).sum())
        assert diff.item() < 8e-3, f'hardware-scaled fp8 forward differs: {diff.item()}'
    layer.destroy()


@pytest.mark.gpu
def test_moe_layer_single_gpu(master_port):
    run_distributed(_moe_worker, 1, master_port, 'nccl', (300, 512, 512, 8, 2))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_moe_layer_multi_gpu(master_port):
    world = min(torch.cuda.device_count(), 8)
    world -= world % 2
    run_distributed(_moe_worker, world, master_port, 'nccl', (300, 512, 512, 16, 4))


def _new_paths_worker(rank, world_size):
    """Opt-in paths against the default ones, bit for bit: the second expert GEMM delivering single-row tokens itself,
    and several warps sharing a row in decode-sized combine calls."""
    import torch.distributed as dist
    import deep_ep
    from deep_ep.models.moe_layer import MoEConfig, MoELayer
    from ep_check import check_dispatch_combine
    dev = torch.device('cuda')
    torch.manual_seed(21)
    cfg = MoEConfig(hidden=512, intermediate=256, num_experts=8 * world_size, num_topk=4, num_max_tokens_per_rank=200,
                    expert_alignment=128)
    layer = MoELayer(dist.group.WORLD, cfg, device=dev)
    torch.manual_seed(300 + rank)
    x = torch.randn(200, 512, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        plain = layer(x)
        layer.config.fuse_combine = True
        fused = layer(x)
        fused_again = layer(x)
    torch.cuda.synchronize()
    layer.buffer.runtime.check_status()
    assert torch.equal(plain, fused) and torch.equal(plain, fused_again), 'fused combine route changes the result'
    # forward + backward: the data-gradient GEMM of the first layer delivers single-row tokens of the backward combine
    grads = []
    for fuse in (False, True):
        layer.config.fuse_combine = fuse
        xg = x.clone().requires_grad_()
        layer(xg).backward(torch.ones_like(x))
        grads.append(xg.grad.clone())
    torch.cuda.synchronize()
    layer.buffer.runtime.check_status()
    assert torch.equal(grads[0], grads[1]), 'fused combine route changes the input gradient'
    layer.destroy()

    # shared expert on a side stream: same numbers, forward and backward
    cfg_s = MoEConfig(hidden=512, intermediate=256, num_experts=8 * world_size, num_topk=4, num_shared_experts=1,
                      num_max_tokens_per_rank=200, expert_alignment=128)
    layer_s = MoELayer(dist.group.WORLD, cfg_s, device=dev)
    results = []
    for overlap in (False, True):
        layer_s.config.overlap_shared_expert = overlap
        xs = x.clone().requires_grad_()
        ys = layer_s(xs)
        ys.backward(torch.ones_like(ys))
        torch.cuda.synchronize()
        results.append((ys.detach().clone(), xs.grad.clone()))
    # same output bit for bit; the input gradient is a sum of three contributions (dispatch, router, shared expert) whose
    # order of accumulation depends on the streams, so it may differ in the last bf16 digit
    assert torch.equal(results[0][0], results[1][0])
    ga, gb = results[0][1].float(), results[1][1].float()
    assert torch.allclose(ga, gb, atol=2e-2 * ga.abs().max().item(), rtol=2e-2)
    layer_s.destroy()

    # the same through the FP8 inference path with power-of-two scales (GEMM2 = the hardware-scaled kernel)
    cfg8 = MoEConfig(hidden=512, intermediate=512, num_experts=8 * world_size, num_topk=4, num_max_tokens_per_rank=200,
                     expert_alignment=128, fp8_scales='ue8m0')
    layer8 = MoELayer(dist.group.WORLD, cfg8, device=dev)
    plain8 = layer8.forward_fp8(x)
    layer8.config.fuse_combine = True
    fused8 = layer8.forward_fp8(x)
    torch.cuda.synchronize()
    layer8.buffer.runtime.check_status()
    assert torch.equal(plain8, fused8), 'fused combine route changes the FP8 result'

    # FP8 training of the routed experts against the bf16 layer: output, input gradient and weight gradients
    results8 = []
    for fp8 in (False, True):
        layer8.config.fuse_combine, layer8.config.fp8_training = False, fp8
        for p in layer8.parameters():
            p.grad = None
        xt = x.clone().requires_grad_()
        yt = layer8(xt)
        yt.backward(torch.ones_like(yt))
        torch.cuda.synchronize()
        results8.append((yt.detach().float(), xt.grad.float(), layer8.w_gate_up.grad.float(), layer8.w_down.grad.float()))
    for name, a, b in zip(('y', 'dx', 'dw_gate_up', 'dw_down'), results8[1], results8[0]):
        rel = ((a - b).norm() / b.norm().clamp(min=1e-12)).item()
        assert torch.isfinite(a).all() and rel < 0.12, f'FP8 training {name} deviates from bf16 by {rel}'
    layer8.config.fp8_training = False

    # the whole inference layer as ONE CUDA graph: the dispatch does not wait on the host (`host_sync=False`), outputs have
    # their worst-case size, the grouped GEMMs read the counts on the device
    layer8.config.host_sync = False
    eager = layer8.forward_fp8(x)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(2):
            layer8.forward_fp8(x)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            captured = layer8.forward_fp8(x)
    torch.cuda.synchronize()
    dist.barrier()
    graph.replay()
    torch.cuda.synchronize()
    layer8.buffer.runtime.check_status()
    assert torch.equal(eager, plain8), 'the layer without host synchronisation differs from the synchronised one'
    assert torch.equal(captured, eager), 'graph replay of the whole layer differs from the eager run'
    layer8.destroy()

    # weights applied inside the combine kernel against weights applied by the caller (one rounding less, so not bitwise)
    with torch.inference_mode():
        buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=96, hidden=512, num_topk=4, explicitly_destroy=True,
                                  num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        xb = torch.randn(96, 512, device=dev, dtype=torch.bfloat16)
        idx = torch.rand(96, 8 * world_size, device=dev).topk(4, dim=-1).indices
        w = torch.rand(96, 4, device=dev)
        recv_x, _, recv_w, handle, _ = buffer.dispatch(xb, topk_idx=idx, topk_weights=w, num_experts=8 * world_size,
                                                       expert_alignment=16, do_expand=True, do_zero_padding=True)
        inside, w_back, _ = buffer.combine(recv_x, handle, topk_weights=recv_w, apply_weights=True)
        outside, _, _ = buffer.combine((recv_x.float() * recv_w.unsqueeze(1)).to(torch.bfloat16), handle, topk_weights=recv_w)
        torch.cuda.synchronize()
        assert torch.equal(w_back, w)
        expected = xb.float() * w.sum(dim=1, keepdim=True)
        assert torch.allclose(inside.float(), expected, atol=3e-2, rtol=2e-2)
        assert torch.allclose(inside.float(), outside.float(), atol=3e-2, rtol=2e-2)
        buffer.destroy()

    deep_ep._C.set_warp_cooperation(True)
    try:
        with torch.inference_mode():
            buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=64, hidden=1024, num_topk=8, explicitly_destroy=True,
                                      num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
            check_dispatch_combine(buffer, 64, 1024, 8, 8 * world_size, do_cpu_sync=True, defer=True, masked_ratio=0.1,
                                   unbalanced_ratio=2.0, quick=True, num_sms=16)
            buffer.destroy()
    finally:
        deep_ep._C.set_warp_cooperation(False)


@pytest.mark.gpu
def test_opt_in_paths_match_default_paths(master_port):
    world = max(1, min(torch.cuda.device_count(), 8))
    if world > 1:
        world -= world % 2
    run_distributed(_new_paths_worker, world, master_port, 'nccl')
