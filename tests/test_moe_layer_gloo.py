"""The MoE layer's autograd plumbing on CPU ranks (gloo): dispatch <-> combine duality, routing weights, expert FFN with
the per-expert torch backend, against a dense fp32 computation of the same layer."""
import torch

from dist_utils import run_distributed
from test_moe_layer_gpu import _dense_reference


def _moe_cpu_worker(rank, world_size):
    import torch.distributed as dist
    from deep_ep.models.moe_layer import MoEConfig, MoELayer
    torch.manual_seed(5)
    num_tokens, hidden, inter, num_experts, num_topk = 48, 128, 64, 8, 3
    cfg = MoEConfig(hidden=hidden, intermediate=inter, num_experts=num_experts, num_topk=num_topk, num_shared_experts=1,
                    num_max_tokens_per_rank=num_tokens, expert_alignment=16, expert_backend='torch')
    gate = torch.randn(num_experts, hidden) * 0.5
    w1 = (torch.randn(num_experts, 2 * inter, hidden) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(num_experts, hidden, inter) * 0.05).to(torch.bfloat16)
    layer = MoELayer(dist.group.WORLD, cfg)
    assert layer.buffer.is_simulated
    local = num_experts // world_size
    with torch.no_grad():
        layer.gate.copy_(gate)
        layer.w_gate_up.copy_(w1[rank * local:(rank + 1) * local])
        layer.w_down.copy_(w2[rank * local:(rank + 1) * local])
        layer.shared_gate_up.zero_(), layer.shared_down.zero_()          # the dense reference has no shared expert
    torch.manual_seed(100 + rank)
    x = torch.randn(num_tokens, hidden).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(num_tokens, hidden).to(torch.bfloat16)
    y = layer(x)
    y.backward(dy)

    xr = x.detach().clone().requires_grad_()
    w1r, w2r = w1.clone().requires_grad_(), w2.clone().requires_grad_()
    gate_r = gate.clone().requires_grad_()
    ref = _dense_reference(xr, gate_r, w1r, w2r, num_topk, bf16_gate=False)
    ref.backward(dy.float())
    gate_rel = ((layer.gate.grad - gate_r.grad).norm() / gate_r.grad.norm()).item()
    assert gate_rel < 0.03, f'gate gradient (through the routing weights) deviates by {gate_rel}'
    scale = ref.abs().max().item()
    assert torch.allclose(y.float(), ref.detach(), atol=3e-2 * scale, rtol=3e-2), f'forward: {(y.float() - ref).abs().max()} of {scale}'
    gscale = xr.grad.abs().max().item()
    assert torch.allclose(x.grad.float(), xr.grad.float(), atol=4e-2 * gscale, rtol=4e-2), 'input gradient'
    g1, g2 = w1r.grad.float(), w2r.grad.float()
    dist.all_reduce(g1), dist.all_reduce(g2)
    sl = slice(rank * local, (rank + 1) * local)
    assert torch.allclose(layer.w_gate_up.grad.float(), g1[sl], atol=4e-2 * g1[sl].abs().max().item(), rtol=4e-2), 'gate/up gradient'
    assert torch.allclose(layer.w_down.grad.float(), g2[sl], atol=4e-2 * g2[sl].abs().max().item(), rtol=4e-2), 'down gradient'
    # without the host wait for the received-token counts the outputs have their worst-case size; same numbers
    layer.config.host_sync = False
    with torch.no_grad():
        assert torch.equal(layer(x.detach()), y.detach())
    layer.destroy()


def test_moe_layer_two_cpu_ranks(master_port):
    run_distributed(_moe_cpu_worker, 2, master_port, 'gloo', timeout_s=180)


def _moe_fp8_training_cpu_worker(rank, world_size):
    """`MoEConfig.fp8_training` through the layer on CPU ranks (PyTorch emulation of the FP8 kernels)."""
    import torch.distributed as dist
    from deep_ep.models.moe_layer import MoEConfig, MoELayer
    torch.manual_seed(6)
    num_tokens, hidden, inter, num_experts, num_topk = 40, 512, 512, 4, 2
    cfg = MoEConfig(hidden=hidden, intermediate=inter, num_experts=num_experts, num_topk=num_topk,
                    num_max_tokens_per_rank=num_tokens, expert_alignment=128, fp8_training=True)
    gate = torch.randn(num_experts, hidden) * 0.5
    w1 = (torch.randn(num_experts, 2 * inter, hidden) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(num_experts, hidden, inter) * 0.05).to(torch.bfloat16)
    layer = MoELayer(dist.group.WORLD, cfg)
    local = num_experts // world_size
    with torch.no_grad():
        layer.gate.copy_(gate)
        layer.w_gate_up.copy_(w1[rank * local:(rank + 1) * local])
        layer.w_down.copy_(w2[rank * local:(rank + 1) * local])
    torch.manual_seed(200 + rank)
    x = torch.randn(num_tokens, hidden).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(num_tokens, hidden).to(torch.bfloat16)
    y = layer(x)
    y.backward(dy)

    xr = x.detach().clone().requires_grad_()
    w1r, w2r = w1.clone().requires_grad_(), w2.clone().requires_grad_()
    gate_r = gate.clone().requires_grad_()
    ref = _dense_reference(xr, gate_r, w1r, w2r, num_topk, bf16_gate=False)
    ref.backward(dy.float())
    gate_rel = ((layer.gate.grad - gate_r.grad).norm() / gate_r.grad.norm()).item()
    assert gate_rel < 0.12, f'gate gradient (through the routing weights) deviates by {gate_rel}'
    g1, g2 = w1r.grad.float(), w2r.grad.float()
    dist.all_reduce(g1), dist.all_reduce(g2)
    sl = slice(rank * local, (rank + 1) * local)

    def rel(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm()).item()
    for name, got, want in (('forward', y, ref.detach()), ('input gradient', x.grad, xr.grad),
                            ('gate/up gradient', layer.w_gate_up.grad, g1[sl]), ('down gradient', layer.w_down.grad, g2[sl])):
        assert rel(got, want) < 0.12, f'{name}: {rel(got, want)}'
    # a second step reuses the quantised weights; an in-place update refreshes them
    first = layer._fp8_cache.get(layer.w_gate_up)[0]
    layer(x.detach())
    assert layer._fp8_cache.get(layer.w_gate_up)[0] is first
    with torch.no_grad():
        layer.w_gate_up.mul_(0.5)
    assert layer._fp8_cache.get(layer.w_gate_up)[0] is not first
    layer.destroy()


def test_moe_layer_fp8_training_two_cpu_ranks(master_port):
    run_distributed(_moe_fp8_training_cpu_worker, 2, master_port, 'gloo', timeout_s=180)
