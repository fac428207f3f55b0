"""FP8 training path of the expert FFN (`deep_ep.ops.fp8_training`): the composition (quantisers, transposed weight
copies, autograd wiring, weight cache) on CPU through the PyTorch emulation, and, on a GPU, the CUDA quantisers bit for
bit against that emulation and the whole FFN against it within FP8 tolerance. Also here: the autograd wiring of the
bf16 FFN node with its kernels emulated, and the routing-weight gradient both nodes share."""
import os

import pytest
import torch
import torch.nn.functional as F

from test_grouped_gemm_gpu import make_layout



def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


def _problem(counts, alignment, hidden, inter, dev):
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    x = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)
    dy = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)
    for s, c in zip(starts, counts):
        x[s:s + c] = torch.randn(c, hidden, device=dev).to(torch.bfloat16)
        dy[s:s + c] = torch.randn(c, hidden, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(len(counts), 2 * inter, hidden, device=dev) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(len(counts), hidden, inter, device=dev) * 0.05).to(torch.bfloat16)
    row_scale = torch.rand(rows, device=dev) + 0.5
    return psum, count, rows, starts, x, dy, w1, w2, row_scale


def _fp32_reference(x, dy, w1, w2, row_scale, starts, counts):
    x32, w1f, w2f = x.float().requires_grad_(), w1.float().requires_grad_(), w2.float().requires_grad_()
    out = torch.zeros(x.size(0), w2.size(1), device=x.device)
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c:
            g, u = (x32[s:s + c] @ w1f[e].t()).chunk(2, dim=-1)
            out[s:s + c] = (F.silu(g) * u * row_scale[s:s + c, None]) @ w2f[e].t()
    out.backward(dy.float())
    return out.detach(), x32.grad, w1f.grad, w2f.grad


def _run(x, dy, w1, w2, row_scale, psum, count, alignment):
    from deep_ep.ops.fp8_training import Fp8WeightCache, grouped_swiglu_ffn_fp8_training
    xr, w1r, w2r = x.clone().requires_grad_(), w1.clone().requires_grad_(), w2.clone().requires_grad_()
    cache = Fp8WeightCache()
    y = grouped_swiglu_ffn_fp8_training(xr, w1r, w2r, psum, count, alignment, cache, row_scale=row_scale)
    y.backward(dy)
    return y.detach(), xr.grad, w1r.grad, w2r.grad


def test_fp8_training_ffn_emulation_matches_fp32():
    torch.manual_seed(0)
    counts, alignment, hidden, inter = [100, 0, 37], 128, 512, 512
    psum, count, rows, starts, x, dy, w1, w2, row_scale = _problem(counts, alignment, hidden, inter, torch.device('cpu'))
    got = _run(x, dy, w1, w2, row_scale, psum, count, alignment)
    ref = _fp32_reference(x, dy, w1, w2, row_scale, starts, counts)
    for name, g, r in zip(('y', 'dx', 'dw_gate_up', 'dw_down'), got, ref):
        assert _rel(g, r) < 0.1, f'{name}: {_rel(g, r)}'
    # padding rows and the expert without rows stay zero
    y, dx, dw1, _ = got
    assert y[100:128].abs().max() == 0 and dx[100:128].abs().max() == 0 and dw1[1].abs().max() == 0


def test_fp8_weight_cache_follows_parameter_versions():
    from deep_ep.ops.fp8_training import Fp8WeightCache, block_quant
    from deep_ep.ops.grouped_gemm import ue8m0_to_float
    torch.manual_seed(1)
    w = (torch.randn(2, 256, 384) * 0.1).to(torch.bfloat16).requires_grad_()
    cache = Fp8WeightCache()
    q, sf, qt, sft = cache.get(w)
    assert cache.get(w)[0] is q                       # same version: no new quantisation
    assert q.shape == (2, 256, 384) and qt.shape == (2, 384, 256) and sf.shape == (2, 2, 3) and sft.shape == (2, 3, 2)
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).transpose(1, 2)) and torch.equal(sft, sf.transpose(1, 2))
    deq = q.float() * ue8m0_to_float(sf).repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
    assert _rel(deq, w.detach()) < 0.05
    with torch.no_grad():
        w.mul_(2.0)                                   # what an optimizer step does
    q2 = cache.get(w)[0]
    assert q2 is not q and torch.equal(q2.view(torch.uint8), block_quant(w.detach())[0].view(torch.uint8))


@pytest.mark.gpu
def test_cuda_quantisers_match_emulation():
    from deep_ep.ops import fp8_training as ft
    from deep_ep.ops.grouped_gemm import per_block_cast_to_fp8_ue8m0, per_token_cast_to_fp8_ue8m0, ue8m0_to_float
    torch.manual_seed(2)
    dev = torch.device('cuda')
    for rows, cols in [(1, 128), (77, 512), (300, 7168), (1025, 4096)]:
        x = (torch.randn(rows, cols, device=dev) * (1 + torch.arange(cols, device=dev) // 128).float()).to(torch.bfloat16)
        q, sf = ft.row_quant(x)
        ref_q, ref_sf = per_token_cast_to_fp8_ue8m0(x)
        assert torch.equal(sf, ref_sf) and torch.equal(q.view(torch.uint8), ref_q.view(torch.uint8)), (rows, cols)
    for g, n, k in [(1, 128, 128), (3, 512, 384), (2, 1024, 2048)]:
        w = (torch.randn(g, n, k, device=dev) * 0.05).to(torch.bfloat16)
        q, sf, qt, sft = ft.block_quant(w, transposed=True)
        ref_q, ref_sf = per_block_cast_to_fp8_ue8m0(w)
        assert torch.equal(sf, ref_sf) and torch.equal(q.view(torch.uint8), ref_q.view(torch.uint8)), (g, n, k)
        assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).transpose(1, 2)) and torch.equal(sft, sf.transpose(1, 2))
        q_only, sf_only = ft.block_quant(w)
        assert torch.equal(q_only.view(torch.uint8), q.view(torch.uint8)) and torch.equal(sf_only, sf)
    for rows, inter in [(5, 128), (300, 2048), (1025, 512)]:
        h = torch.randn(rows, 2 * inter, device=dev).to(torch.bfloat16)
        scale = torch.rand(rows, device=dev) + 0.5
        act, q, sf = ft.swiglu_quant(h, scale)
        g, u = h.float().chunk(2, dim=-1)
        ref = F.silu(g) * u * scale[:, None]
        assert _rel(act, ref) < 0.01
        deq = q.float() * ue8m0_to_float(sf).repeat_interleave(128, dim=1)
        assert _rel(deq, ref) < 0.05
        assert ft.swiglu_quant(h, None, keep_bf16=False)[0] is None


@pytest.mark.gpu
def test_fp8_training_ffn_on_gpu():
    torch.manual_seed(3)
    dev = torch.device('cuda')
    counts, alignment, hidden, inter = [200, 0, 129, 64, 511, 1], 128, 1024, 512
    psum, count, rows, starts, x, dy, w1, w2, row_scale = _problem(counts, alignment, hidden, inter, dev)
    got = _run(x, dy, w1, w2, row_scale, psum, count, alignment)
    torch.cuda.synchronize()
    emulated = _run(x.cpu(), dy.cpu(), w1.cpu(), w2.cpu(), row_scale.cpu(), psum.cpu(), count.cpu(), alignment)
    ref = _fp32_reference(x, dy, w1, w2, row_scale, starts, counts)
    for name, g, e, r in zip(('y', 'dx', 'dw_gate_up', 'dw_down'), got, emulated, ref):
        assert torch.isfinite(g.float()).all(), name
        assert _rel(g.cpu(), e) < 0.03, f'{name} against the emulation: {_rel(g.cpu(), e)}'
        assert _rel(g, r) < 0.1, f'{name} against fp32: {_rel(g, r)}'


def test_row_scale_grad_matches_fp32():
    """`<dact, act> / s` per row with products in bf16 and fp32 accumulation against a pure fp32 evaluation."""
    from deep_ep.ops.grouped_gemm import row_scale_grad
    torch.manual_seed(4)
    dact = torch.randn(200, 2048).to(torch.bfloat16)
    act = (torch.randn(200, 2048) * 0.3).to(torch.bfloat16)
    scale = torch.rand(200) + 0.1
    scale[::17] = 0                                         # padding rows
    got = row_scale_grad(dact, act, scale)
    ref = (dact.double() * act.double()).sum(1) / scale.double()
    live = scale != 0
    assert got.dtype == torch.float32 and bool((got[~live] == 0).all())
    err = (got[live].double() - ref[live]).abs().max() / ref[live].abs().max()
    assert err < 2e-3, err


def test_bf16_ffn_autograd_wiring_with_emulated_kernels(monkeypatch):
    """`GroupedSwiGLUFFN` (the bf16 training node) with its CUDA kernels replaced by PyTorch stand-ins: every returned
    gradient, the routing-weight gradient included, must match autograd on the plain formula."""
    from deep_ep.ops import grouped_gemm as gg
    from deep_ep.ops.fp8_training import _swiglu_backward

    def forward(x, w, psum, count, swiglu=False, num_sms=0, alignment=1, row_scale=None, keep_preactivation=False, route=None):
        y = torch.zeros(x.size(0), w.size(1), dtype=torch.float32)
        for e, (s, c) in enumerate(gg._ranges(psum, count)):
            y[s:s + c] = x[s:s + c].float() @ w[e].float().t()
        if not swiglu:
            return y.to(torch.bfloat16)
        h = y.to(torch.bfloat16)
        g, u = h.float().chunk(2, dim=-1)
        act = F.silu(g) * u * (1.0 if row_scale is None else row_scale[:, None])
        return (act.to(torch.bfloat16), h) if keep_preactivation else act.to(torch.bfloat16)

    def dgrad(dy, w, psum, count, num_sms=0, alignment=1, route=None):
        dx = torch.zeros(dy.size(0), w.size(2), dtype=torch.float32)
        for e, (s, c) in enumerate(gg._ranges(psum, count)):
            dx[s:s + c] = dy[s:s + c].float() @ w[e].float()
        return dx.to(torch.bfloat16)

    class FakeC:
        swiglu_backward = staticmethod(_swiglu_backward)

    monkeypatch.setattr(gg, 'grouped_gemm_forward', forward)
    monkeypatch.setattr(gg, 'grouped_gemm_dgrad', dgrad)
    monkeypatch.setattr(gg, '_wgrad', lambda dy, x, w, psum, count, alignment, _orig=gg._wgrad: _orig(dy, x, w, psum, count, 1))
    monkeypatch.setattr(gg, '_C', FakeC)

    torch.manual_seed(8)
    counts, alignment, hidden, inter = [50, 0, 77], 128, 128, 128
    psum, count, rows, starts, x, dy, w1, w2, row_scale = _problem(counts, alignment, hidden, inter, torch.device('cpu'))
    for s, c in zip(starts, counts):                       # padding rows carry weight 0, as the dispatch delivers them
        row_scale[s + c:(s + c + alignment - 1) // alignment * alignment] = 0
    xr, w1r, w2r, sr = x.clone().requires_grad_(), w1.clone().requires_grad_(), w2.clone().requires_grad_(), \
        row_scale.clone().requires_grad_()
    y = gg.GroupedSwiGLUFFN.apply(xr, w1r, w2r, sr, psum, count, alignment)
    y.backward(dy)

    x32, w1f, w2f, s32 = x.float().requires_grad_(), w1.float().requires_grad_(), w2.float().requires_grad_(), \
        row_scale.clone().requires_grad_()
    out = torch.zeros(rows, hidden)
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c:
            g, u = (x32[s:s + c] @ w1f[e].t()).chunk(2, dim=-1)
            out[s:s + c] = (F.silu(g) * u * s32[s:s + c, None]) @ w2f[e].t()
    out.backward(dy.float())
    for name, got, want in (('y', y, out), ('dx', xr.grad, x32.grad), ('dw_gate_up', w1r.grad, w1f.grad),
                            ('dw_down', w2r.grad, w2f.grad), ('d_row_scale', sr.grad, s32.grad)):
        assert got is not None and _rel(got, want.detach()) < 0.02, f'{name}: {_rel(got, want.detach())}'
