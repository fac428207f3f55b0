"""tcgen05 grouped GEMM kernels against plain fp32 PyTorch on the same expert layout."""
import pytest
import torch


def make_layout(counts, alignment, device):
    counts = torch.tensor(counts, dtype=torch.int32)
    aligned = (counts + alignment - 1) // alignment * alignment
    starts = torch.cumsum(aligned, 0) - aligned
    return (starts + counts).to(torch.int32).to(device), counts.to(device), int(aligned.sum()), starts.tolist()


CASES = [
    # counts per expert, alignment, K, N
    ([128, 0, 37, 256, 1, 300], 128, 256, 256),
    ([77, 130, 5, 64], 64, 512, 384),
    ([500, 12, 0, 0, 129, 128, 127, 1000], 128, 1024, 512),
]


@pytest.fixture(params=[False, True], ids=['single_cta', 'cta_pairs'])
def pairs(request):
    from deep_ep.ops import grouped_gemm as gg
    saved, gg.USE_PAIRS = gg.USE_PAIRS, request.param
    yield request.param
    gg.USE_PAIRS = saved


@pytest.mark.gpu
@pytest.mark.parametrize('counts,alignment,k,n', CASES)
def test_grouped_forward_dgrad_wgrad(counts, alignment, k, n, pairs):
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(0)
    dev = torch.device('cuda')
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    g = len(counts)
    x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
    w = (torch.randn(g, n, k, device=dev) * 0.05).to(torch.bfloat16)
    dy = torch.randn(rows, n, device=dev, dtype=torch.bfloat16)
    valid = torch.zeros(rows, dtype=torch.bool, device=dev)
    for s, c in zip(starts, counts):
        valid[s:s + c] = True
    x = x * valid.unsqueeze(1)            # zero padding rows, as a zero-padded dispatch delivers them
    dy = dy * valid.unsqueeze(1)

    y = torch.full((rows, n), float('nan'), device=dev, dtype=torch.bfloat16)
    out = gg.grouped_gemm_forward(x, w, psum, count)
    dx = gg.grouped_gemm_dgrad(dy, w, psum, count)
    dw = torch.zeros(g, n, k, device=dev, dtype=torch.float32)
    if alignment % 64 == 0:
        gg.grouped_gemm_wgrad(dy, x, dw, psum, count)
        gg.grouped_gemm_wgrad(dy, x, dw, psum, count)      # accumulates
        dw_store = torch.full((g, n, k), float('nan'), device=dev, dtype=torch.float32)
        gg.grouped_gemm_wgrad(dy, x, dw_store, psum, count, accumulate=False)
        torch.cuda.synchronize()
        assert torch.allclose(dw_store * 2, dw, atol=1e-3, rtol=1e-4)
        dw_bf16 = torch.full((g, n, k), float('nan'), device=dev, dtype=torch.bfloat16)
        gg.grouped_gemm_wgrad(dy, x, dw_bf16, psum, count, accumulate=False)
        torch.cuda.synchronize()
        assert torch.equal(dw_bf16, dw_store.to(torch.bfloat16))
    torch.cuda.synchronize()
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c == 0:
            assert dw[e].abs().max() == 0
            continue
        ref = x[s:s + c].float() @ w[e].float().t()
        assert torch.allclose(out[s:s + c].float(), ref, atol=2e-2, rtol=2e-2), f'forward expert {e}'
        ref_dx = dy[s:s + c].float() @ w[e].float()
        assert torch.allclose(dx[s:s + c].float(), ref_dx, atol=3e-2, rtol=2e-2), f'dgrad expert {e}'
        ref_dw = 2 * (dy[s:s + c].float().t() @ x[s:s + c].float())
        assert torch.allclose(dw[e], ref_dw, atol=5e-2, rtol=1e-2), f'wgrad expert {e}'


@pytest.mark.gpu
def test_grouped_swiglu_ffn_matches_torch(pairs):
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(1)
    dev = torch.device('cuda')
    counts, alignment, h, inter = [200, 0, 129, 64, 511], 128, 512, 256
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    w1 = (torch.randn(len(counts), 2 * inter, h, device=dev) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(len(counts), h, inter, device=dev) * 0.05).to(torch.bfloat16)
    with torch.no_grad():
        fused = gg.grouped_swiglu_ffn(x, w1, w2, psum, count, None, alignment, backend='grouped')
        ref = gg.grouped_swiglu_ffn(x, w1, w2, psum, count, None, alignment, backend='torch')
    # the fused epilogue keeps gate/up in fp32 while the loop rounds them to bf16: compare in the Frobenius norm
    def rel_err(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-6)).item()
    assert rel_err(fused, ref) < 2e-2

    # autograd path: gradients against the library-GEMM loop
    xs = [x.clone().requires_grad_() for _ in range(2)]
    w1s = [w1.clone().requires_grad_() for _ in range(2)]
    w2s = [w2.clone().requires_grad_() for _ in range(2)]
    outs = [gg.grouped_swiglu_ffn(xs[i], w1s[i], w2s[i], psum, count, None, alignment, backend=b)
            for i, b in enumerate(('grouped', 'torch'))]
    grad = torch.randn_like(outs[0])
    for o in outs:
        o.backward(grad)
    valid = torch.zeros(rows, dtype=torch.bool, device=dev)
    for s, c in zip(starts, counts):
        valid[s:s + c] = True
    assert rel_err(outs[0], outs[1]) < 2e-2
    assert rel_err(xs[0].grad[valid], xs[1].grad[valid]) < 3e-2
    assert rel_err(w1s[0].grad, w1s[1].grad) < 3e-2
    assert rel_err(w2s[0].grad, w2s[1].grad) < 3e-2


@pytest.mark.gpu
def test_fused_ffn_row_scale_and_zero_padding(pairs):
    """The fused FFN node: routing weights applied in the GEMM1 epilogue, padding rows exactly zero, gradients right."""
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(2)
    dev = torch.device('cuda')
    counts, alignment, h, inter = [130, 1, 0, 255], 128, 256, 128
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    valid = torch.zeros(rows, dtype=torch.bool, device=dev)
    for s, c in zip(starts, counts):
        valid[s:s + c] = True
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16) * valid.unsqueeze(1)
    scale = torch.rand(rows, device=dev) * valid
    w1 = (torch.randn(len(counts), 2 * inter, h, device=dev) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(len(counts), h, inter, device=dev) * 0.05).to(torch.bfloat16)
    params = [[t.clone().requires_grad_() for t in (x, w1, w2)] for _ in range(2)]
    outs = [gg.grouped_swiglu_ffn(p[0], p[1], p[2], psum, count, None, alignment, backend=b, row_scale=scale)
            for p, b in zip(params, ('grouped', 'torch'))]
    assert torch.count_nonzero(outs[0][~valid]).item() == 0
    grad = torch.randn_like(outs[0]) * valid.unsqueeze(1)
    for o in outs:
        o.backward(grad)

    def rel_err(a, b):
        return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-6)).item()
    assert rel_err(outs[0][valid], outs[1][valid]) < 2e-2
    for a, b in zip(params[0], params[1]):
        assert rel_err(a.grad, b.grad) < 3e-2


FP8_CASES = [
    # counts per expert, alignment, K, N
    ([128, 0, 37, 256, 1, 300], 128, 256, 256),
    ([77, 130, 5, 64], 64, 512, 512),
    ([500, 12, 0, 0, 129, 128, 127, 1000], 128, 1024, 768),
]


def _fp8_inputs(counts, alignment, k, n, dev):
    from deep_ep.ops import grouped_gemm as gg
    from deep_ep.utils.math import per_token_cast_to_fp8
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
    # uneven magnitudes per 128-column block and per weight block, so that a wrong scale index shows
    x = x * (1 + torch.arange(k, device=dev) // 128).to(torch.bfloat16)
    w = torch.randn(len(counts), n, k, device=dev) * 0.05
    w = w * (1 + (torch.arange(n, device=dev) // 128).float()).view(1, n, 1) * (1 + (torch.arange(k, device=dev) // 128).float() * 0.5)
    x_fp8, x_sf = per_token_cast_to_fp8(x)
    w_fp8, w_sf = gg.per_block_cast_to_fp8(w)
    x_deq = x_fp8.float() * x_sf.repeat_interleave(128, dim=1)
    w_deq = gg.per_block_cast_back(w_fp8, w_sf)
    return psum, count, rows, starts, x_fp8, x_sf, w_fp8, w_sf, x_deq, w_deq


@pytest.mark.gpu
@pytest.mark.parametrize('counts,alignment,k,n', FP8_CASES)
def test_grouped_fp8_forward(counts, alignment, k, n):
    """Block-scaled e4m3 GEMM against fp32 PyTorch on the de-quantised operands."""
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(2)
    dev = torch.device('cuda')
    psum, count, rows, starts, x_fp8, x_sf, w_fp8, w_sf, x_deq, w_deq = _fp8_inputs(counts, alignment, k, n, dev)
    out = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w_fp8, w_sf, psum, count, alignment=alignment)
    torch.cuda.synchronize()
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c == 0:
            continue
        ref = x_deq[s:s + c] @ w_deq[e].t()
        got = out[s:s + c].float()
        assert torch.allclose(got, ref, atol=1e-2 * ref.abs().max().item(), rtol=1e-2), f'expert {e}: {(got - ref).abs().max()}'
        pad = (c + alignment - 1) // alignment * alignment
        if pad > c:
            assert out[s + c:s + pad].abs().max().item() == 0


@pytest.mark.gpu
def test_grouped_fp8_swiglu_and_ffn():
    """SwiGLU epilogue (bf16 and re-quantised e4m3 output) and the two-GEMM FP8 FFN against fp32 PyTorch."""
    from deep_ep.ops import grouped_gemm as gg
    import torch.nn.functional as F
    torch.manual_seed(3)
    dev = torch.device('cuda')
    counts, alignment, h, inter = [200, 0, 129, 64, 511], 128, 512, 256
    psum, count, rows, starts, x_fp8, x_sf, w1_fp8, w1_sf, x_deq, w1_deq = _fp8_inputs(counts, alignment, h, 2 * inter, dev)
    w2 = torch.randn(len(counts), h, inter, device=dev) * 0.05
    w2_fp8, w2_sf = gg.per_block_cast_to_fp8(w2)
    w2_deq = gg.per_block_cast_back(w2_fp8, w2_sf)
    row_scale = torch.rand(rows, device=dev) + 0.5

    act = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w1_fp8, w1_sf, psum, count, swiglu=True, alignment=alignment, row_scale=row_scale)
    act_q, act_sf = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w1_fp8, w1_sf, psum, count, swiglu=True, quantize_output=True,
                                                alignment=alignment, row_scale=row_scale)
    y = gg.grouped_swiglu_ffn_fp8(x_fp8, x_sf, w1_fp8, w1_sf, w2_fp8, w2_sf, psum, count, alignment=alignment, row_scale=row_scale)
    torch.cuda.synchronize()
    act_deq = act_q.float() * act_sf.repeat_interleave(128, dim=1)
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c == 0:
            continue
        g, u = (x_deq[s:s + c] @ w1_deq[e].t()).chunk(2, dim=-1)
        ref_act = F.silu(g) * u * row_scale[s:s + c].unsqueeze(1)
        scale = ref_act.abs().max().item()
        assert torch.allclose(act[s:s + c].float(), ref_act, atol=1e-2 * scale, rtol=1e-2), f'swiglu expert {e}'
        # e4m3 has 3 mantissa bits: relative error up to 2^-4 of each row block's maximum
        err = (act_deq[s:s + c] - ref_act).abs().max().item()
        assert err <= 0.07 * scale, f'quantised swiglu expert {e}: {err} vs {scale}'
        # the FFN result against the same math on what the second GEMM actually consumed
        ref_y = act_deq[s:s + c] @ w2_deq[e].t()
        assert torch.allclose(y[s:s + c].float(), ref_y, atol=1e-2 * ref_y.abs().max().item(), rtol=1e-2), f'ffn expert {e}'
        pad = (c + alignment - 1) // alignment * alignment
        if pad > c:
            assert y[s + c:s + pad].abs().max().item() == 0 and act[s + c:s + pad].abs().max().item() == 0


UE8M0_CASES = [
    # counts per expert, alignment, K (multiple of 512), N
    ([128, 0, 37, 256, 1, 300], 128, 512, 256),
    ([77, 130, 5, 64], 64, 1024, 512),
    ([500, 12, 0, 0, 129, 128, 127, 1000], 128, 2048, 768),
]


def _ue8m0_inputs(counts, alignment, k, n, dev):
    from deep_ep.ops import grouped_gemm as gg
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    x = torch.randn(rows, k, device=dev) * (1 + torch.arange(k, device=dev) // 128).float() * 3.0
    w = torch.randn(len(counts), n, k, device=dev) * 0.05
    w = w * (1 + (torch.arange(n, device=dev) // 128).float() * 7).view(1, n, 1) * (1 + (torch.arange(k, device=dev) // 128).float() * 0.5)
    x_fp8, x_sf = gg.per_token_cast_to_fp8_ue8m0(x)
    w_fp8, w_sf = gg.per_block_cast_to_fp8_ue8m0(w)
    x_deq = x_fp8.float() * gg.ue8m0_to_float(x_sf).repeat_interleave(128, dim=1)
    w_deq = w_fp8.float() * gg.ue8m0_to_float(w_sf).repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
    return psum, count, rows, starts, x_fp8, x_sf, w_fp8, w_sf, x_deq, w_deq


@pytest.mark.gpu
@pytest.mark.parametrize('counts,alignment,k,n', UE8M0_CASES)
def test_grouped_fp8_hardware_scaled_forward(counts, alignment, k, n):
    """`kind::mxf8f6f4.block_scale` GEMM with UE8M0 scales against fp32 PyTorch on the de-quantised operands."""
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(4)
    dev = torch.device('cuda')
    psum, count, rows, starts, x_fp8, x_sf, w_fp8, w_sf, x_deq, w_deq = _ue8m0_inputs(counts, alignment, k, n, dev)
    out = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w_fp8, w_sf, psum, count, alignment=alignment)
    torch.cuda.synchronize()
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c == 0:
            continue
        ref = x_deq[s:s + c] @ w_deq[e].t()
        got = out[s:s + c].float()
        assert torch.allclose(got, ref, atol=1e-2 * ref.abs().max().item(), rtol=1e-2), f'expert {e}: {(got - ref).abs().max()}'
        pad = (c + alignment - 1) // alignment * alignment
        if pad > c:
            assert out[s + c:s + pad].abs().max().item() == 0


@pytest.mark.gpu
def test_grouped_fp8_hardware_scaled_swiglu_chain():
    """SwiGLU epilogue with e4m3 + UE8M0 output feeding the second hardware-scaled GEMM."""
    from deep_ep.ops import grouped_gemm as gg
    import torch.nn.functional as F
    torch.manual_seed(6)
    dev = torch.device('cuda')
    counts, alignment, h, inter = [200, 0, 129, 64, 511], 128, 512, 512
    psum, count, rows, starts, x_fp8, x_sf, w1_fp8, w1_sf, x_deq, w1_deq = _ue8m0_inputs(counts, alignment, h, 2 * inter, dev)
    w2 = torch.randn(len(counts), h, inter, device=dev) * 0.05
    w2_fp8, w2_sf = gg.per_block_cast_to_fp8_ue8m0(w2)
    w2_deq = w2_fp8.float() * gg.ue8m0_to_float(w2_sf).repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
    row_scale = torch.rand(rows, device=dev) + 0.5
    act = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w1_fp8, w1_sf, psum, count, swiglu=True, alignment=alignment, row_scale=row_scale)
    act_q, act_sf = gg.grouped_gemm_fp8_forward(x_fp8, x_sf, w1_fp8, w1_sf, psum, count, swiglu=True, quantize_output=True,
                                                alignment=alignment, row_scale=row_scale)
    assert act_sf.dtype == torch.uint8
    y = gg.grouped_gemm_fp8_forward(act_q, act_sf, w2_fp8, w2_sf, psum, count, alignment=alignment)
    torch.cuda.synchronize()
    act_deq = act_q.float() * gg.ue8m0_to_float(act_sf).repeat_interleave(128, dim=1)
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c == 0:
            continue
        g, u = (x_deq[s:s + c] @ w1_deq[e].t()).chunk(2, dim=-1)
        ref_act = F.silu(g) * u * row_scale[s:s + c].unsqueeze(1)
        scale = ref_act.abs().max().item()
        assert torch.allclose(act[s:s + c].float(), ref_act, atol=1e-2 * scale, rtol=1e-2), f'swiglu expert {e}'
        err = (act_deq[s:s + c] - ref_act).abs().max().item()
        assert err <= 0.07 * scale, f'quantised swiglu expert {e}: {err} vs {scale}'
        ref_y = act_deq[s:s + c] @ w2_deq[e].t()
        assert torch.allclose(y[s:s + c].float(), ref_y, atol=1e-2 * ref_y.abs().max().item(), rtol=1e-2), f'ffn expert {e}'


@pytest.mark.gpu
@pytest.mark.parametrize('rows', [64, 300, 1024])
def test_dense_linear_and_dense_ffn_match_torch(rows):
    """The one-group kernels behind the router and the shared expert: fp32 logits, data and weight gradients of
    `dense_linear`, and the fused dense SwiGLU FFN, against fp32 PyTorch."""
    from deep_ep.ops.dense import dense_linear, dense_swiglu_ffn
    torch.manual_seed(rows)
    dev = torch.device('cuda')
    k, n = 512, 256
    x = (torch.randn(rows, k, device=dev) * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(n, k, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
    y = dense_linear(x, w, out_fp32=True)
    assert y.dtype == torch.float32 and y.shape == (rows, n)
    ref = x.detach().float() @ w.detach().float().t()
    assert torch.allclose(y, ref, atol=1e-3 * ref.abs().max().item(), rtol=1e-3)        # fp32 accumulator, not rounded to bf16
    dy = torch.randn(rows, n, device=dev)
    y.backward(dy)
    dyb = dy.to(torch.bfloat16).float()
    ref_dx, ref_dw = dyb @ w.detach().float(), dyb.t() @ x.detach().float()
    assert torch.allclose(x.grad.float(), ref_dx, atol=2e-2 * ref_dx.abs().max().item(), rtol=2e-2)
    assert torch.allclose(w.grad.float(), ref_dw, atol=2e-2 * ref_dw.abs().max().item(), rtol=2e-2)
    # dense SwiGLU FFN (rows that are no multiple of 128 are padded inside)
    inter = 256
    w1 = (torch.randn(2 * inter, k, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(k, inter, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
    x2 = x.detach().clone().requires_grad_()
    out = dense_swiglu_ffn(x2, w1, w2)
    g, u = (x2.detach().float() @ w1.detach().float().t()).chunk(2, dim=-1)
    ref_out = (torch.nn.functional.silu(g) * u) @ w2.detach().float().t()
    assert out.shape == (rows, k)
    assert torch.allclose(out.float(), ref_out, atol=3e-2 * ref_out.abs().max().item(), rtol=3e-2)
    out.backward(torch.ones_like(out))
    assert torch.isfinite(x2.grad.float()).all() and torch.isfinite(w1.grad.float()).all() and torch.isfinite(w2.grad.float()).all()


@pytest.mark.gpu
def test_unfused_ffn_with_alignment_64_survives_poisoned_padding():
    """Expert alignment 64 takes the un-fused autograd path (two `GroupedLinear` nodes). Its intermediate tensors come from
    `torch.empty`; the tensor-core weight gradient reads whole 64-row blocks, padding included, so the padding rows of every
    intermediate must have been written as zeros. The allocator is seeded with NaN blocks first, so that a row that was
    left unwritten shows up as a NaN in a weight gradient."""
    from deep_ep.ops import grouped_gemm as gg
    torch.manual_seed(3)
    dev = torch.device('cuda')
    counts, alignment, hidden, inter = [70, 1, 0, 130, 64], 64, 256, 128
    psum, count, rows, starts = make_layout(counts, alignment, dev)
    g = len(counts)
    x = torch.zeros(rows, hidden, device=dev, dtype=torch.bfloat16)
    for s, c in zip(starts, counts):
        x[s:s + c] = torch.randn(c, hidden, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(g, 2 * inter, hidden, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(g, hidden, inter, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    # blocks of the sizes the layer is about to ask for, filled with NaN and handed back to the caching allocator
    for cols in (2 * inter, inter, hidden, 2 * inter, inter, hidden):
        poison = torch.full((rows, cols), float('nan'), device=dev, dtype=torch.bfloat16)
        del poison
    xg = x.clone().requires_grad_()
    y = gg.grouped_swiglu_ffn(xg, w1, w2, psum, count, None, alignment)
    dy = torch.zeros_like(y)
    for s, c in zip(starts, counts):
        dy[s:s + c] = torch.randn(c, hidden, device=dev).to(torch.bfloat16)
    y.backward(dy)
    torch.cuda.synchronize()
    for name, t in (('y', y), ('dx', xg.grad), ('dw_gate_up', w1.grad), ('dw_down', w2.grad)):
        assert torch.isfinite(t.float()).all(), f'{name} holds a value that came from an unwritten padding row'
    # against the per-expert fp32 computation
    w1r, w2r = w1.detach().float().requires_grad_(), w2.detach().float().requires_grad_()
    xr = x.float().requires_grad_()
    ref = torch.zeros(rows, hidden, device=dev)
    for e, (s, c) in enumerate(zip(starts, counts)):
        if c:
            gate, up = (xr[s:s + c] @ w1r[e].t()).chunk(2, dim=-1)
            ref[s:s + c] = (torch.nn.functional.silu(gate) * up) @ w2r[e].t()
    ref.backward(dy.float())
    for name, got, want in (('y', y, ref), ('dx', xg.grad, xr.grad), ('dw_gate_up', w1.grad, w1r.grad), ('dw_down', w2.grad, w2r.grad)):
        scale = want.abs().max().item()
        assert torch.allclose(got.float(), want.detach(), atol=4e-2 * scale, rtol=4e-2), name
