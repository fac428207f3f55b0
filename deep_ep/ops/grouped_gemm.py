"""Grouped GEMMs of the expert FFNs over the expanded dispatch layout, on tcgen05 tensor cores.

Expert e owns rows `[psum[e] - count[e], psum[e])` of the expanded activations (`psum` and `count` are the
handle's `psum_num_recv_tokens_per_expert` and `num_unaligned_recv_tokens_per_expert`, on the device: no host
synchronisation is needed to launch). Three kernels modes cover a linear layer's forward, data gradient and
weight gradient; `GroupedLinear` ties them into autograd and `grouped_swiglu_ffn` builds the SwiGLU FFN.
Backend `'torch'` is the library-GEMM loop used as the comparison baseline and as the oracle in tests.
"""
import os
from typing import List, Optional

import torch
import torch.nn.functional as F

from .._C_loader import _C

MODE_FORWARD, MODE_DGRAD, MODE_WGRAD = 0, 1, 2

# Which kernel runs a GEMM: CTA pairs (`tcgen05.mma.cta_group::2`, 256 x 256 tiles) or one CTA per 128 x 256 tile.
# Measured on B200: the single-CTA kernel is ahead for the forward GEMMs (K-major weights, one TMA box per operand),
# the pair kernel for data and weight gradients (MN-major operands, where a pair halves the TMA boxes per CTA).
# EP_GEMM_PAIRS=1 / 0 forces one of them everywhere; the default 'auto' picks per mode.
USE_PAIRS = {'0': False, '1': True}.get(os.environ.get('EP_GEMM_PAIRS', 'auto'), None)


def _pairs(mode: int) -> bool:
    return (mode != MODE_FORWARD) if USE_PAIRS is None else USE_PAIRS

EPILOGUE_STORE, EPILOGUE_SWIGLU, EPILOGUE_SWIGLU_KEEP = 0, 1, 2


def grouped_gemm_forward(x: torch.Tensor, w: torch.Tensor, psum: torch.Tensor, count: torch.Tensor,
                         swiglu: bool = False, num_sms: int = 0, alignment: int = 1,
                         row_scale: Optional[torch.Tensor] = None, keep_preactivation: bool = False,
                         route: Optional[torch.Tensor] = None):
    """`y[rows_e] = x[rows_e] @ w[e].T` with `w [G, N, K]`; with `swiglu`, `w[e] = [gate; up]` and
    `y = silu(x @ gate.T) * (x @ up.T) * row_scale` (`[rows, N / 2]`); `keep_preactivation` also returns the bf16
    `[gate | up]` matrix. Padding rows inside an expert's aligned region are written as zeros; rows that belong to no
    region are left untouched. `route` (plain store only, from `EPBuffer.build_combine_route`): rows with an entry are
    stored at that address (the combine landing slot of their token's owner) instead of the returned tensor."""
    n_out = w.size(1) // 2 if swiglu else w.size(1)
    y = torch.empty((x.size(0), n_out), dtype=torch.bfloat16, device=x.device)
    if not swiglu:
        assert row_scale is None and not keep_preactivation
        _C.grouped_gemm(x, w, y, psum, count, MODE_FORWARD, EPILOGUE_STORE, num_sms, alignment, None, None, _pairs(MODE_FORWARD),
                        route)
        return y
    assert route is None
    keep = torch.empty((x.size(0), w.size(1)), dtype=torch.bfloat16, device=x.device) if keep_preactivation else None
    _C.grouped_gemm(x, w, y, psum, count, MODE_FORWARD, EPILOGUE_SWIGLU_KEEP if keep_preactivation else EPILOGUE_SWIGLU,
                    num_sms, alignment, row_scale, keep, _pairs(MODE_FORWARD))
    return (y, keep) if keep_preactivation else y


def grouped_gemm_dgrad(dy: torch.Tensor, w: torch.Tensor, psum: torch.Tensor, count: torch.Tensor,
                       num_sms: int = 0, alignment: int = 1, route: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`dx[rows_e] = dy[rows_e] @ w[e]` with `w [G, N, K]` read as stored (no transpose copy); `route` as in
    `grouped_gemm_forward`."""
    dx = torch.empty((dy.size(0), w.size(2)), dtype=torch.bfloat16, device=dy.device)
    _C.grouped_gemm(dy, w, dx, psum, count, MODE_DGRAD, EPILOGUE_STORE, num_sms, alignment, None, None, _pairs(MODE_DGRAD), route)
    return dx


def _wgrad(dy, x, w, psum, count, alignment):
    """Weight gradient of one grouped linear layer, honouring a persistent fp32 `main_grad` buffer on the parameter."""
    main_grad = getattr(w, 'main_grad', None)
    if alignment % 64 == 0:
        # fp32 accumulation happens in tensor memory; without a persistent fp32 buffer the result is rounded once and
        # stored in the parameter's dtype, which avoids materialising an fp32 copy of every expert
        acc = main_grad if main_grad is not None else torch.empty(w.shape, dtype=w.dtype, device=w.device)
        grouped_gemm_wgrad(dy, x, acc, psum, count, accumulate=main_grad is not None)
    else:
        acc = main_grad if main_grad is not None else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        for e, (start, c) in enumerate(_ranges(psum, count)):
            if c:
                acc[e].addmm_(dy[start:start + c].float().t(), x[start:start + c].float())
    return None if main_grad is not None else (acc if acc.dtype == w.dtype else acc.to(w.dtype))


def row_scale_grad(dact: torch.Tensor, act: torch.Tensor, row_scale: torch.Tensor) -> torch.Tensor:
    """Gradient of the per-row scale `s` of `act = s * silu(gate) * up` given `dact = dL/dact`: `<dact, act> / s` per row
    (rows with `s == 0`, i.e. padding, get 0). This is what carries the loss back to the routing weights."""
    # products in the tensors' own precision (one rounding each, errors average out over the row), fp32 accumulation:
    # two passes over [rows, I] instead of the four that an fp32 copy of both operands would cost
    dot = torch.sum(dact * act, dim=1, dtype=torch.float32)
    return torch.where(row_scale != 0, dot / row_scale, torch.zeros_like(dot))


class GroupedSwiGLUFFN(torch.autograd.Function):
    """Whole expert FFN as one autograd node: `y = (silu(x Wg^T) * (x Wu^T) * row_scale) Wd^T` per expert.

    Forward: GEMM1 with the SwiGLU (and row-scale) epilogue that also keeps the pre-activation, then GEMM2.
    Backward: dgrad and wgrad of GEMM2, one elementwise SwiGLU-backward kernel, dgrad and wgrad of GEMM1.
    Requires the expert alignment to be a multiple of 128 (every padding row is then written as zero by a tile)."""

    @staticmethod
    def forward(ctx, x, w_gate_up, w_down, row_scale, psum, count, alignment, route=None, backward_route=None):
        act, h = grouped_gemm_forward(x, w_gate_up, psum, count, swiglu=True, alignment=alignment, row_scale=row_scale,
                                      keep_preactivation=True)
        # with `route`, rows that are their token's only one leave this GEMM for the owner's combine landing slot
        y = grouped_gemm_forward(act, w_down, psum, count, alignment=alignment, route=route)
        ctx.save_for_backward(x, w_gate_up, w_down, row_scale, psum, count, h, act)
        ctx.alignment = alignment
        # `backward_route = (table, barrier)`: the data-gradient GEMM of the first layer feeds the combine that is the
        # backward of dispatch, so it can deliver single-row tokens the same way; `barrier()` is called right before it
        ctx.backward_route = backward_route
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_gate_up, w_down, row_scale, psum, count, h, act = ctx.saved_tensors
        dy = dy.contiguous()
        dact = grouped_gemm_dgrad(dy, w_down, psum, count, alignment=ctx.alignment)
        dw_down = _wgrad(dy, act, w_down, psum, count, ctx.alignment) if ctx.needs_input_grad[2] else None
        d_row_scale = row_scale_grad(dact, act, row_scale) if row_scale is not None and ctx.needs_input_grad[3] else None
        dh = _C.swiglu_backward(h, dact, row_scale)
        dx = None
        if ctx.needs_input_grad[0]:
            table = None
            if ctx.backward_route is not None:
                table, barrier = ctx.backward_route
                barrier()
            dx = grouped_gemm_dgrad(dh, w_gate_up, psum, count, alignment=ctx.alignment, route=table)
        dw_gate_up = _wgrad(dh, x, w_gate_up, psum, count, ctx.alignment) if ctx.needs_input_grad[1] else None
        return dx, dw_gate_up, dw_down, d_row_scale, None, None, None, None, None


def grouped_gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, dw: torch.Tensor, psum: torch.Tensor, count: torch.Tensor,
                       num_sms: int = 0, accumulate: bool = True) -> torch.Tensor:
    """`dw[e] += dy[rows_e].T @ x[rows_e]` in fp32 (`dw [G, N, K]` fp32); with `accumulate=False` the result
    overwrites `dw` (experts without rows get zeros), which saves reading it. Padding rows of `dy` or `x` up to the
    next multiple of 64 rows must be zero."""
    _C.grouped_gemm_wgrad(dy, x, dw, psum, count, num_sms, accumulate, _pairs(MODE_WGRAD))
    return dw


def _zero_padding_rows(t: torch.Tensor, psum: torch.Tensor, count: torch.Tensor, alignment: int) -> torch.Tensor:
    """`t` with the alignment padding rows forced to zero when the tensor-core weight gradient is going to read them
    (an upstream gradient may hold anything there, and NaN x 0 is NaN)."""
    return mask_padding_rows(t, psum, count) if alignment % 64 == 0 else t


def _ranges(psum: torch.Tensor, count: torch.Tensor):
    return [(e - c, c) for e, c in zip(psum.tolist(), count.tolist())]


def _supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.size(1) % 128 == 0 and \
        w.size(2) % 128 == 0


class GroupedLinear(torch.autograd.Function):
    """`y = x @ w[e].T` per expert. Weight gradients are accumulated in fp32: into `w.main_grad` when the parameter
    carries such a buffer, otherwise into a fresh fp32 tensor that is cast to the parameter dtype."""

    @staticmethod
    def forward(ctx, x, w, psum, count, alignment):
        ctx.save_for_backward(x, w, psum, count)
        ctx.alignment = alignment
        # the alignment reaches the kernels so that the padding rows of every expert's region are written as zeros: the
        # tensor-core weight-gradient GEMM reads whole 64-row blocks, padding included
        return grouped_gemm_forward(x, w, psum, count, alignment=alignment)

    @staticmethod
    def backward(ctx, dy):
        x, w, psum, count = ctx.saved_tensors
        dy = dy.contiguous()
        dx = grouped_gemm_dgrad(dy, w, psum, count, alignment=ctx.alignment) if ctx.needs_input_grad[0] else None
        dw = _wgrad(_zero_padding_rows(dy, psum, count, ctx.alignment), x, w, psum, count, ctx.alignment) \
            if ctx.needs_input_grad[1] else None
        return dx, dw, None, None, None


# ---------------------------------------------------------------------------------------------- FP8 forward path
# EP_FP8_REG_SPLIT=0 selects the 320-thread kernel without the `setmaxnreg` register split (kept for comparison).
FP8_REG_SPLIT = os.environ.get('EP_FP8_REG_SPLIT', '1') != '0'

def per_block_cast_to_fp8(w: torch.Tensor):
    """Quantise weights `[..., n, k]` to e4m3 with one fp32 scale per 128 x 128 block (`n`, `k` multiples of 128).
    Returns `(w_fp8 [..., n, k], scales [..., n / 128, k / 128])`; `w ~= w_fp8 * scales` expanded over the blocks."""
    *lead, n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    if lead and w.numel() > (1 << 28):
        # one leading slice at a time: the fp32 temporaries of a whole expert stack would be several times its size
        parts = [per_block_cast_to_fp8(w[i]) for i in range(w.size(0))]
        return torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts])
    blocks = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
    amax = blocks.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-4)
    q = (blocks * (448.0 / amax)).to(torch.float8_e4m3fn).reshape(*lead, n, k)
    return q.contiguous(), (amax / 448.0).reshape(*lead, n // 128, k // 128).contiguous()


def per_block_cast_back(w_fp8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """fp32 `[..., n, k]` from `per_block_cast_to_fp8` output."""
    return w_fp8.float() * scales.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)


def _ue8m0_ceil(amax_over_448: torch.Tensor):
    """Smallest power of two >= each (positive) entry, as `(uint8 UE8M0 bytes, fp32 values)`: value = 2^(byte - 127)."""
    bits = amax_over_448.float().contiguous().view(torch.int32)
    byte = ((bits >> 23) & 0xff) + ((bits & 0x7fffff) != 0).int()
    byte = byte.clamp(1, 253)
    return byte.to(torch.uint8), (byte << 23).view(torch.float32)


def per_token_cast_to_fp8_ue8m0(x: torch.Tensor):
    """`[m, n]` -> `(e4m3 [m, n], uint8 [m, n / 128])` with power-of-two scales `2^ceil(log2(amax / 448))` stored as UE8M0
    bytes: the format the hardware-scaled FP8 GEMM reads. Same quantiser as
    `deep_ep.utils.math.per_token_cast_to_fp8(x, round_scale=True)` (and as the dispatch kernel's `'ue8m0'` mode), with
    the scales reduced to their exponent byte."""
    from ..utils.math import per_token_cast_to_fp8
    assert x.size(1) % 128 == 0
    q, scale = per_token_cast_to_fp8(x, round_scale=True)
    return q, ((scale.contiguous().view(torch.int32) >> 23) & 0xff).to(torch.uint8).contiguous()


def per_block_cast_to_fp8_ue8m0(w: torch.Tensor):
    """Weights `[..., n, k]` -> `(e4m3, uint8 [..., n / 128, k / 128])` with one power-of-two scale per 128 x 128 block."""
    *lead, n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    if lead and w.numel() > (1 << 28):
        parts = [per_block_cast_to_fp8_ue8m0(w[i]) for i in range(w.size(0))]
        return torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts])
    blocks = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
    byte, scale = _ue8m0_ceil(blocks.abs().amax(dim=(-3, -1), keepdim=True).clamp(min=1e-4) * (1.0 / 448.0))
    q = (blocks / scale).to(torch.float8_e4m3fn).reshape(*lead, n, k)
    return q.contiguous(), byte.reshape(*lead, n // 128, k // 128).contiguous()


def ue8m0_to_float(sf: torch.Tensor) -> torch.Tensor:
    """fp32 value `2^(byte - 127)` of UE8M0 scale bytes."""
    return (sf.to(torch.int32) << 23).view(torch.float32)


def grouped_gemm_fp8_forward(x_fp8: torch.Tensor, x_sf: torch.Tensor, w_fp8: torch.Tensor, w_sf: torch.Tensor,
                             psum: torch.Tensor, count: torch.Tensor, swiglu: bool = False, quantize_output: bool = False,
                             num_sms: int = 0, alignment: int = 1, row_scale: Optional[torch.Tensor] = None,
                             route: Optional[torch.Tensor] = None):
    """`y[rows_e] = (x_fp8 * x_sf)[rows_e] @ (w_fp8[e] * w_sf[e]).T` on the FP8 tensor cores.

    `x_fp8 [rows, K]` e4m3 with `x_sf [rows, K / 128]` fp32 (what an FP8 dispatch returns), `w_fp8 [G, N, K]` e4m3 with
    `w_sf [G, N / 128, K / 128]`. Result: bf16 `[rows, N]`; with `swiglu` (`w[e] = [gate; up]`) bf16 `[rows, N / 2]`, or
    with `quantize_output` the pair `(e4m3 [rows, N / 2], scales [rows, N / 256])` ready to feed the next FP8 GEMM.
    Padding rows inside an expert's aligned region are written as zeros.

    Scales are either fp32 (applied in registers after every K block of 128) or uint8 UE8M0 bytes (powers of two,
    `per_token_cast_to_fp8_ue8m0` / `per_block_cast_to_fp8_ue8m0`), which the tensor core applies itself; the latter
    needs K to be a multiple of 512."""
    rows, n = x_fp8.size(0), w_fp8.size(1)
    if not swiglu:
        assert not quantize_output and row_scale is None
        y = torch.empty((rows, n), dtype=torch.bfloat16, device=x_fp8.device)
        _C.grouped_gemm_fp8(x_fp8, x_sf, w_fp8, w_sf, y, psum, count, EPILOGUE_STORE, num_sms, alignment, None, None, FP8_REG_SPLIT,
                            route)
        return y
    assert route is None
    if quantize_output:
        y = torch.empty((rows, n // 2), dtype=torch.float8_e4m3fn, device=x_fp8.device)
        y_sf = torch.empty((rows, n // 256), dtype=w_sf.dtype, device=x_fp8.device)
        _C.grouped_gemm_fp8(x_fp8, x_sf, w_fp8, w_sf, y, psum, count, EPILOGUE_SWIGLU, num_sms, alignment, row_scale, y_sf, FP8_REG_SPLIT)
        return y, y_sf
    y = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=x_fp8.device)
    _C.grouped_gemm_fp8(x_fp8, x_sf, w_fp8, w_sf, y, psum, count, EPILOGUE_SWIGLU, num_sms, alignment, row_scale, None, FP8_REG_SPLIT)
    return y


def grouped_swiglu_ffn_fp8(x_fp8: torch.Tensor, x_sf: torch.Tensor, w_gate_up: torch.Tensor, w_gate_up_sf: torch.Tensor,
                           w_down: torch.Tensor, w_down_sf: torch.Tensor, psum: torch.Tensor, count: torch.Tensor,
                           alignment: int = 128, row_scale: Optional[torch.Tensor] = None,
                           route: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Forward-only FP8 expert FFN over dispatched FP8 rows: GEMM1 with the SwiGLU epilogue re-quantises its output per
    row and 128 columns, GEMM2 consumes that directly; the result is bf16 `[rows, H]`. No elementwise pass touches
    global memory between the dispatch and the combine."""
    act, act_sf = grouped_gemm_fp8_forward(x_fp8, x_sf, w_gate_up, w_gate_up_sf, psum, count, swiglu=True,
                                           quantize_output=True, alignment=alignment, row_scale=row_scale)
    # `route` (power-of-two scales only): single-row tokens leave GEMM2 for their owners' combine landing slots
    return grouped_gemm_fp8_forward(act, act_sf, w_down, w_down_sf, psum, count, alignment=alignment, route=route)


def _torch_ffn(x, w_gate_up, w_down, psum, count):
    pieces, cursor = [], 0
    w1s, w2s = w_gate_up.unbind(0), w_down.unbind(0)
    for e, (start, c) in enumerate(_ranges(psum, count)):
        if c == 0:
            continue
        if start > cursor:
            pieces.append(x.new_zeros((start - cursor, w_down.size(1))))
        g, u = F.linear(x[start:start + c], w1s[e]).chunk(2, dim=-1)
        pieces.append(F.linear(F.silu(g) * u, w2s[e]))
        cursor = start + c
    if cursor < x.size(0):
        pieces.append(x.new_zeros((x.size(0) - cursor, w_down.size(1))))
    return torch.cat(pieces)


def grouped_swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, psum: torch.Tensor,
                       unaligned: torch.Tensor, per_expert_list: Optional[List[int]], alignment: int,
                       backend: str = 'grouped', row_scale: Optional[torch.Tensor] = None,
                       route: Optional[torch.Tensor] = None, backward_route=None) -> torch.Tensor:
    """SwiGLU FFN of every local expert on its rows. `w_gate_up [G, 2I, H]` (gate rows first), `w_down [G, H, I]`.

    Padding rows of the result are zero. In inference mode the SwiGLU is fused into the first GEMM's epilogue;
    under autograd the pre-activation is kept for the backward pass.
    """
    if backend == 'torch' or not (_supported(x, w_gate_up) and _supported(x, w_down)):
        assert route is None
        y = _torch_ffn(x, w_gate_up, w_down, psum, unaligned)
        return y if row_scale is None else y * row_scale.unsqueeze(1).to(y.dtype)
    if alignment % 128 == 0 and w_gate_up.size(1) % 256 == 0:
        # fused path: no elementwise passes, padding rows come out as zeros
        return GroupedSwiGLUFFN.apply(x, w_gate_up, w_down, row_scale, psum, unaligned, alignment, route, backward_route)
    assert route is None and backward_route is None, 'a combine route needs the fused FFN path (alignment % 128 == 0, intermediate % 128 == 0)'
    if row_scale is not None:
        y = grouped_swiglu_ffn(x, w_gate_up, w_down, psum, unaligned, per_expert_list, alignment, backend)
        return y * row_scale.unsqueeze(1).to(y.dtype)
    if not torch.is_grad_enabled() or not (x.requires_grad or w_gate_up.requires_grad or w_down.requires_grad):
        if w_gate_up.size(1) % 256 == 0:
            act = grouped_gemm_forward(x, w_gate_up, psum, unaligned, swiglu=True)
        else:
            g, u = grouped_gemm_forward(x, w_gate_up, psum, unaligned).chunk(2, dim=-1)
            act = F.silu(g) * u
        y = grouped_gemm_forward(act, w_down, psum, unaligned)
    else:
        h = GroupedLinear.apply(x, w_gate_up, psum, unaligned, alignment)
        g, u = h.chunk(2, dim=-1)
        y = GroupedLinear.apply((F.silu(g) * u).contiguous(), w_down, psum, unaligned, alignment)
    return mask_padding_rows(y, psum, unaligned)


def mask_padding_rows(y: torch.Tensor, psum: torch.Tensor, count: torch.Tensor) -> torch.Tensor:
    """Zero the rows of `y` that belong to no expert (alignment padding), without a host synchronisation."""
    rows = torch.arange(y.size(0), device=y.device)
    idx = torch.searchsorted(psum.long(), rows, right=True).clamp(max=psum.numel() - 1)
    start = (psum - count).long()[idx]
    valid = (rows >= start) & (rows < psum.long()[idx])
    return torch.where(valid.unsqueeze(1), y, torch.zeros((), dtype=y.dtype, device=y.device))
