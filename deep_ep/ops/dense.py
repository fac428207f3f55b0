"""Dense (one-group) linear layers on the grouped tcgen05 GEMM kernels.

The MoE layer's router and shared expert are ordinary dense matrix products. They run on the same hand-written
kernels as the routed experts, with a single group that covers all rows, so that no library GEMM sits on the layer's
path: `dense_linear` (forward, data gradient and weight gradient of `y = x @ w.T`, bf16 operands, fp32 accumulation,
bf16 or fp32 result) and `dense_swiglu_ffn` (the fused SwiGLU FFN node of `grouped_gemm.py` with one group).
Shapes the kernels do not cover (CPU tensors, dimensions that are not multiples of 128) fall back to `F.linear`.
"""
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from .._C_loader import _C
from .grouped_gemm import (EPILOGUE_STORE, MODE_DGRAD, MODE_FORWARD, GroupedSwiGLUFFN, _pairs, grouped_gemm_wgrad)

_ONE_GROUP: Dict[Tuple[int, torch.device], torch.Tensor] = {}


def _one_group(rows: int, device: torch.device) -> torch.Tensor:
    """`[rows]` as a one-element int32 device tensor: both the `psum` and the `count` of a single group of `rows` rows.
    Cached, so that steady-state calls launch nothing for it."""
    key = (rows, device)
    t = _ONE_GROUP.get(key)
    if t is None:
        if len(_ONE_GROUP) > 64:
            _ONE_GROUP.clear()
        t = _ONE_GROUP[key] = torch.full((1,), rows, dtype=torch.int32, device=device)
    return t


def _supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (_C is not None and x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            x.size(0) > 0 and w.size(0) % 128 == 0 and w.size(1) % 128 == 0)


class DenseLinear(torch.autograd.Function):
    """`y = x @ w.T` with `x [T, K]`, `w [N, K]` (both bf16); `y` is bf16, or fp32 (the accumulator as it is) with
    `out_fp32`. Backward: `dx = dy @ w` (bf16), `dw = dy.T @ x` accumulated in fp32 on the tensor core and rounded once."""

    @staticmethod
    def forward(ctx, x, w, out_fp32):
        one = _one_group(x.size(0), x.device)
        y = torch.empty((x.size(0), w.size(0)), dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
        _C.grouped_gemm(x, w.unsqueeze(0), y, one, one, MODE_FORWARD, EPILOGUE_STORE, 0, 1, None, None, _pairs(MODE_FORWARD), None)
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        one = _one_group(x.size(0), x.device)
        dy = dy.to(torch.bfloat16).contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _C.grouped_gemm(dy, w.unsqueeze(0), dx, one, one, MODE_DGRAD, EPILOGUE_STORE, 0, 1, None, None, _pairs(MODE_DGRAD), None)
        if ctx.needs_input_grad[1]:
            # rows beyond the last one are outside the tensors, where the TMA loads of the kernel read zeros
            dw = torch.empty((1, *w.shape), dtype=w.dtype, device=w.device)
            grouped_gemm_wgrad(dy, x, dw, one, one, accumulate=False)
            dw = dw[0]
        return dx, dw, None


def dense_linear(x: torch.Tensor, w: torch.Tensor, out_fp32: bool = False) -> torch.Tensor:
    """`x @ w.T` for 2-D `x`; on a GPU with bf16 operands and 128-aligned `w` it runs on the tcgen05 kernel."""
    if not _supported(x, w):
        # library fallback; an fp32 result is computed in fp32 from the same operands, not rounded to bf16 on the way
        return F.linear(x.float(), w.float()) if out_fp32 else F.linear(x, w)
    return DenseLinear.apply(x.contiguous(), w.contiguous(), out_fp32)


def dense_swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """`(silu(x Wg^T) * (x Wu^T)) Wd^T` with `w_gate_up = [Wg; Wu] [2I, H]` and `w_down [H, I]`: the fused FFN node of the
    routed experts (SwiGLU in the first GEMM's epilogue, tensor-core weight gradients) with one group over all rows."""
    rows = x.size(0)
    if not (_supported(x, w_gate_up) and _supported(x, w_down) and w_gate_up.size(0) % 256 == 0):
        g, u = F.linear(x, w_gate_up).chunk(2, dim=-1)
        return F.linear(F.silu(g) * u, w_down)
    padded = -rows % 128          # the fused node writes whole 128-row tiles of its group
    if padded:
        x = F.pad(x, (0, 0, 0, padded))
    one = _one_group(rows + padded, x.device)
    y = GroupedSwiGLUFFN.apply(x.contiguous(), w_gate_up.unsqueeze(0), w_down.unsqueeze(0), None, one, one, 128, None, None)
    return y[:rows] if padded else y
