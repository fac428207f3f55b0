"""FP8 training path of the expert FFN (opt-in: `MoEConfig.fp8_training`).

The two forward GEMMs and the two data-gradient GEMMs of the SwiGLU FFN run on the hardware-scaled FP8 tensor-core
kernel (`tcgen05.mma.kind::mxf8f6f4.block_scale`): e4m3 operands, power-of-two scales (UE8M0 bytes), one per row and
128 columns for activations and gradients, one per 128 x 128 block for weights. The weight gradients stay in bf16
(fp32 accumulation in tensor memory), so the master weights, their gradients and the optimizer never see FP8.

    forward    x --row quant--> GEMM1 (store) --> h = [gate | up] bf16 --SwiGLU + quant--> GEMM2 (store) --> y
    backward   dy --row quant--> dgrad GEMM2 (weights transposed at quantisation time) --> dact
               dh = SwiGLU'(h, dact) --row quant--> dgrad GEMM1 --> dx;   dW2 = dy^T act,  dW1 = dh^T x  (bf16)

A 128 x 128 block scale is its own transpose, so the transposed weight copy that the data-gradient GEMMs read holds
exactly the same quantised values as the forward copy. Quantised weights are cached per parameter version: they are
refreshed after every optimizer step (in-place update), not on every micro-batch.

Everything also runs on CPU tensors through a plain PyTorch emulation of the same arithmetic (dequantise, matmul in
fp32, round to bf16): that is the oracle of the GPU tests and what the CPU tests exercise.
The reference contains no matrix math; this follows the usage the layer is meant for (`README.md:178-194` there).
"""
from typing import Dict, Optional, Tuple

import torch

from .._C_loader import _C
from .grouped_gemm import (_ranges, _wgrad, grouped_gemm_fp8_forward, per_block_cast_to_fp8_ue8m0,
                           per_token_cast_to_fp8_ue8m0, row_scale_grad, ue8m0_to_float)


# --------------------------------------------------------------------------------------------- quantisers
def row_quant(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 `[rows, n]` -> `(e4m3 [rows, n], UE8M0 bytes [rows, n / 128])`."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    if x.is_cuda:
        return _C.row_quant_ue8m0(x.contiguous())
    return per_token_cast_to_fp8_ue8m0(x)


def swiglu_quant(h: torch.Tensor, row_scale: Optional[torch.Tensor], keep_bf16: bool = True):
    """`h = [gate | up]` bf16 `[rows, 2 I]` -> `(act bf16 or None, act e4m3, UE8M0 bytes [rows, I / 128])` with
    `act = silu(gate) * up * row_scale`; the quantised copy is taken from the fp32 values, not from the rounded bf16."""
    assert h.dim() == 2 and h.size(1) % 256 == 0
    if h.is_cuda:
        return _C.swiglu_quant_ue8m0(h.contiguous(), row_scale, keep_bf16)
    g, u = h.float().chunk(2, dim=-1)
    act = g / (1.0 + torch.exp(-g)) * u
    if row_scale is not None:
        act = act * row_scale.unsqueeze(1)
    q, sf = per_token_cast_to_fp8_ue8m0(act)
    return (act.to(torch.bfloat16) if keep_bf16 else None), q, sf


def block_quant(w: torch.Tensor, transposed: bool = False):
    """bf16 `[g, n, k]` -> `(e4m3 [g, n, k], UE8M0 [g, n / 128, k / 128])`, with `transposed` followed by the same
    quantised matrices transposed: `(e4m3 [g, k, n], UE8M0 [g, k / 128, n / 128])`."""
    assert w.dim() == 3 and w.size(1) % 128 == 0 and w.size(2) % 128 == 0
    if w.is_cuda:
        return tuple(_C.block_quant_ue8m0(w.contiguous(), transposed))
    q, sf = per_block_cast_to_fp8_ue8m0(w)
    if not transposed:
        return q, sf
    qt = q.view(torch.uint8).transpose(1, 2).contiguous().view(torch.float8_e4m3fn)
    return q, sf, qt, sf.transpose(1, 2).contiguous()


class Fp8WeightCache:
    """Quantised copies (forward and transposed) of weight stacks, refreshed when a parameter's version changes."""

    def __init__(self):
        self._entries: Dict[int, Tuple[int, int, tuple]] = {}

    def get(self, w: torch.Tensor) -> tuple:
        key = id(w)
        entry = self._entries.get(key)
        if entry is None or entry[0] != w._version or entry[1] != w.data_ptr():
            with torch.no_grad():
                entry = (w._version, w.data_ptr(), block_quant(w.detach(), transposed=True))
            self._entries[key] = entry
        return entry[2]

    def clear(self) -> None:
        self._entries.clear()


# --------------------------------------------------------------------------------------------- GEMM
def _dequant_rows(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    scale = ue8m0_to_float(sf) if sf.dtype == torch.uint8 else sf
    return q.float() * scale.repeat_interleave(128, dim=1)


def _dequant_blocks(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    scale = ue8m0_to_float(sf) if sf.dtype == torch.uint8 else sf
    return q.float() * scale.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)


def fp8_gemm(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor, psum: torch.Tensor,
             count: torch.Tensor, alignment: int, route: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 `y[rows_e] = (a_q * a_sf)[rows_e] @ (b_q[e] * b_sf[e]).T`, rows outside the experts' regions zero."""
    if a_q.is_cuda:
        assert a_q.size(1) % 512 == 0 and b_q.size(1) % 256 == 0, \
            'the hardware-scaled FP8 GEMM needs K to be a multiple of 512 and N a multiple of 256'
        return grouped_gemm_fp8_forward(a_q, a_sf, b_q, b_sf, psum, count, alignment=alignment, route=route)
    assert route is None
    y = torch.zeros((a_q.size(0), b_q.size(1)), dtype=torch.bfloat16)
    a = _dequant_rows(a_q, a_sf)
    for e, (start, c) in enumerate(_ranges(psum, count)):
        if c:
            y[start:start + c] = (a[start:start + c] @ _dequant_blocks(b_q[e], b_sf[e]).t()).to(torch.bfloat16)
    return y


def _swiglu_backward(h: torch.Tensor, dact: torch.Tensor, row_scale: Optional[torch.Tensor]) -> torch.Tensor:
    if h.is_cuda:
        return _C.swiglu_backward(h, dact, row_scale)
    g, u = h.float().chunk(2, dim=-1)
    d = dact.float() if row_scale is None else dact.float() * row_scale.unsqueeze(1)
    sig = torch.sigmoid(g)
    return torch.cat([d * u * sig * (1.0 + g * (1.0 - sig)), d * g * sig], dim=-1).to(torch.bfloat16)


class GroupedSwiGLUFFNFp8(torch.autograd.Function):
    """`y = (silu(x Wg^T) * (x Wu^T) * row_scale) Wd^T` per expert with FP8 forward and data-gradient GEMMs.

    `route` / `backward_route` have the meaning they have in `GroupedSwiGLUFFN`: rows that are their token's only one
    are stored by the producing GEMM straight into the owner's combine landing slot."""

    @staticmethod
    def forward(ctx, x, w_gate_up, w_down, row_scale, psum, count, alignment, cache, route=None, backward_route=None):
        w1_q, w1_sf, w1t_q, w1t_sf = cache.get(w_gate_up)
        w2_q, w2_sf, w2t_q, w2t_sf = cache.get(w_down)
        x_q, x_sf = row_quant(x)
        h = fp8_gemm(x_q, x_sf, w1_q, w1_sf, psum, count, alignment)
        act, act_q, act_sf = swiglu_quant(h, row_scale, keep_bf16=True)
        y = fp8_gemm(act_q, act_sf, w2_q, w2_sf, psum, count, alignment, route=route)
        ctx.save_for_backward(x, w_gate_up, w_down, row_scale, psum, count, h, act)
        ctx.transposed = (w1t_q, w1t_sf, w2t_q, w2t_sf)
        ctx.alignment, ctx.backward_route = alignment, backward_route
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_gate_up, w_down, row_scale, psum, count, h, act = ctx.saved_tensors
        w1t_q, w1t_sf, w2t_q, w2t_sf = ctx.transposed
        # the weight-gradient kernel wants 64-row aligned regions; on the CPU the per-expert loop is used
        wgrad_alignment = ctx.alignment if dy.is_cuda else 1
        dy = dy.contiguous()
        dy_q, dy_sf = row_quant(dy)
        dact = fp8_gemm(dy_q, dy_sf, w2t_q, w2t_sf, psum, count, ctx.alignment)
        dw_down = _wgrad(dy, act, w_down, psum, count, wgrad_alignment) if ctx.needs_input_grad[2] else None
        d_row_scale = row_scale_grad(dact, act, row_scale) if row_scale is not None and ctx.needs_input_grad[3] else None
        dh = _swiglu_backward(h, dact, row_scale)
        dx = None
        if ctx.needs_input_grad[0]:
            table = None
            if ctx.backward_route is not None:
                table, barrier = ctx.backward_route
                barrier()
            dh_q, dh_sf = row_quant(dh)
            dx = fp8_gemm(dh_q, dh_sf, w1t_q, w1t_sf, psum, count, ctx.alignment, route=table)
        dw_gate_up = _wgrad(dh, x, w_gate_up, psum, count, wgrad_alignment) if ctx.needs_input_grad[1] else None
        return dx, dw_gate_up, dw_down, d_row_scale, None, None, None, None, None, None


def grouped_swiglu_ffn_fp8_training(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, psum: torch.Tensor,
                                    count: torch.Tensor, alignment: int, cache: Fp8WeightCache,
                                    row_scale: Optional[torch.Tensor] = None, route: Optional[torch.Tensor] = None,
                                    backward_route=None) -> torch.Tensor:
    """Differentiable SwiGLU FFN of every local expert with FP8 forward and data-gradient GEMMs (see the module text).
    `w_gate_up [G, 2 I, H]`, `w_down [G, H, I]` bf16 master weights; `H` and `I` multiples of 512, `alignment` of 128."""
    hidden, inter = w_down.size(1), w_down.size(2)
    assert x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert alignment % 128 == 0 and hidden % 512 == 0 and inter % 512 == 0 and w_gate_up.size(1) == 2 * inter
    return GroupedSwiGLUFFNFp8.apply(x, w_gate_up, w_down, row_scale, psum, count, alignment, cache, route, backward_route)
