"""Numeric helpers: alignment arithmetic, similarity metric and the 1x128 FP8 cast.

Behavioural parity with the reference's `deep_ep/utils/math.py:1-64`; the FP8 cast is the
host-side oracle for the fused quantisation done inside the dispatch kernel.
"""
from typing import Tuple

import torch

FP8_E4M3_MAX = 448.0
SF_GROUP = 128


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def safe_div(a, b) -> float:
    """`a / b`, with `0 / 0 == 0` (any other division by zero still raises)."""
    if b == 0 and a == 0:
        return 0
    return a / b


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """`1 - cosine-like similarity` of `x + 1` and `y + 1` in fp64 (0 means identical)."""
    xd, yd = x.double() + 1, y.double() + 1
    return (1 - 2 * (xd * yd).sum() / (xd.square().sum() + yd.square().sum())).item()


def per_token_cast_to_fp8(x: torch.Tensor, round_scale: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise `[m, n]` to e4m3 with one fp32 scale per 128 consecutive columns.

    `scale = max(amax, 1e-4) / 448`; the value stored is `x * (448 / max(amax, 1e-4))` rounded
    to e4m3. Returns `(x_fp8 [m, n], scales [m, ceil(n / 128)] fp32)`.
    With `round_scale` every scale is rounded up to a power of two (`2^ceil(log2(amax * (1 / 448)))`, the UE8M0 form)
    and the stored value is `x / scale`.
    """
    assert x.dim() == 2
    m, n = x.shape
    n_pad = align(n, SF_GROUP)
    xp = torch.nn.functional.pad(x, (0, n_pad - n)) if n_pad != n else x
    groups = xp.reshape(m, n_pad // SF_GROUP, SF_GROUP)
    amax = groups.abs().float().amax(dim=2).clamp(min=1e-4)
    if round_scale:
        bits = (amax * (1.0 / FP8_E4M3_MAX)).contiguous().view(torch.int32)
        exponent = (((bits >> 23) & 0xff) + ((bits & 0x7fffff) != 0).int()).clamp(1, 253)
        scale = (exponent << 23).view(torch.float32)
        q = (groups.float() / scale.unsqueeze(2)).to(torch.float8_e4m3fn)
        return q.reshape(m, n_pad)[:, :n].contiguous(), scale
    q = (groups * (FP8_E4M3_MAX / amax).unsqueeze(2)).to(torch.float8_e4m3fn)
    return q.reshape(m, n_pad)[:, :n].contiguous(), amax / FP8_E4M3_MAX


def per_token_cast_back(x_fp8: torch.Tensor, x_scales: torch.Tensor) -> torch.Tensor:
    """Inverse of `per_token_cast_to_fp8`; int32 scales are read as packed UE8M0 exponents."""
    if x_fp8.numel() == 0:
        return x_fp8.to(torch.bfloat16)
    assert x_fp8.dim() == 2
    m, n = x_fp8.shape
    n_pad = align(n, SF_GROUP)
    xp = torch.nn.functional.pad(x_fp8.view(torch.uint8), (0, n_pad - n)).view(torch.float8_e4m3fn) \
        if n_pad != n else x_fp8
    if x_scales.dtype == torch.int:
        # four exponent bytes per int32, each is the biased exponent of a power-of-two scale
        x_scales = (x_scales.contiguous().view(torch.uint8).to(torch.int) << 23).view(torch.float)
    vals = xp.to(torch.float32).reshape(m, n_pad // SF_GROUP, SF_GROUP)
    out = vals * x_scales.reshape(m, -1, 1)[:, :n_pad // SF_GROUP]
    return out.reshape(m, n_pad).to(torch.bfloat16)[:, :n].contiguous()


def count_bytes(*tensors) -> int:
    """Total logical bytes of tensors (nested tuples/lists allowed, `None` ignored)."""
    n = 0
    for t in tensors:
        if t is None:
            continue
        n += count_bytes(*t) if isinstance(t, (tuple, list)) else t.numel() * t.element_size()
    return n
