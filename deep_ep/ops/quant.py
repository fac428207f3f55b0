"""Per-token FP8 (e4m3, 1x128 fp32 scales) quantisation as a run-time specialised CUDA kernel."""
from typing import Dict, Tuple

import torch

from . import jit

_SOURCE = '''
#include <deep_ep/kernels/quant.cuh>

extern "C" __global__ void __launch_bounds__(256) per_token_quant(const __nv_bfloat16* x, uint8_t* q, float* sf, int num_rows) {
    deep_ep::kernels::per_token_quant_body<%d>(x, q, sf, num_rows);
}
'''
_cubins: Dict[int, str] = {}


def per_token_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """`[m, n]` bf16 on a GPU -> `(e4m3 [m, n], fp32 scales [m, n / 128])`, `n` a multiple of 128.

    Bit-identical to `deep_ep.utils.math.per_token_cast_to_fp8` on CUDA tensors; the kernel is compiled once per
    hidden size (hidden is a template constant, so the per-row loop is fully unrolled).
    """
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous() and x.size(1) % 128 == 0
    m, n = x.shape
    if n not in _cubins:
        _cubins[n] = jit.compile_kernel(f'per_token_quant_{n}', _SOURCE % n)
    q = torch.empty((m, n), dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty((m, n // 128), dtype=torch.float32, device=x.device)
    if m:
        grid = min((m + 7) // 8, 148 * 8)
        jit.launch(_cubins[n], 'per_token_quant', grid, 256, [x, q, sf, m])
    return q, sf
