"""Run-time kernel specialisation: compile a translation unit against the package's `include/` tree with nvcc
for sm_100a, cache the cubin on disk by content hash, load it through the driver and launch it on the current
stream. The counterpart of the reference's DeepJIT layer (`csrc/runtime/jit.hpp:15-118`); environment switches:
`EP_JIT_CACHE_DIR`, `EP_JIT_NVCC`, `EP_JIT_DEBUG`, `EP_JIT_PRINT_COMPILER_COMMAND`, `EP_JIT_KERNEL_DEBUG_INFO`
(each also read with the `DJ_JIT_` prefix).
"""
from typing import Sequence, Tuple, Union

import torch

from .._C_loader import _C

Arg = Union[torch.Tensor, int, float, Tuple[str, Union[int, float]]]


def compile_kernel(name: str, source: str, arch: str = 'sm_100a') -> str:
    """Compile `source` (a full `.cu` translation unit) and return the path of the cached cubin."""
    return _C.jit_compile(name, source, arch)


def _pack(arg: Arg):
    if isinstance(arg, torch.Tensor):
        return 'ptr', arg.data_ptr()
    if isinstance(arg, tuple):
        return arg
    if isinstance(arg, bool) or isinstance(arg, int):
        return 'i32', int(arg)
    if isinstance(arg, float):
        return 'f32', arg
    raise TypeError(f'unsupported kernel argument {arg!r}')


def launch(cubin: str, symbol: str, grid: int, block: int, args: Sequence[Arg], smem_bytes: int = 0,
           cooperative: bool = False) -> None:
    """Launch `symbol` from `cubin` on the current stream. Tensors are passed as device pointers, Python ints as
    32-bit ints, floats as fp32; use `('i64', value)` for 64-bit integers."""
    _C.jit_launch(cubin, symbol, grid, block, smem_bytes, [_pack(a) for a in args], cooperative,
                  torch.cuda.current_stream().cuda_stream)
