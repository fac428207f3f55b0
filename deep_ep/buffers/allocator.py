"""Plan-then-materialise arena (reference: `deep_ep/buffers/allocator.py:11-37`)."""
from typing import List, Tuple

import torch

from .._C_loader import _C
from ..utils.math import align


class BufferAllocator:
    """Records aligned sub-allocations as meta tensors; `materialize` turns them into views of one storage."""

    def __init__(self):
        self.alignment = _C.get_num_allocation_alignment()
        self.allocations: List[Tuple[torch.Tensor, int]] = []
        self.num_bytes = 0
        self.materialized = False

    def allocate(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """Reserve an aligned region; the returned meta tensor becomes real at `materialize`."""
        assert not self.materialized, 'A materialized allocation plan cannot be changed'
        placeholder = torch.empty(shape, dtype=dtype, device='meta')
        offset = align(self.num_bytes, self.alignment)
        self.allocations.append((placeholder, offset))
        self.num_bytes = align(offset + placeholder.nbytes, self.alignment)
        return placeholder

    def materialize(self, storage: torch.Tensor) -> None:
        """Swap every placeholder for a view of `storage` (contiguous uint8, exactly `num_bytes` long)."""
        assert not self.materialized, 'An allocation plan can only be materialized once'
        assert storage.is_contiguous() and storage.dtype == torch.uint8 and storage.dim() == 1
        assert storage.numel() == self.num_bytes, f'{storage.numel()=} != {self.num_bytes=}'
        for placeholder, offset in self.allocations:
            real = storage.narrow(0, offset, placeholder.nbytes).view(placeholder.dtype).view(placeholder.shape)
            torch.utils.swap_tensors(placeholder, real)
        self.materialized = True
