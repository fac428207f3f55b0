"""Two-phase arena for tensors that must live inside a buffer's peer-visible storage.

Phase 1 (`allocate`): the caller describes the tensors it will need; each call returns a `meta` tensor that stands in
for the real one and records where it will sit (offsets are multiples of the allocation alignment, 2 MiB).
Phase 2 (`materialize`): once the owning buffer has created its storage (`num_bytes` long), every stand-in is exchanged
in place for a view of that storage with `torch.utils.swap_tensors`, so that every reference the caller kept now
points at registered memory. Same contract as the reference's `deep_ep/buffers/allocator.py:11-37`
(`BucketBuffer(allocation_plan_or_num_bytes=...)`, `EPBuffer(lb_allocation_plan_or_num_bytes=...)`); this version also
keeps a record per region (`regions`, `describe()`) for diagnostics.
"""
from dataclasses import dataclass
from typing import List, Sequence, Tuple, Union

import torch

from .._C_loader import _C
from ..utils.math import align


@dataclass
class _Region:
    stand_in: torch.Tensor      # meta tensor until the plan is materialised, then the real view (swapped in place)
    offset: int                 # byte offset inside the storage
    num_bytes: int


class BufferAllocator:
    """Plan of aligned regions inside one storage; see the module docstring for the two phases."""

    def __init__(self):
        self.alignment: int = _C.get_num_allocation_alignment()
        self.regions: List[_Region] = []
        self.num_bytes: int = 0             # storage size the plan needs so far (a multiple of the alignment)
        self.materialized: bool = False

    def allocate(self, shape: Union[int, Sequence[int]], dtype: torch.dtype) -> torch.Tensor:
        """Add a tensor of `shape` / `dtype` to the plan and return its stand-in."""
        if self.materialized:
            raise AssertionError('A materialized allocation plan cannot be changed')
        stand_in = torch.empty(shape, dtype=dtype, device='meta')
        region = _Region(stand_in, offset=self.num_bytes, num_bytes=stand_in.nbytes)
        self.regions.append(region)
        # `num_bytes` is kept aligned, so the next region starts on a boundary and the total is a legal storage size
        self.num_bytes = align(region.offset + region.num_bytes, self.alignment)
        return stand_in

    def materialize(self, storage: torch.Tensor) -> None:
        """Turn every stand-in into a view of `storage` (1-D contiguous uint8 of exactly `num_bytes` bytes). Once only."""
        if self.materialized:
            raise AssertionError('An allocation plan can only be materialized once')
        assert storage.dtype == torch.uint8 and storage.dim() == 1 and storage.is_contiguous(), \
            'the storage of an allocation plan is a flat contiguous uint8 tensor'
        assert storage.numel() == self.num_bytes, f'the plan needs {self.num_bytes} bytes, the storage has {storage.numel()}'
        for region in self.regions:
            stand_in = region.stand_in
            view = storage[region.offset:region.offset + region.num_bytes].view(stand_in.dtype).view(stand_in.shape)
            torch.utils.swap_tensors(stand_in, view)          # every holder of the stand-in now holds the view
        self.materialized = True

    @property
    def allocations(self) -> List[Tuple[torch.Tensor, int]]:
        """`(tensor, byte offset)` of every region, in the order of the `allocate` calls."""
        return [(region.stand_in, region.offset) for region in self.regions]

    def describe(self) -> str:
        """One line per region: offset, bytes, dtype and shape (for logs)."""
        lines = [f'{len(self.regions)} regions, {self.num_bytes} bytes, alignment {self.alignment}, '
                 f'{"materialized" if self.materialized else "planned"}']
        lines += [f'  +{r.offset:>12d}  {r.num_bytes:>12d} B  {str(r.stand_in.dtype):<16s} {tuple(r.stand_in.shape)}' for r in self.regions]
        return '\n'.join(lines)
