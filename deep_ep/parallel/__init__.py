"""Process-group layout for the communication buffers: which ranks form an expert-parallel group, a pipeline and a
data-parallel (bucket all-gather / reduce-scatter) group, and the buffers built on them.

The buffers of this library take a `torch.distributed` process group each. A job that combines expert, pipeline and
data parallelism needs one group per dimension and per rank, created in the same order on every rank (group creation
is collective). `ParallelMesh` does that bookkeeping: ranks are laid out as `[pp][dp][ep]` with `ep` innermost, so
that the ranks of one expert-parallel group are neighbours (the GPUs of one NVSwitch domain).
"""
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch.distributed as dist

__all__ = ['ParallelMesh']


@dataclass
class _Axis:
    size: int
    stride: int
    group: Optional[dist.ProcessGroup] = None
    ranks: Tuple[int, ...] = ()


class ParallelMesh:
    """`world = pp x dp x ep` ranks; every rank belongs to exactly one group per axis.

    `mesh.group('ep')` etc. are the process groups of the calling rank, `mesh.coords` its position, and the
    `ep_buffer / pp_buffer / bucket_buffer / engram_buffer` helpers construct the library's buffers on the matching
    group. All ranks of the world must construct the mesh (with the same sizes): `dist.new_group` is collective.
    """

    AXES = ('pp', 'dp', 'ep')

    def __init__(self, ep_size: int = 1, pp_size: int = 1, dp_size: Optional[int] = None, backend: Optional[str] = None,
                 *, world_size: Optional[int] = None, rank: Optional[int] = None):
        """`world_size` and `rank` are taken from `torch.distributed`; passing both instead gives a layout-only mesh
        (coordinates and group membership, no process groups), which is what planning tools and tests need."""
        layout_only = world_size is not None and rank is not None
        if layout_only:
            self.world_size, self.rank = world_size, rank
        else:
            assert dist.is_initialized(), 'initialise torch.distributed first'
            self.world_size, self.rank = dist.get_world_size(), dist.get_rank()
        assert ep_size >= 1 and pp_size >= 1 and self.world_size % (ep_size * pp_size) == 0, \
            f'{self.world_size} ranks cannot be split into pp={pp_size} x ep={ep_size}'
        dp_size = self.world_size // (ep_size * pp_size) if dp_size is None else dp_size
        assert pp_size * dp_size * ep_size == self.world_size, 'pp x dp x ep must equal the world size'
        self.axes: Dict[str, _Axis] = {'pp': _Axis(pp_size, dp_size * ep_size), 'dp': _Axis(dp_size, ep_size), 'ep': _Axis(ep_size, 1)}
        self.coords = self.coords_of(self.rank)
        for name in self.AXES:
            for ranks in self.groups_of(name):
                # one-rank groups are created too: the buffers run on them as loop-back groups
                group = None if layout_only else dist.new_group(list(ranks), backend=backend)
                if self.rank in ranks:
                    self.axes[name].group, self.axes[name].ranks = group, ranks

    def coords_of(self, rank: int) -> Dict[str, int]:
        return {name: (rank // axis.stride) % axis.size for name, axis in self.axes.items()}

    def rank_of(self, **coords: int) -> int:
        """Global rank at the given coordinates; axes that are not named keep the calling rank's coordinate."""
        full = dict(self.coords, **coords)
        assert all(0 <= full[name] < self.axes[name].size for name in self.AXES)
        return sum(full[name] * self.axes[name].stride for name in self.AXES)

    def groups_of(self, name: str) -> List[Tuple[int, ...]]:
        """Every group of one axis (the same list, in the same order, on every rank)."""
        axis = self.axes[name]
        seen, groups = set(), []
        for rank in range(self.world_size):
            base = rank - ((rank // axis.stride) % axis.size) * axis.stride
            if base not in seen:
                seen.add(base)
                groups.append(tuple(base + i * axis.stride for i in range(axis.size)))
        return groups

    def group(self, name: str) -> dist.ProcessGroup:
        return self.axes[name].group

    def size(self, name: str) -> int:
        return self.axes[name].size

    # neighbours along the pipeline (global ranks of this rank's pipeline group, wrapping around)
    def pp_next(self) -> int:
        return self.rank_of(pp=(self.coords['pp'] + 1) % self.axes['pp'].size)

    def pp_prev(self) -> int:
        return self.rank_of(pp=(self.coords['pp'] - 1) % self.axes['pp'].size)

    # ---- buffers on the matching groups
    def ep_buffer(self, **kwargs):
        from ..buffers.ep import EPBuffer
        return EPBuffer(self.group('ep'), **kwargs)

    def pp_buffer(self, *args, **kwargs):
        from ..buffers.pp import PPBuffer
        return PPBuffer(self.group('pp'), *args, **kwargs)

    def bucket_buffer(self, *args, **kwargs):
        from ..buffers.bucket import BucketBuffer
        return BucketBuffer(self.group('dp'), *args, **kwargs)

    def engram_buffer(self, *args, **kwargs):
        from ..buffers.engram import EngramBuffer
        return EngramBuffer(self.group('ep'), *args, **kwargs)
