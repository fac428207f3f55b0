"""Parallelism strategies of the library by name (the reference's README lists the same set, `README.md:64-84`).

* `ep`: expert parallelism: `EPBuffer.dispatch` / `combine` (all-to-all with per-rank deduplication, expanded
  expert-major layout, cached handles, deferred epilogues), `MoELayer` on top of it.
* `pp`: pipeline parallelism: `PPBuffer.send` / `recv` between ring neighbours with a bounded number of tensors in flight.
* `dp`: data / fully-sharded parallelism and context parallelism building blocks: `BucketBuffer.all_gather`
  (batched, several groups, sessions), `reduce_scatter`, `all_reduce`.
* `engram`: remote memory access: `EngramBuffer` (sharded tables gathered per layer).

Tensor parallelism, sequence parallelism and hybrid scale-out x scale-up domains are not part of the reference
(`csrc/kernels/comm/api.hpp:82-89` there returns one flat domain) and are not provided here either.
"""
from ..buffers.bucket import BucketBuffer, BucketSession
from ..buffers.engram import EngramBuffer
from ..buffers.ep import EPBuffer, EPHandle
from ..buffers.pp import PPBuffer
from ..models.moe_layer import MoEConfig, MoELayer

ep = (EPBuffer, EPHandle, MoELayer, MoEConfig)
pp = (PPBuffer,)
dp = (BucketBuffer, BucketSession)
engram = (EngramBuffer,)

__all__ = ['EPBuffer', 'EPHandle', 'MoELayer', 'MoEConfig', 'PPBuffer', 'BucketBuffer', 'BucketSession', 'EngramBuffer',
           'ep', 'pp', 'dp', 'engram']
