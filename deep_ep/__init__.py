"""deep_ep for NVIDIA B200: expert-parallel dispatch/combine, pipeline send/recv, batched all-gather
and remote embedding gathers over NVLink peer memory. Public surface of the reference's
`deep_ep/__init__.py:26-40`."""
import os

import torch

# Written by setup.py at build time: the version with the source revision, and the values that the run-time compiler's
# environment switches had during the build. Those become defaults; the caller's environment always wins.
__version__ = '1.0.0'
try:
    from ._build_info import persistent_envs, version as __version__
    for _key, _value in persistent_envs.items():
        os.environ.setdefault(_key, _value)
except ImportError:
    pass

from ._C_loader import _C


def init_jit() -> None:
    """Point the runtime kernel compiler at this package (its `include/` tree ships with the package)."""
    _C.init_jit(os.path.dirname(os.path.abspath(__file__)))


init_jit()
# EP_WARP_COOPERATION=1: decode-sized combine calls let several warps share one row (`_C.set_warp_cooperation`)
if os.environ.get('EP_WARP_COOPERATION', '0') == '1':
    _C.set_warp_cooperation(True)

from . import comm
from .comm import (destroy_all_managed_comm, destroy_all_managed_hccl_comm, get_logical_domain_size,
                   get_physical_domain_size)
from .buffers.allocator import BufferAllocator
from .buffers.base import BufferBase
from .buffers.ep import EPBuffer, EPHandle
from .buffers.engram import EngramBuffer
from .buffers.bucket import BucketBuffer, BucketSession
from .buffers.pp import PPBuffer
from .utils.event import EventOverlap, EventHandle
from .utils.envs import init_seed, get_local_seed, get_global_seed, dist_print, init_dist
from .utils.testing import KernelProfile, bench, bench_kineto, bench_msprof

get_num_allocation_alignment = _C.get_num_allocation_alignment
get_num_rdma_alignment = _C.get_num_rdma_alignment
get_num_tma_alignment = _C.get_num_tma_alignment
topk_idx_t = _C.topk_idx_t
EPException = _C.EPException
