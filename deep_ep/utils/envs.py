"""Process-group bootstrap, seeding and rank-ordered printing.

Reference: `deep_ep/utils/envs.py:1-117` (HCCL/NPU). Here the backend is NCCL with one process per
B200, or gloo on CPU when no GPU is present (used by the CPU test tier).
"""
import os
import random
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_local_rank: Optional[int] = None
_local_seed = 0
_global_seed = 0


def has_cuda() -> bool:
    return torch.cuda.is_available()


def default_device() -> torch.device:
    """`cuda:<current>` on a GPU box, else `cpu`."""
    return torch.device('cuda', torch.cuda.current_device()) if has_cuda() else torch.device('cpu')


def bind_to_device_numa_node(device_index: int) -> Optional[int]:
    """Restrict this process to the CPUs of the NUMA node that the given GPU is attached to.

    Pinned host buffers allocated afterwards then sit in memory local to the GPU's PCIe root, which is what host-to-device
    copies of several ranks at once are limited by on two-socket machines. Only this process's CPU affinity changes.
    Returns the node, or `None` when it cannot be determined (nothing is changed then).
    """
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = f'{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0'
        with open(f'/sys/bus/pci/devices/{bus}/numa_node') as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f'/sys/devices/system/node/node{node}/cpulist') as f:
            cpus = set()
            for part in f.read().strip().split(','):
                lo, _, hi = part.partition('-')
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:   # no CUDA device, no sysfs, no permission: leave the process as it is
        return None


def init_seed(global_seed: int) -> None:
    """Seed torch and `random` with `global_seed + rank` so that ranks draw different data."""
    global _local_seed, _global_seed
    _global_seed = global_seed
    _local_seed = global_seed + (dist.get_rank() if dist.is_initialized() else 0)
    torch.manual_seed(_local_seed)
    random.seed(_local_seed)


def get_local_seed() -> int:
    return _local_seed


def get_global_seed() -> int:
    return _global_seed


def dist_print(s: str = '', once_in_node: bool = False) -> None:
    """Print from every rank (or only local rank 0 of each node), then barrier."""
    local_rank = _local_rank if _local_rank is not None else int(os.environ.get('LOCAL_RANK', 0))
    if not once_in_node or local_rank == 0:
        print(s, flush=True)
    if dist.is_initialized():
        dist.barrier()


def get_comm_name(group: dist.ProcessGroup, rank_idx: int) -> str:
    """A stable per-group identifier (the NCCL analogue of the reference's HCCL communicator name)."""
    return f'{getattr(group, "group_name", "group")}:{group.size()}:{rank_idx}'


def init_dist(local_rank: int, num_local_ranks: int, seed: int = 0,
              backend: Optional[str] = None) -> Tuple[int, int, dist.ProcessGroup]:
    """Initialise `torch.distributed` for a spawned worker.

    `MASTER_ADDR`/`MASTER_PORT` locate the rendezvous, `WORLD_SIZE` is the number of *nodes* and
    `RANK` the node index (the launch convention of the reference, `deep_ep/utils/envs.py:93-110`).
    Sets bf16 as default dtype and the rank's GPU as default device when CUDA is available.
    """
    global _local_rank
    _local_rank = local_rank
    ip = os.getenv('MASTER_ADDR', '127.0.0.1')
    port = int(os.getenv('MASTER_PORT', '8361'))
    num_nodes = int(os.getenv('WORLD_SIZE', 1))
    node_rank = int(os.getenv('RANK', 0))
    use_cuda = has_cuda()
    backend = backend or ('nccl' if use_cuda else 'gloo')
    kwargs = dict(backend=backend, init_method=f'tcp://{ip}:{port}',
                  world_size=num_nodes * num_local_ranks, rank=node_rank * num_local_ranks + local_rank)
    if use_cuda:
        torch.cuda.set_device(local_rank)
        if backend == 'nccl':
            kwargs['device_id'] = torch.device('cuda', local_rank)
    dist.init_process_group(**kwargs)
    if use_cuda:
        torch.set_default_dtype(torch.bfloat16)
        torch.set_default_device(f'cuda:{local_rank}')
    init_seed(seed)
    return dist.get_rank(), dist.get_world_size(), dist.distributed_c10d._get_default_group()
