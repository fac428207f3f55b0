"""Spawns N worker processes that form a process group (gloo on CPU, NCCL on GPUs) on 127.0.0.1."""
import os
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world_size, port, backend, fn, args, timeout_s=None):
    import faulthandler
    faulthandler.enable()
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    kwargs = dict(backend=backend, init_method=f'tcp://127.0.0.1:{port}', world_size=world_size, rank=rank)
    if timeout_s is not None:
        import datetime
        kwargs['timeout'] = datetime.timedelta(seconds=timeout_s)
    if backend == 'nccl':
        torch.cuda.set_device(rank)
        kwargs['device_id'] = torch.device('cuda', rank)
    dist.init_process_group(**kwargs)
    try:
        fn(rank, world_size, *args)
    except Exception:
        traceback.print_exc()
        raise
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    if backend == 'gloo':
        # The test body has passed. Leave without interpreter finalisation: background threads of the CPU process group
        # occasionally abort the process while static objects are being destroyed ("terminate called without an active
        # exception"), which would turn a passed test into a failed one.
        sys.stdout.flush(), sys.stderr.flush()
        os._exit(0)


def run_distributed(fn, world_size, port, backend='gloo', args=(), timeout_s=None):
    """Run `fn(rank, world_size, *args)` in `world_size` processes; raises if any of them fails."""
    for attempt in range(3):
        try:
            mp.spawn(_worker, args=(world_size, port, backend, fn, args, timeout_s), nprocs=world_size, join=True)
            return
        except Exception as exc:
            # the port was free when it was chosen and taken when rank 0 tried to listen on it: take another one
            if 'EADDRINUSE' not in str(exc) or attempt == 2:
                raise
            import socket
            with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as probe:
                probe.bind(('127.0.0.1', 0))
                port = probe.getsockname()[1]
