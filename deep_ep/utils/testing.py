"""Benchmark helpers: CUDA-event timing, per-kernel timing through `torch.profiler` (CUPTI), L2
flushing and the "device busy + cross-rank barrier" preamble that hides launch skew between ranks.

Reference: `deep_ep/utils/testing.py:1-394` (`bench`, `parse_num_bytes`, `KernelProfile`, `bench_msprof`).
`bench_msprof` is kept as an alias of `bench_kineto` so that scripts written for the reference run.
"""
import os
import re
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

__all__ = ['KernelProfile', 'bench', 'bench_kineto', 'bench_msprof', 'parse_num_bytes', 'L2Flusher', 'device_busy',
           'bench_events_max_over_ranks']

L2_FLUSH_BYTES = 256 << 20      # larger than the 126 MB L2 of a B200


class L2Flusher:
    """Overwrites a buffer larger than L2 so the next kernel starts with a cold cache."""

    def __init__(self, num_bytes: int = L2_FLUSH_BYTES):
        self.buffer = torch.empty(num_bytes // 4, dtype=torch.int32, device='cuda')

    def __call__(self) -> None:
        self.buffer.zero_()


def device_busy(cycles: int = 2_000_000) -> None:
    """Keep the GPU spinning for a while so that host launch overhead of the next ops is hidden."""
    torch.cuda._sleep(cycles)


def bench(fn: Callable, num_warmups: int = 30, num_tests: int = 30, post_fn: Optional[Callable] = None,
          barrier: Optional[Callable] = None) -> Tuple[float, float, float]:
    """Mean, min and max seconds of `fn` measured with CUDA events on the current stream (this rank only).

    `fn` must enqueue its whole operation, deferred epilogue included. `post_fn` runs after each timed
    iteration, outside the events; `barrier` runs once after warm-up.
    """
    if num_warmups < 0 or num_tests <= 0:
        raise ValueError('num_warmups must be nonnegative and num_tests must be positive')
    torch.cuda.synchronize()
    for _ in range(num_warmups):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    if barrier is not None:
        barrier()
    for start, end in zip(starts, ends):
        start.record()
        fn()
        end.record()
        if post_fn is not None:
            post_fn()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)]
    return sum(times) / len(times), min(times), max(times)


def bench_events_max_over_ranks(times_ms: List[float], group: Optional[dist.ProcessGroup] = None) -> Tuple[float, float, float]:
    """Reduce per-rank mean milliseconds to (max, min, mean) over the ranks of `group`."""
    mean_ms = sum(times_ms) / len(times_ms)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return mean_ms, mean_ms, mean_ms
    t = torch.tensor([mean_ms], dtype=torch.float64, device='cuda')
    gathered = [torch.zeros_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(gathered, t, group=group)
    vals = [g.item() for g in gathered]
    return max(vals), min(vals), sum(vals) / len(vals)


def parse_num_bytes(text: str) -> int:
    """`"1G"`, `"64M"`, `"512K"`, `"1.5GiB"`, `"1048576"` -> bytes (binary multiples)."""
    m = re.fullmatch(r'\s*([0-9]+(?:\.[0-9]+)?)\s*([kmgt])?(?:i?b)?\s*', text, re.IGNORECASE)
    if m is None:
        raise ValueError('Expected a byte count such as 1G, 64M, 512K, or 1048576')
    shift = {'': 0, 'k': 10, 'm': 20, 'g': 30, 't': 40}[(m.group(2) or '').lower()]
    value = int(float(m.group(1)) * (1 << shift))
    if value <= 0:
        raise ValueError('Byte count must be positive')
    return value


@dataclass
class KernelProfile:
    """Average device time of one kernel over the profiled iterations.

    The reference's profile also carries Ascend pipe utilisations; the CUDA counterpart of those
    (tensor pipe, DRAM, NVLink counters) comes from `ncu`, not from a timeline profiler, so only the
    duration and the launch count are recorded here.
    """
    dur_ns: float
    num_calls: int = 1
    name: str = ''
    extra: Dict[str, float] = field(default_factory=dict)

    def __add__(self, other: 'KernelProfile') -> 'KernelProfile':
        return KernelProfile(self.dur_ns + other.dur_ns, max(self.num_calls, other.num_calls),
                             f'{self.name}+{other.name}')

    @property
    def dur_us(self) -> float:
        return self.dur_ns / 1e3

    @property
    def us(self) -> float:
        return self.dur_us

    @property
    def ns(self) -> float:
        return self.dur_ns

    def tflops(self, flops: float) -> float:
        return flops / self.dur_ns / 1e3

    def gbps(self, bytes_moved: float) -> float:
        return bytes_moved / self.dur_ns

    def __str__(self) -> str:
        return f'{self.name or "kernel"}: {self.dur_us:.1f} us x{self.num_calls}'


def bench_kineto(fn: Callable, kernel_names: Union[str, List[str], None] = None, num_warmups: int = 10,
                 num_tests: int = 30, suppress_verbose_output: bool = True, return_all_kernels: bool = False,
                 flush_l2: bool = True, barrier_comm_profiling: bool = False,
                 barrier: Optional[Callable] = None) -> Union[KernelProfile, List[KernelProfile], Dict[str, KernelProfile]]:
    """Per-kernel device time from `torch.profiler` (CUPTI activity records).

    `kernel_names`: `None` requires exactly one kernel; a string selects the unique kernel whose name contains
    it; a list returns one profile per entry. With `barrier_comm_profiling` a device-busy spin and a
    cross-rank barrier run before every iteration (disable with `EP_DISABLE_BARRIER_PROFILING=1`).
    Figures taken under a profiler are for analysis; headline numbers are timed with CUDA events.
    """
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    flusher = L2Flusher() if flush_l2 else None
    barrier_comm_profiling &= int(os.environ.get('EP_DISABLE_BARRIER_PROFILING', 0)) == 0
    dummy = torch.ones(1, device='cuda') if barrier_comm_profiling and barrier is None and dist.is_initialized() else None

    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            if flusher is not None:
                flusher()
            if barrier_comm_profiling:
                device_busy()
                if barrier is not None:
                    barrier()
                elif dummy is not None:
                    dist.all_reduce(dummy)
            fn()
        torch.cuda.synchronize()

    totals: Dict[str, List[float]] = {}
    for evt in prof.events():
        if evt.device_type == torch.autograd.DeviceType.CUDA and evt.device_time_total > 0:
            totals.setdefault(evt.name, []).append(evt.device_time_total * 1e3)
    profiles = {name: KernelProfile(sum(v) / len(v), len(v) // max(num_tests, 1) or 1, name) for name, v in totals.items()}
    if return_all_kernels:
        return profiles

    def pick(pattern: str) -> KernelProfile:
        matched = [p for n, p in profiles.items() if pattern in n]
        if len(matched) != 1:
            listing = '\n'.join(f'  - {n}' for n in profiles) or '  (none)'
            raise RuntimeError(f"No unique kernel matching '{pattern}':\n{listing}")
        return matched[0]

    if kernel_names is None:
        if len(profiles) != 1:
            listing = '\n'.join(f'  - {n}' for n in profiles) or '  (none)'
            raise RuntimeError(f'Expected unique kernel, but found {len(profiles)}:\n{listing}')
        return next(iter(profiles.values()))
    if isinstance(kernel_names, str):
        return pick(kernel_names)
    return [pick(n) for n in kernel_names]


bench_msprof = bench_kineto
