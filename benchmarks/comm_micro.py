"""Timing of the non-EP buffers, shaped after the performance sections of the reference's own tests.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/comm_micro.py

* Engram fetch (`tests/engram/test_engram.py:111-130` of the reference): 2 layers, 512 tokens, 24 entries per token,
  hidden 256 (512 B per bf16 entry), tables of 524,288 and 524,309 entries per rank; bf16 and FP8 + scale factors.
  GB/s = fetched bytes / kernel time.
* Barrier latency (`tests/comm/test_barrier.py:18-36`): 1000 back-to-back device barriers; time per barrier.
* BucketBuffer all-gather size sweep (`tests/bucket/test_session.py:187-235`): 2 tensors of 1 MiB ... 64 MiB per rank
  in flight, in place and out of place, batched (one call) and one call per tensor, inside a session.
All times are CUDA events on the launching stream (or per-kernel device times from the CUPTI activity records where
the reference reports kernel time), maximum over ranks; one JSON line per section on rank 0.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deep_ep  # noqa: E402
from deep_ep.utils.math import align, per_token_cast_to_fp8  # noqa: E402
from deep_ep.utils.testing import L2Flusher, bench_kineto  # noqa: E402


def max_over_ranks(value: float) -> float:
    t = torch.tensor([value], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def timed_ms(fn, iters: int, warmup: int = 3, flusher=None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in pairs:
        if flusher is not None:
            flusher()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return max_over_ranks(sum(a.elapsed_time(b) for a, b in pairs) / iters)


def engram(args, group, rank, world, out):
    entries = [int(v) for v in args.num_entries_per_layer.split(',')]
    hidden, tokens, per_token = args.hidden, args.num_tokens, args.num_entries_per_token
    flusher = L2Flusher()
    for use_fp8 in (False, True):
        dtype = torch.float8_e4m3fn if use_fp8 else torch.bfloat16
        packs = (hidden // 128) * 2 if use_fp8 else 0
        recv_bytes, storage_bytes = deep_ep.EngramBuffer.get_storage_size_hint(group, entries, hidden, tokens, per_token, dtype, packs)
        buf = deep_ep.EngramBuffer(group, recv_bytes, storage_bytes, explicitly_destroy=True)
        buf.set_config(entries, hidden, tokens, per_token, dtype, packs)
        torch.manual_seed(100 + rank)
        tables = [torch.randn(n, hidden, device='cuda', dtype=torch.bfloat16) for n in entries]
        if use_fp8:
            quant = [per_token_cast_to_fp8(t) for t in tables]
            # the tables are sharded over the ranks, their scale factors are replicated: every rank passes all of them
            def everyone(t):              # as bytes: the collective library has no 16-bit integer type
                raw = t.contiguous().view(torch.uint8)
                parts = [torch.empty_like(raw) for _ in range(world)]
                dist.all_gather(parts, raw)
                return torch.cat(parts).view(t.dtype)
            buf.write([q for q, _ in quant], [everyone(s.view(torch.int16)) for _, s in quant])
        else:
            buf.write(tables)
        del tables
        torch.manual_seed(7)
        idx = torch.stack([torch.randint(0, world * n, (tokens, per_token), device='cuda', dtype=torch.int32) for n in entries])

        def fetch_and_wait():
            for hook in buf.fetch(idx, use_tma_aligned_col_major_sf=use_fp8):
                hook()

        ms = timed_ms(fetch_and_wait, args.iters, flusher=flusher)
        profile = bench_kineto(fetch_and_wait, kernel_names='engram_fetch', num_warmups=3, num_tests=args.iters, flush_l2=True,
                               barrier=buf.barrier)
        kernel_us = max_over_ranks(profile.us)
        fetched = len(entries) * tokens * per_token * (hidden * dtype.itemsize + packs * 2)
        out.append({'bench': 'engram_fetch', 'dtype': 'fp8_e4m3+sf' if use_fp8 else 'bf16', 'n_gpus': world,
                    'layers': len(entries), 'tokens': tokens, 'entries_per_token': per_token, 'entry_bytes': hidden * dtype.itemsize,
                    'fetched_bytes': fetched, 'kernel_us': round(kernel_us, 2), 'kernel_gbs': round(fetched / kernel_us / 1e3, 2),
                    'call_ms_events': round(ms, 4), 'remote_share': round((world - 1) / world, 3)})
        buf.destroy()


def barrier_latency(args, group, rank, world, out):
    buffer = deep_ep.EPBuffer(group, num_max_tokens_per_rank=128, hidden=1024, num_topk=8, explicitly_destroy=True)
    n = args.num_barriers

    def loop():
        for _ in range(n):
            buffer.barrier()

    loop()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    loop()
    b.record()
    torch.cuda.synchronize()
    per_call_us = max_over_ranks(a.elapsed_time(b) * 1e3 / n)
    profile = bench_kineto(lambda: [buffer.barrier() for _ in range(100)], kernel_names='rank_barrier', num_warmups=1, num_tests=5,
                           flush_l2=False, barrier=buffer.barrier)
    # the barrier's own latency: n barriers inside ONE kernel launch (every rank passes the same count)
    def in_kernel():
        deep_ep._C.barrier(buffer.context, False, True, False, n)
    in_kernel()
    torch.cuda.synchronize()
    dist.barrier()
    a.record()
    in_kernel()
    b.record()
    torch.cuda.synchronize()
    in_kernel_us = max_over_ranks(a.elapsed_time(b) * 1e3 / n)
    out.append({'bench': 'barrier', 'n_gpus': world, 'barriers': n, 'us_per_barrier_in_one_kernel': round(in_kernel_us, 3),
                'us_per_barrier_back_to_back': round(per_call_us, 3),
                'kernel_us': round(max_over_ranks(profile.us), 3),
                'what': 'in_one_kernel: 1000 barriers executed by one launch / 1000 (the device-side latency of a barrier); back-to-back: events around 1000 launches / 1000 (launch-bound on the host when the kernel is shorter '
                        'than a launch); kernel_us: device time of one barrier kernel from the activity records'})
    buffer.destroy()


def bucket_sweep(args, group, rank, world, out):
    inflight = 2
    max_bytes = 1 << args.max_log2_bytes
    storage = align(inflight * align(world * max_bytes, 2 << 20), 2 << 20)
    bucket = deep_ep.BucketBuffer(group, storage, explicitly_destroy=True)
    rows = []
    for log2 in range(20, args.max_log2_bytes + 1):
        num_bytes = 1 << log2
        tensors = [torch.randn(num_bytes // 2, dtype=torch.bfloat16, device='cuda') for _ in range(inflight)]
        for inplace in (False, True):
            for batched in (False, True):
                def run():
                    with bucket.session() as session:
                        if inplace:
                            regs = [session.allocate((world, num_bytes // 2), torch.bfloat16) for _ in range(inflight)]
                            srcs = [r[rank] for r in regs]
                            handles = [bucket.all_gather(srcs)] if batched else [bucket.all_gather(s) for s in srcs]
                        else:
                            handles = [bucket.all_gather(tensors)] if batched else [bucket.all_gather(t) for t in tensors]
                        for h in handles:
                            h.wait()
                    bucket.barrier()
                ms = timed_ms(run, args.iters)
                rows.append({'bytes_per_rank': num_bytes, 'inplace': inplace, 'batched': batched,
                             'us_per_tensor': round(ms * 1e3 / inflight, 2),
                             'gathered_gbs': round(num_bytes * world * inflight / (ms * 1e6), 2)})
    out.append({'bench': 'bucket_all_gather_sweep', 'n_gpus': world, 'tensors_in_flight': inflight, 'rows': rows,
                'what': 'session + all-gather(s) + wait + barrier per iteration, as the reference times it; GB/s = gathered '
                        'bytes (all ranks\' shards) per rank / time'})
    bucket.destroy()


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--iters', type=int, default=20)
    p.add_argument('--only', default='engram,barrier,bucket')
    p.add_argument('--num-entries-per-layer', default='524288,524309')
    p.add_argument('--hidden', type=int, default=256)
    p.add_argument('--num-tokens', type=int, default=512)
    p.add_argument('--num-entries-per-token', type=int, default=24)
    p.add_argument('--num-barriers', type=int, default=1000)
    p.add_argument('--max-log2-bytes', type=int, default=26)
    args = p.parse_args()
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29563')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', local_rank))
    group = dist.group.WORLD
    out = []
    with torch.inference_mode():
        if 'engram' in args.only:
            engram(args, group, rank, world, out)
        if 'barrier' in args.only:
            barrier_latency(args, group, rank, world, out)
        if 'bucket' in args.only:
            bucket_sweep(args, group, rank, world, out)
    if rank == 0:
        for line in out:
            print(json.dumps(line))
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
