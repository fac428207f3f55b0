"""Batched all-gather and all-reduce through `BucketBuffer` and pipeline send/recv through `PPBuffer`, the latter overlapped with a GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bucket_pp.py

All-gather: 64 bf16 tensors with sizes log-uniform in 4 KB - 64 MB, values ~ N(0,1), gathered in two batches over two
process groups that share one registered storage; compared with one NCCL `all_gather_into_tensor` per tensor.
Bandwidth = bytes RECEIVED per rank / time ("algorithm bandwidth x (N-1)/N" convention of bus bandwidth is also given).
Pipeline: a bf16 [4096, 7168] activation travels to the next rank while a [4096, 7168] x [7168, 7168] GEMM runs on the
compute stream. Times are CUDA events, maximum over ranks.
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deep_ep  # noqa: E402


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev) / iters], device='cuda', dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--num-tensors', type=int, default=64)
    p.add_argument('--iters', type=int, default=10)
    args = p.parse_args()
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29561')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    group_a = dist.group.WORLD
    group_b = dist.new_group(list(range(world)))
    gen = torch.Generator().manual_seed(5)            # same sizes on every rank
    sizes = [int(math.exp(torch.empty(1).uniform_(math.log(4096), math.log(64 << 20), generator=gen).item())) // 256 * 256
             for _ in range(args.num_tensors)]
    shards = [torch.randn(n // 2, device=dev, dtype=torch.bfloat16) for n in sizes]
    total = sum(sizes)
    storage_bytes = (total * world + (2 << 20) * 2 + (2 << 20) - 1) // (2 << 20) * (2 << 20)
    bucket = deep_ep.BucketBuffer([group_a, group_b], storage_bytes, explicitly_destroy=True)
    dsts, off = [], 0
    for n in sizes:
        dsts.append(bucket.storage.narrow(0, off, n * world).view(torch.bfloat16))
        off += n * world
    half = len(sizes) // 2

    def ours():
        h1 = bucket.all_gather(shards[:half], dsts[:half], group=group_a)
        h2 = bucket.all_gather(shards[half:], dsts[half:], group=group_b)
        h1.wait(), h2.wait()

    nccl_out = [torch.empty(n // 2 * world, device=dev, dtype=torch.bfloat16) for n in sizes]

    def nccl():
        for s, o in zip(shards, nccl_out):
            dist.all_gather_into_tensor(o, s)

    # the most NCCL can do for this job: ONE all-gather of all shards laid end to end (the result is rank-major over the
    # whole batch, so a real user would still have to re-slice it per tensor; that pass is not charged)
    flat_shard = torch.cat(shards)
    flat_out = torch.empty(flat_shard.numel() * world, device=dev, dtype=torch.bfloat16)

    def nccl_flat():
        dist.all_gather_into_tensor(flat_out, flat_shard)

    ours()
    torch.cuda.synchronize()
    for d, s in zip(dsts[:4] + dsts[-4:], shards[:4] + shards[-4:]):       # spot check against the local shard
        assert torch.equal(d.view(world, -1)[rank], s)
    ours_ms, nccl_ms, nccl_flat_ms = timed(ours, args.iters), timed(nccl, args.iters), timed(nccl_flat, args.iters)
    del flat_out
    recv_bytes = total * world
    result = {'bench': 'bucket_all_gather+pp_overlap', 'n_gpus': world, 'num_tensors': len(sizes), 'bytes_per_rank_shards': total,
              'all_gather': {'ours_ms': round(ours_ms, 3), 'nccl_ms': round(nccl_ms, 3),
                             'nccl_one_flat_call_ms': round(nccl_flat_ms, 3),
                             'ours_recv_gbs': round(recv_bytes / ours_ms / 1e6, 1), 'nccl_recv_gbs': round(recv_bytes / nccl_ms / 1e6, 1),
                             'ours_bus_gbs': round(recv_bytes * (world - 1) / world / ours_ms / 1e6, 1)}}

    # ---- batched in-place all-reduce of the same 64 registered tensors (the reference declares it without a kernel)
    def ours_ar():
        bucket.all_reduce(dsts, group=group_a).wait()

    def nccl_ar():
        for o in nccl_out:
            dist.all_reduce(o)

    for d in dsts:
        d.normal_()
    check = [d.float().clone() for d in dsts[:2]]
    for c in check:
        dist.all_reduce(c)                           # fp32 reference of the first two tensors
    ours_ar()
    torch.cuda.synchronize()
    for d, c in zip(dsts[:2], check):
        assert torch.allclose(d.float(), c, atol=0.05 * world, rtol=0.02), 'all_reduce differs from the NCCL fp32 sum'
    for d in dsts:
        d.zero_()                                    # keep values finite over the timed repetitions
    for o in nccl_out:
        o.zero_()
    flat_ar = torch.zeros(sum(o.numel() for o in nccl_out), device=dev, dtype=torch.bfloat16)
    ar_ms, nccl_ar_ms = timed(ours_ar, args.iters), timed(nccl_ar, args.iters)
    nccl_ar_flat_ms = timed(lambda: dist.all_reduce(flat_ar), args.iters)      # one call over the same number of bytes
    del flat_ar
    ar_bytes = total * world
    result['all_reduce'] = {'bytes_per_rank': ar_bytes, 'ours_ms': round(ar_ms, 3), 'nccl_ms': round(nccl_ar_ms, 3),
                            'nccl_one_flat_call_ms': round(nccl_ar_flat_ms, 3),
                            'ours_bus_gbs': round(2 * ar_bytes * (world - 1) / world / ar_ms / 1e6, 1),
                            'nccl_bus_gbs': round(2 * ar_bytes * (world - 1) / world / nccl_ar_ms / 1e6, 1)}
    bucket.destroy()

    # ---- pipeline send/recv overlapped with a GEMM
    act = torch.randn(4096, 7168, device=dev, dtype=torch.bfloat16)
    recv = torch.empty_like(act)
    w = torch.randn(7168, 7168, device=dev, dtype=torch.bfloat16)
    pp = deep_ep.PPBuffer(group_a, act.nbytes, 2, explicitly_destroy=True)
    nxt, prv = (rank + 1) % world, (rank + world - 1) % world
    side = torch.cuda.Stream()

    def pp_only():
        pp.send(act, nxt, num_sms=16)
        pp.recv(recv, prv, num_sms=16)

    def gemm_only():
        torch.mm(act, w)

    def overlapped():
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            pp.send(act, nxt, num_sms=16)
            pp.recv(recv, prv, num_sms=16)
        torch.mm(act, w)
        torch.cuda.current_stream().wait_stream(side)

    pp_ms, gemm_ms, both_ms = timed(pp_only, args.iters), timed(gemm_only, args.iters), timed(overlapped, args.iters)
    result['pp_overlap'] = {'pp_ms': round(pp_ms, 3), 'gemm_ms': round(gemm_ms, 3), 'overlapped_ms': round(both_ms, 3),
                            'pp_gbs': round(act.nbytes / pp_ms / 1e6, 1),
                            'overlap_efficiency': round((pp_ms + gemm_ms - both_ms) / min(pp_ms, gemm_ms), 3)}

    # the same exchange with NCCL point-to-point (send to the next rank, receive from the previous one), alone and
    # overlapped with the GEMM, for comparison
    if world > 1:
        def nccl_pp():
            ops = [dist.P2POp(dist.isend, act, nxt), dist.P2POp(dist.irecv, recv, prv)]
            for work in dist.batch_isend_irecv(ops):
                work.wait()

        def nccl_overlapped():
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                nccl_pp()
            torch.mm(act, w)
            torch.cuda.current_stream().wait_stream(side)

        try:
            nccl_ms, nccl_both_ms = timed(nccl_pp, args.iters), timed(nccl_overlapped, args.iters)
            result['pp_overlap'].update({'nccl_p2p_ms': round(nccl_ms, 3), 'nccl_p2p_overlapped_ms': round(nccl_both_ms, 3),
                                         'nccl_p2p_gbs': round(act.nbytes / nccl_ms / 1e6, 1)})
        except Exception as e:
            result['pp_overlap']['nccl_p2p_error'] = str(e).splitlines()[0][:200]
        # `PPBuffer(transport='nccl')`: the same buffered API on top of NCCL point-to-point (staging slots, two process
        # groups for the two directions of a pair)
        try:
            pp_lib = deep_ep.PPBuffer(group_a, act.nbytes, 2, explicitly_destroy=True, transport='nccl')

            def lib_only():
                pp_lib.send(act, nxt)
                pp_lib.recv(recv, prv)

            def lib_overlapped():
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    lib_only()
                torch.mm(act, w)
                torch.cuda.current_stream().wait_stream(side)

            lib_ms, lib_both_ms = timed(lib_only, args.iters), timed(lib_overlapped, args.iters)
            result['pp_overlap'].update({'ppbuffer_nccl_transport_ms': round(lib_ms, 3),
                                         'ppbuffer_nccl_transport_overlapped_ms': round(lib_both_ms, 3)})
            pp_lib.destroy()
        except Exception as e:
            result['pp_overlap']['ppbuffer_nccl_transport_error'] = str(e).splitlines()[0][:200]
    if rank == 0:
        print(json.dumps(result))
    pp.destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
