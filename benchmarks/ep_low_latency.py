"""Low-latency (decode) dispatch/combine captured in CUDA graphs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/ep_low_latency.py

128 tokens per rank, hidden 7168, 256 experts, top-8 with skewed routing (gating logits N(0,1) plus a per-expert
bias N(0,2), so a few experts are hot), FP8 dispatch quantised inside the kernel (1x128 scales), BF16 combine,
`do_cpu_sync=False` (outputs have worst-case capacity, nothing blocks the host), deferred epilogues. Two graphs are
captured: dispatch (issue + expand) and combine (issue + reduce). Times are CUDA-event times per replay, maximum
over ranks. The reference cannot be captured in a graph (`README.md:84`); this mode is new.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deep_ep  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--num-tokens', type=int, default=128)
    p.add_argument('--hidden', type=int, default=7168)
    p.add_argument('--num-topk', type=int, default=8)
    p.add_argument('--num-experts', type=int, default=256)
    p.add_argument('--num-sms', type=int, nargs='+', default=[8, 16, 32])
    p.add_argument('--replays', type=int, default=100)
    p.add_argument('--profile', action='store_true', help='print per-kernel device times of eager iterations (analysis only)')
    p.add_argument('--layers', type=int, default=0,
                   help='also capture this many dispatch + combine pairs in one graph and report the time per pair')
    p.add_argument('--warp-cooperation', action='store_true', help='let several warps share one row in the combine kernels')
    p.add_argument('--phase-trace', action='store_true', help='print the per-phase time breakdown of the four EP kernels')
    args = p.parse_args()

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29541')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(99)
    T, H, K, E = args.num_tokens, args.hidden, args.num_topk, args.num_experts
    expert_bias = torch.randn(E, device=dev) * 2.0                  # same on every rank: a few hot experts
    torch.manual_seed(100 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(T, E, device=dev) + expert_bias
    top_logits, topk_idx = logits.topk(K, dim=-1)
    topk_w = torch.softmax(top_logits, dim=-1).float()

    if args.warp_cooperation:
        deep_ep._C.set_warp_cooperation(True)
    buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=T, hidden=H, num_topk=K, explicitly_destroy=True)
    results = []
    for num_sms in args.num_sms:
        common = dict(num_experts=E, num_max_tokens_per_rank=T, expert_alignment=1, num_sms=num_sms, do_expand=True,
                      do_cpu_sync=False, async_with_compute_stream=True, defer_epilogue=True, fused_fp8_quant=True)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(3):                                       # warm-up outside of capture
                (rx, rsf), _, rw, handle = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_w, **common).current_stream_wait()
                y = torch.randn(rx.size(0), H, device=dev, dtype=torch.bfloat16)
                buffer.combine(y, handle, topk_weights=rw, async_with_compute_stream=True, defer_epilogue=True).current_stream_wait()
            torch.cuda.synchronize()
            dist.barrier()
            g_dispatch, g_combine = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_dispatch, stream=side):
                (rx, rsf), _, rw, handle = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_w, **common).current_stream_wait()
            with torch.cuda.graph(g_combine, stream=side):
                combined, combined_w = buffer.combine(y, handle, topk_weights=rw, async_with_compute_stream=True,
                                                      defer_epilogue=True).current_stream_wait()
        torch.cuda.synchronize()
        dist.barrier()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.replays)]
        for i in range(10 + args.replays):
            e = ev[max(i - 10, 0)]
            e[0].record()
            g_dispatch.replay()
            e[1].record()
            g_combine.replay()
            e[2].record()
        torch.cuda.synchronize()
        buffer.runtime.check_status()
        d_us = sum(e[0].elapsed_time(e[1]) for e in ev) / len(ev) * 1e3
        c_us = sum(e[1].elapsed_time(e[2]) for e in ev) / len(ev) * 1e3
        # replayed result must equal an eager run (weights routed back exactly)
        assert torch.equal(combined_w, topk_w), 'graph replay returned wrong routed weights'
        t = torch.tensor([d_us, c_us], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        num_recv = int(handle.psum_num_recv_tokens_per_rank[-1])
        entry = {'num_sms': num_sms, 'dispatch_us': round(t[0].item(), 2), 'combine_us': round(t[1].item(), 2),
                 'recv_tokens_rank0': num_recv}
        if args.layers > 0:
            # a decode step as a serving engine captures it: `layers` dispatch + combine pairs in ONE graph, so the cost of
            # launching a graph is paid once per step and not once per operation
            g_step = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g_step, stream=side):
                    for _ in range(args.layers):
                        (rx2, _), _, rw2, h2 = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_w, **common).current_stream_wait()
                        buffer.combine(y, h2, topk_weights=rw2, async_with_compute_stream=True, defer_epilogue=True).current_stream_wait()
            torch.cuda.synchronize()
            dist.barrier()
            step_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.replays)]
            for i in range(3 + args.replays):
                a_ev, b_ev = step_ev[max(i - 3, 0)]
                a_ev.record()
                g_step.replay()
                b_ev.record()
            torch.cuda.synchronize()
            buffer.runtime.check_status()
            per_pair = torch.tensor([sum(a_ev.elapsed_time(b_ev) for a_ev, b_ev in step_ev) / len(step_ev) * 1e3 / args.layers],
                                    device=dev, dtype=torch.float64)
            dist.all_reduce(per_pair, op=dist.ReduceOp.MAX)
            entry['dispatch_plus_combine_us_in_one_graph'] = round(per_pair.item(), 2)
            entry['layers_per_graph'] = args.layers
        results.append(entry)
    if args.profile:
        from deep_ep.utils.testing import bench_kineto
        common = dict(num_experts=E, num_max_tokens_per_rank=T, expert_alignment=1, num_sms=args.num_sms[-1], do_expand=True,
                      do_cpu_sync=False, async_with_compute_stream=True, defer_epilogue=True, fused_fp8_quant=True)

        def eager():
            (rx, rsf), _, rw, h = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_w, **common).current_stream_wait()
            buffer.combine(y, h, topk_weights=rw, async_with_compute_stream=True, defer_epilogue=True).current_stream_wait()

        profiles = bench_kineto(eager, return_all_kernels=True, num_tests=20, flush_l2=False, barrier_comm_profiling=True)
        if rank == 0:
            for name, prof in sorted(profiles.items(), key=lambda kv: -kv[1].dur_ns):
                print(f'  {prof.dur_us:9.2f} us x{prof.num_calls}  {name[:100]}')
    if args.phase_trace:
        # where the time goes inside the four kernels: `%globaltimer` stamps at the phase boundaries (eager launches)
        common = dict(num_experts=E, num_max_tokens_per_rank=T, expert_alignment=1, num_sms=args.num_sms[-1], do_expand=True,
                      do_cpu_sync=False, async_with_compute_stream=True, defer_epilogue=True, fused_fp8_quant=True)

        def traced():
            (rx, rsf), _, rw, h = buffer.dispatch(x, topk_idx=topk_idx, topk_weights=topk_w, **common).current_stream_wait()
            buffer.combine(y, h, topk_weights=rw, async_with_compute_stream=True, defer_epilogue=True).current_stream_wait()

        buffer.enable_phase_trace()
        for _ in range(5):
            traced()
        torch.cuda.synchronize()
        dist.barrier()
        traced()
        trace = buffer.read_phase_trace()
        gathered = [None] * world
        dist.all_gather_object(gathered, trace)
        buffer.disable_phase_trace()
        if rank == 0:
            for r, tr in enumerate(gathered):
                print(f'phase trace rank {r} (us): ' + json.dumps({k: ({p: round(v, 2) for p, v in val.items()} if isinstance(val, dict)
                                                                      else round(val, 2)) for k, val in tr.items()}))
    if rank == 0:
        print(json.dumps({'bench': 'ep_low_latency_cuda_graph', 'n_gpus': world, 'tokens_per_rank': T, 'hidden': H,
                          'topk': K, 'experts': E, 'routing': 'skewed: N(0,1) logits + N(0,2) expert bias',
                          'dispatch': 'bf16 in, e4m3 + 1x128 scales on the wire (quantised in kernel)', 'results': results}))
    buffer.destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
