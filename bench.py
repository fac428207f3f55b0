"""Headline benchmark: expert-parallel dispatch/combine bandwidth per rank.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 5

Configuration (the one the reference publishes its numbers for): 16,384 tokens per rank, hidden 7168,
top-6 of 256 experts chosen from N(0,1) gating logits, expert alignment 128, no bias; dispatch in FP8 e4m3
with fp32 1x128 row-major scales, combine in BF16. One step = dispatch (issue + expand epilogue) followed by
combine (issue + reduce epilogue) through `deep_ep.EPBuffer`.

Accounting (same as the reference's test): bytes = rank-deduplicated tokens RECEIVED by a rank (its own
included) x logical bytes per source token (dispatch 7168 + 56*4 + 6*8 + 6*4 = 7464 B, combine 14336 B);
time = device time of the issue kernel with the arrival wait moved into it (`set_barrier_in_prologue(True)`),
i.e. issue + wire + completion, epilogue excluded. Times come from CUDA events, maximum over ranks.
The JSON `value` is the aggregate over all ranks (per-rank figure x N); `per_rank` holds the per-rank numbers.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PUBLISHED_DISPATCH_GBS = 375.0    # README of the reference, EP8, Ascend 950DT
PUBLISHED_COMBINE_GBS = 347.0


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument('--gpus', type=int, default=1)
    p.add_argument('--steps', type=int, default=50)
    p.add_argument('--warmup', type=int, default=5)
    p.add_argument('--impl', default='ours', choices=['ours', 'reference', 'nccl'])
    p.add_argument('--num-tokens', type=int, default=16384)
    p.add_argument('--hidden', type=int, default=7168)
    p.add_argument('--num-topk', type=int, default=6)
    p.add_argument('--num-experts', type=int, default=256)
    p.add_argument('--num-sms', type=int, default=0)
    p.add_argument('--dispatch-input', default='fp8', choices=['fp8', 'bf16-fused'],
                   help='fp8: tokens are quantised before the timed call (what the reference measures); '
                        'bf16-fused: BF16 tokens quantised inside the dispatch kernel')
    p.add_argument('--skip-e2e', action='store_true')
    p.add_argument('--skip-check', action='store_true')
    p.add_argument('--skip-nccl', action='store_true', help='do not measure the NCCL all_to_all_single anchor after the timed region')
    return p.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) from a background thread while
    the timed region runs."""

    REASONS = {'hw_slowdown': 0x8, 'sw_power_cap': 0x4, 'hw_thermal_slowdown': 0x40, 'sw_thermal_slowdown': 0x20}

    def __init__(self, device_index: int, interval_s: float = 0.01):
        import threading
        self.device_index, self.interval_s = device_index, interval_s
        self.samples, self.max_clock, self.error = [], None, None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _physical_index(self) -> int:
        visible = os.environ.get('CUDA_VISIBLE_DEVICES')
        if visible:
            ids = [v.strip() for v in visible.split(',') if v.strip()]
            if self.device_index < len(ids) and ids[self.device_index].isdigit():
                return int(ids[self.device_index])
        return self.device_index

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, 'nvmlDeviceGetCurrentClocksEventReasons', None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop.is_set():
                self.samples.append((time.time(), float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)),
                                     int(reasons_fn(handle))))
                time.sleep(self.interval_s)
        except Exception as e:       # NVML missing: the bench still runs, the record says why it has no clocks
            self.error = repr(e)

    def start(self):
        self._thread.start()

    def stop(self, t_begin: float = 0.0, t_end: float = float('inf')) -> dict:
        """Summarise the samples taken inside [t_begin, t_end] (the timed region)."""
        self._stop.set()
        self._thread.join(timeout=2)
        inside = [s for s in self.samples if t_begin <= s[0] <= t_end] or self.samples[-3:]
        reasons = sorted(name for name, bit in self.REASONS.items() if any(s[2] & bit for s in inside))
        out = {'sm_mhz': statistics.median(s[1] for s in inside) if inside else None, 'sm_max_mhz': self.max_clock,
               'reasons': reasons, 'samples': len(inside)}
        if self.error:
            out['error'] = self.error
        return out


def reference_arm(args):
    """The reference is Ascend C + CANN/HCCL: it has no CUDA path and cannot be installed or run on a B200 box."""
    why = 'reference needs Ascend CANN/Bisheng/torch_npu and Ascend 950 hardware; its pip install fails at `import torch_npu`'
    marker = os.path.join(ROOT, 'baseline', 'reference_install.txt')
    if os.path.exists(marker):
        with open(marker) as f:
            why = f.readline().strip() or why
    if int(os.environ.get('RANK', 0)) == 0:
        print(json.dumps({'impl': 'reference', 'unavailable': why}))


def measure_nccl(args, dev, world, rank, steps, warmup):
    """Baseline on the same box: dispatch/combine built from NCCL `all_to_all_single` (what a framework without
    this library would do), same configuration and byte accounting. Dispatch = permute + count exchange + payload
    exchanges; combine = exchange back + index-add reduction. Two times per phase, CUDA events, max over ranks:
    the whole operation (it contains the host read of the split sizes and the index kernels a framework needs) and
    the `all_to_all_single` calls alone (events around every collective, summed)."""
    import torch
    import torch.distributed as dist
    from deep_ep.utils.math import per_token_cast_to_fp8
    from deep_ep.utils.testing import L2Flusher
    torch.manual_seed(1234 + rank)
    T, H, K, E = args.num_tokens, args.hidden, args.num_topk, args.num_experts
    per_rank = E // world
    x = torch.randn(T, H, dtype=torch.bfloat16, device=dev)
    top_logits, topk_idx = torch.randn(T, E, device=dev).topk(K, dim=-1)
    topk_w = torch.softmax(top_logits, dim=-1).float()
    x_fp8, sf = per_token_cast_to_fp8(x)
    flusher = L2Flusher()
    wire = []           # (start, end) event pairs around the collectives of the current phase

    def a2a(out, inp, out_splits=None, in_splits=None):
        pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        pair[0].record()
        dist.all_to_all_single(out, inp, out_splits, in_splits)
        pair[1].record()
        wire.append(pair)

    def dispatch():
        dst = topk_idx // per_rank
        hit = torch.zeros(T, world, dtype=torch.bool, device=dev).scatter_(1, dst, True)
        order = hit.t().reshape(-1).nonzero(as_tuple=True)[0] % T            # tokens grouped by destination rank
        send_counts = hit.sum(0)
        recv_counts = torch.empty_like(send_counts)
        a2a(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        outs = []
        for t in (x_fp8.view(torch.uint8), sf, topk_idx, topk_w):
            out = torch.empty((sum(rc), t.size(1)), dtype=t.dtype, device=dev)
            a2a(out, t[order].contiguous(), rc, sc)
            outs.append(out)
        return outs, order, sc, rc

    def combine(y, order, sc, rc):
        back = torch.empty((sum(sc), H), dtype=torch.bfloat16, device=dev)
        a2a(back, y, sc, rc)
        return torch.zeros(T, H, dtype=torch.float32, device=dev).index_add_(0, order, back.float()).to(torch.bfloat16)

    outs, order, sc, rc = dispatch()
    num_recv = sum(rc)
    y = torch.randn(num_recv, H, dtype=torch.bfloat16, device=dev)
    for _ in range(max(warmup, 3)):
        o, order, sc, rc = dispatch()
        combine(y, order, sc, rc)
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    wires = []
    dist.barrier()
    torch.cuda.synchronize()
    for ev in events:
        flusher()
        wire = []
        ev[0].record()
        o, order, sc, rc = dispatch()
        ev[1].record()
        d_wire = wire
        flusher()
        wire = []
        ev[2].record()
        combine(y, order, sc, rc)
        ev[3].record()
        wires.append((d_wire, wire))
    torch.cuda.synchronize()
    d_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in events)
    c_ms = statistics.mean(e[2].elapsed_time(e[3]) for e in events)
    dw_ms = statistics.mean(sum(a.elapsed_time(b) for a, b in w[0]) for w in wires)
    cw_ms = statistics.mean(sum(a.elapsed_time(b) for a, b in w[1]) for w in wires)
    stats = torch.tensor([d_ms, c_ms, dw_ms, cw_ms, float(num_recv)], dtype=torch.float64, device=dev)
    gathered = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    g = torch.stack(gathered).cpu()
    d_ms, c_ms, dw_ms, cw_ms = (g[:, i].max().item() for i in range(4))
    d_bytes = g[:, 4] * (H + (H // 128) * 4 + K * 8 + K * 4)
    c_bytes = g[:, 4] * H * 2
    return {'dispatch_gbs': round(d_bytes.min().item() / (d_ms * 1e6), 2), 'combine_gbs': round(c_bytes.min().item() / (c_ms * 1e6), 2),
            'dispatch_ms': round(d_ms, 4), 'combine_ms': round(c_ms, 4),
            'collectives_only': {'dispatch_gbs': round(d_bytes.min().item() / (dw_ms * 1e6), 2),
                                 'combine_gbs': round(c_bytes.min().item() / (cw_ms * 1e6), 2),
                                 'dispatch_ms': round(dw_ms, 4), 'combine_ms': round(cw_ms, 4)},
            'aggregate_dispatch_gbs': round(d_bytes.sum().item() / (d_ms * 1e6), 2), 'steps': steps,
            'what': 'per-rank GB/s of NCCL all_to_all_single dispatch/combine, same shapes and byte accounting; the first '
                    'pair of figures is the whole operation (host read of split sizes, permutation and index-add kernels '
                    'included), `collectives_only` sums the device time of the all_to_all_single calls alone'}


def nccl_arm(args):
    """`--impl nccl`: only the NCCL baseline (see `measure_nccl`)."""
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29517')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    r = measure_nccl(args, dev, world, rank, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps({'impl': 'nccl', 'metric': 'EP dispatch GB/s with NCCL all_to_all_single (same accounting)',
                          'value': r['aggregate_dispatch_gbs'], 'unit': 'GB/s', 'n_gpus': world,
                          'steps': args.steps, 'warmup': max(args.warmup, 3), 'per_rank': r}))
    dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == 'reference':
        reference_arm(args)
        return
    if args.impl == 'nccl':
        nccl_arm(args)
        return

    import torch
    import torch.distributed as dist
    import deep_ep
    from deep_ep.utils.math import per_token_cast_to_fp8
    from deep_ep.utils.testing import L2Flusher

    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    assert world == args.gpus, f'launched with WORLD_SIZE={world} but --gpus {args.gpus}'
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29517')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    group = dist.group.WORLD
    torch.manual_seed(1234 + rank)

    T, H, K, E = args.num_tokens, args.hidden, args.num_topk, args.num_experts
    align = 128
    buffer = deep_ep.EPBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=False,
                              explicitly_destroy=True)
    # the published figures use the whole chip for communication; so does this benchmark unless told otherwise
    num_sms = args.num_sms or min(128, deep_ep._C.get_num_device_sms())

    # synthetic inputs, generated on the host in pinned memory (the end-to-end arm copies them every step); the process
    # first moves to the CPUs next to its GPU so that those buffers are local to the GPU's PCIe root
    from deep_ep.utils.envs import bind_to_device_numa_node
    numa_node = bind_to_device_numa_node(local_rank)
    x_host = torch.randn(T, H, dtype=torch.bfloat16).pin_memory()
    logits_host = torch.randn(T, E)
    top_logits, topk_idx_host = logits_host.topk(K, dim=-1)
    topk_w_host = torch.softmax(top_logits, dim=-1).float().pin_memory()
    topk_idx_host = topk_idx_host.long().pin_memory()
    x = x_host.to(dev)
    topk_idx, topk_w = topk_idx_host.to(dev), topk_w_host.to(dev)
    x_fp8, sf = per_token_cast_to_fp8(x)
    sf_packs = sf.view(torch.int16)

    def dispatch_input():
        return x if args.dispatch_input == 'bf16-fused' else (x_fp8, sf_packs)

    common = dict(num_experts=E, num_max_tokens_per_rank=T, expert_alignment=align, num_sms=num_sms,
                  async_with_compute_stream=True, do_expand=True, do_zero_padding=True, defer_epilogue=True)
    fused = args.dispatch_input == 'bf16-fused'
    flusher = L2Flusher()
    deep_ep._C.set_barrier_in_prologue(True)

    # one untimed pass to size things and to build the combine input
    ev = buffer.dispatch(dispatch_input(), topk_idx=topk_idx, topk_weights=topk_w, fused_fp8_quant=fused, **common)
    (recv_x, recv_sf), _, recv_w, handle = ev.current_stream_wait()
    num_recv = int(handle.psum_num_recv_tokens_per_rank[-1])
    dispatch_bytes = num_recv * (H + (H // 128) * 4 + K * 8 + K * 4)
    combine_bytes = num_recv * H * 2
    # bytes the two epilogues move through HBM (read + write), for their own GB/s figures
    num_rows = int(handle.num_unaligned_recv_tokens_per_expert.sum())
    msg_bytes = H + (H // 128) * 4 + K * 8 + 16
    expand_bytes = num_recv * msg_bytes + num_rows * (H + (H // 128) * 4 + 4) + (recv_x.size(0) - num_rows) * H
    num_partials = int((torch.zeros(T, world, dtype=torch.bool, device=dev).scatter_(1, topk_idx // (E // world), True)).sum())
    reduce_bytes = (num_partials + T) * H * 2

    # Combine input: a deterministic function of (global source token, top-k position), so that every rank can compute
    # the expected result of ITS tokens without communication (the pattern of the reference's test). It is also the
    # input of the timed loop: the combine that is timed is the combine that is checked.
    from deep_ep.utils import refs
    meta = handle.recv_src_metadata[:num_recv]
    y = torch.zeros(recv_x.size(0) + 1, H, dtype=torch.bfloat16, device=dev)
    if not args.skip_check:
        for lo in range(0, num_recv, 4096):            # chunks bound the fp32 temporaries of the generator
            part = refs.generate_pre_combine_data(meta[lo:lo + 4096, -2], T, K, H, world)
            y[meta[lo:lo + 4096, :-2].long().flatten()] = part.view(-1, H)
            del part
    else:
        y.normal_()
    y = y[:-1]

    checks = {}
    if not args.skip_check:      # the timed path must produce what the oracle produces: payload, scales, weights, order
        ref_x, ref_idx, ref_w, ref_src, _ = refs.dispatch((x_fp8.view(torch.uint8), sf_packs), topk_idx, topk_w, T, E)
        valid = meta[:, :-2] >= 0
        flat = meta[:, :-2][valid].long()
        assert torch.equal(meta[:, -2], ref_src) and torch.equal(valid, ref_idx >= 0)
        assert torch.equal(recv_x.view(torch.uint8)[flat], ref_x[0].unsqueeze(1).expand(-1, K, -1)[valid])
        assert torch.equal(recv_sf.view(torch.int16)[flat], ref_x[1].unsqueeze(1).expand(-1, K, -1)[valid])
        assert torch.equal(recv_w[flat], ref_w[valid])
        checks['dispatch'] = 'payload, scales, weights and row order bitwise equal to the all_to_all oracle'
        del ref_x, ref_idx, ref_w, ref_src, valid, flat

    def step(events=None):
        # Before each timed phase: the L2 flush keeps the device busy while the host queues the next launches, then a
        # device-side barrier over the ranks lines them up, so that a phase time does not contain the other ranks' launch
        # skew (the reference's test does the same before every sample: device-busy op + cross-rank barrier,
        # `deep_ep/utils/testing.py:347-371` there). Both are inside `ms_per_step`.
        flusher()
        buffer.barrier(wait_comm_stream=False)
        if events is not None:
            events[0].record()
        ev_d = buffer.dispatch(dispatch_input(), topk_idx=topk_idx, topk_weights=topk_w, fused_fp8_quant=fused, **common)
        if events is not None:
            events[1].record()
        _, _, w_out, h = ev_d.current_stream_wait()
        if events is not None:
            events[2].record()
        flusher()
        buffer.barrier(wait_comm_stream=False)
        if events is not None:
            events[3].record()
        ev_c = buffer.combine(y, h, topk_weights=w_out, num_sms=num_sms, async_with_compute_stream=True, defer_epilogue=True)
        if events is not None:
            events[4].record()
        out = ev_c.current_stream_wait()
        if events is not None:
            events[5].record()
        return out

    sampler = ClockSampler(local_rank)
    sampler.start()                      # nvidia-smi needs a moment to start: launch it before the warm-up
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    events = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(args.steps)]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    t_begin = time.time()
    start.record()
    for i in range(args.steps):
        combined, combined_w = step(events[i])
    end.record()
    torch.cuda.synchronize()
    t_end = time.time()
    dist.barrier()
    clocks = sampler.stop(t_begin, t_end)
    total_ms = start.elapsed_time(end)
    dispatch_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in events)
    combine_ms = statistics.mean(e[3].elapsed_time(e[4]) for e in events)
    expand_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in events)      # host count wait + expand kernel
    reduce_ms = statistics.mean(e[4].elapsed_time(e[5]) for e in events)

    if not args.skip_check:      # the combine of the LAST TIMED step against the strict-order oracle, bitwise
        ref_y = torch.empty(T, K, H, dtype=torch.bfloat16, device=dev)
        for lo in range(0, T, 4096):
            tokens = rank * T + torch.arange(lo, min(lo + 4096, T), device=dev)
            ref_y[lo:lo + 4096] = refs.generate_pre_combine_data(tokens, T, K, H, world)
        ref_combined = refs.combine(ref_y, topk_idx, E, None, True, world)
        assert torch.equal(combined, ref_combined), 'timed combine differs from the oracle'
        assert torch.equal(combined_w, topk_w), 'combined top-k weights differ from the inputs'
        checks['combine'] = 'output of the last timed step bitwise equal to the fp32 strict-order oracle; weights round-trip exactly'
        del ref_y, ref_combined

    # ---- end to end through the public API: H2D of the step's inputs, dispatch + combine, D2H of the result
    e2e = {}
    h2d_bytes = 0
    e2e_error = None
    if not args.skip_e2e:
        deep_ep._C.set_barrier_in_prologue(False)
        # Input pipeline as a training or serving loop would run it: two device-side input sets; the copy of step i + 1
        # (pinned host memory -> device, on a copy stream) overlaps the kernels of step i, and the copy of step i's result
        # (device -> pinned host memory, on a second copy stream) overlaps the kernels of step i + 1. Every step's input
        # copy and every step's result copy happen inside the timed region; the host has every result when the clock stops.
        # The activations cross PCIe in the form the dispatch takes them: e4m3 rows plus their 1x128 scales (the headline
        # configuration), or bf16 rows that the dispatch kernel quantises itself (`--dispatch-input bf16-fused`).
        if fused:
            host_inputs = (x_host, topk_idx_host, topk_w_host)
        else:
            host_inputs = (x_fp8.view(torch.uint8).cpu().pin_memory(), sf_packs.cpu().pin_memory(), topk_idx_host, topk_w_host)
        dev_inputs = [tuple(torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_inputs) for _ in range(2)]
        h2d_bytes = sum(t.nbytes for t in host_inputs)
        metric_host = torch.empty(2, dtype=torch.float32).pin_memory()
        full_host = [(torch.empty(T, H, dtype=torch.bfloat16).pin_memory(), torch.empty(T, K, dtype=torch.float32).pin_memory())
                     for _ in range(2)]
        copy_stream, back_stream = torch.cuda.Stream(), torch.cuda.Stream()
        copy_done = [torch.cuda.Event() for _ in range(2)]
        inputs_free = [torch.cuda.Event() for _ in range(2)]
        back_done = [torch.cuda.Event() for _ in range(2)]

        def issue_copy(i):
            b = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(inputs_free[b])          # the step that last read this set has finished
                for dst, src in zip(dev_inputs[b], host_inputs):
                    dst.copy_(src, non_blocking=True)
                copy_done[b].record(copy_stream)

        def e2e_loop(steps, full_result):
            issue_copy(0)
            for i in range(steps):
                b = i % 2
                *x_dev, idx_dev, w_dev = dev_inputs[b]
                x_dev = x_dev[0] if fused else (x_dev[0].view(torch.float8_e4m3fn), x_dev[1])
                torch.cuda.current_stream().wait_event(copy_done[b])
                if i + 1 < steps:
                    issue_copy(i + 1)
                ev_d = buffer.dispatch(x_dev, topk_idx=idx_dev, topk_weights=w_dev, fused_fp8_quant=fused, **common)
                (rx, rsf), _, w_out, h = ev_d.current_stream_wait()
                ev_c = buffer.combine(y[:rx.size(0)], h, topk_weights=w_out, num_sms=num_sms, async_with_compute_stream=True,
                                      defer_epilogue=True)
                out, out_w = ev_c.current_stream_wait()
                inputs_free[b].record()
                if full_result:
                    # the whole combined tensor and its weights go to the host; the host waits for the copy of the step
                    # before this one (the set of pinned buffers it is about to reuse) while this step's copy runs
                    produced = torch.cuda.Event()
                    produced.record()
                    if i >= 2:
                        back_done[b].synchronize()
                    with torch.cuda.stream(back_stream):
                        back_stream.wait_event(produced)
                        full_host[b][0].copy_(out, non_blocking=True)
                        full_host[b][1].copy_(out_w, non_blocking=True)
                        back_done[b].record(back_stream)
                    out.record_stream(back_stream), out_w.record_stream(back_stream)
                else:
                    metric = torch.stack([out[:, :8].float().sum(), out_w.sum()])
                    metric_host.copy_(metric, non_blocking=True)
                    torch.cuda.current_stream().synchronize()      # the step's metric is on the host
            torch.cuda.synchronize()                               # every result is on the host

        for name, full_result, nbytes in (('full', True, full_host[0][0].nbytes + full_host[0][1].nbytes),
                                          ('metric', False, metric_host.nbytes)):
            try:
                e2e_loop(3, full_result)
            except (TypeError, ValueError, AssertionError, RuntimeError) as exc:
                # a host-side argument error is the same on every rank: report it instead of losing the device-timed numbers
                e2e_error = f'{type(exc).__name__}: {exc}'[:300]
                break
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e2e_loop(args.steps, full_result)
            e2e[name] = ((time.perf_counter() - t0) * 1e3 / args.steps, nbytes)
        if 'full' in e2e and not args.skip_check:
            last = (args.steps - 1) % 2
            assert torch.equal(full_host[last][0], combined.cpu()), 'end-to-end result on the host differs from the timed result'
            checks['e2e'] = 'combined tensor read back on the host equals the device-timed result bitwise'

    # ---- same-box anchor: NCCL all_to_all_single dispatch/combine in this process, after the timed regions
    nccl = None
    if not args.skip_nccl:
        del y
        torch.cuda.empty_cache()
        nccl = measure_nccl(args, dev, world, rank, min(args.steps, 10), 3)

    # ---- reduce over ranks: maximum time, sum of bytes
    stats = torch.tensor([total_ms, dispatch_ms, combine_ms, e2e.get('full', (0.0, 0))[0], float(dispatch_bytes), float(combine_bytes),
                          expand_ms, reduce_ms, float(expand_bytes), float(reduce_bytes), e2e.get('metric', (0.0, 0))[0]],
                         dtype=torch.float64, device=dev)
    gathered = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    g = torch.stack(gathered).cpu()
    total_ms, dispatch_ms, combine_ms, e2e_ms_max = (g[:, i].max().item() for i in range(4))
    expand_ms, reduce_ms, e2e_metric_ms_max = g[:, 6].max().item(), g[:, 7].max().item(), g[:, 10].max().item()
    sum_dispatch_bytes, sum_combine_bytes = g[:, 4].sum().item(), g[:, 5].sum().item()
    ms_per_step = total_ms / args.steps
    dispatch_gbs_rank = [g[r, 4].item() / (dispatch_ms * 1e6) for r in range(world)]
    combine_gbs_rank = [g[r, 5].item() / (combine_ms * 1e6) for r in range(world)]
    dispatch_gbs_agg = sum_dispatch_bytes / (dispatch_ms * 1e6)
    combine_gbs_agg = sum_combine_bytes / (combine_ms * 1e6)

    if rank == 0:
        link_share = (world - 1) / world          # share of the received bytes that crossed NVLink (uniform routing)
        line = {
            'metric': 'EP dispatch GB/s (FP8 e4m3 + 1x128 fp32 scales, h7168, top-6/256, 16384 tokens/rank), aggregate over ranks; '
                      'combine (BF16) reported alongside',
            'value': round(dispatch_gbs_agg, 2), 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': round(ms_per_step, 4), 'higher_is_better': True,
            'scaling': 'weak',
            # the published figure is a per-rank EP8 NVLink-class number: with one GPU nothing crosses a link, so no ratio
            'vs_baseline': round(min(dispatch_gbs_rank) / PUBLISHED_DISPATCH_GBS, 4) if world >= 2 else None,
            'dtype': 'fp8_e4m3 dispatch / bf16 combine (the precisions of the published figures)', 'data': 'synthetic',
            'impl': 'ours',
            'config': {'model': 'DeepSeek-V3-style MoE routing: hidden 7168, 256 experts, top-6, expert alignment 128',
                       'global_batch': T * world, 'seq_len': None, 'tokens_per_rank': T, 'parallelism': f'ep{world}',
                       'dispatch_input': args.dispatch_input, 'num_sms': num_sms,
                       'l2': 'a 256 MiB buffer is overwritten and the ranks meet in a device-side barrier before dispatch and before '
                             'combine in every step (inside ms_per_step, outside the per-phase events)',
                       'timing': 'phase times: CUDA events around the issue kernel with the arrival wait inside it; max over ranks',
                       'vs_baseline_def': 'min per-rank dispatch GB/s / 375 GB/s (published EP8 per-rank figure); null on one GPU, '
                                          'where every message is a local copy'},
            'per_rank': {'dispatch_gbs': round(min(dispatch_gbs_rank), 2), 'combine_gbs': round(min(combine_gbs_rank), 2),
                         'dispatch_ms': round(dispatch_ms, 4), 'combine_ms': round(combine_ms, 4),
                         'recv_tokens': num_recv, 'combine_vs_published': round(min(combine_gbs_rank) / PUBLISHED_COMBINE_GBS, 4),
                         'nvlink_gbs_per_direction': {'dispatch': round(min(dispatch_gbs_rank) * link_share, 2),
                                                      'combine': round(min(combine_gbs_rank) * link_share, 2)},
                         # issue kernel + epilogue, as the reference's test prints both the transport and the epilogue figures
                         'dispatch_with_expand_ms': round(dispatch_ms + expand_ms, 4),
                         'combine_with_reduce_ms': round(combine_ms + reduce_ms, 4),
                         'dispatch_with_expand_gbs': round(min(g[:, 4]).item() / ((dispatch_ms + expand_ms) * 1e6), 2),
                         'combine_with_reduce_gbs': round(min(g[:, 5]).item() / ((combine_ms + reduce_ms) * 1e6), 2),
                         'expand_epilogue': {'ms': round(expand_ms, 4), 'hbm_gbs': round(g[:, 8].min().item() / (expand_ms * 1e6), 1),
                                             'what': 'host count wait + expand kernel; bytes = messages read + rows, scales, weights and padding written'},
                         'reduce_epilogue': {'ms': round(reduce_ms, 4), 'hbm_gbs': round(g[:, 9].min().item() / (reduce_ms * 1e6), 1),
                                             'what': 'reduce kernel; bytes = partials read + combined rows written'}},
            'combine': {'value': round(combine_gbs_agg, 2), 'unit': 'GB/s'},
            'checks': checks,
            'clocks': clocks,
            'gpu_launches': 6 * args.steps,        # dispatch, expand, combine, reduce + two rank-barrier kernels per step
        }
        if nccl is not None:
            line['nccl_baseline'] = nccl
        if 'full' in e2e:
            step_bytes = sum_dispatch_bytes + sum_combine_bytes
            line['e2e'] = {'value': round(sum_dispatch_bytes / (e2e_ms_max * 1e6), 2),
                           'unit': 'GB/s of dispatch bytes over the whole end-to-end step (H2D + dispatch + expand + combine + reduce + D2H)',
                           'h2d_inputs': 'bf16 rows, quantised by the dispatch kernel' if fused else 'e4m3 rows + 1x128 fp32 scales (what the dispatch sends)',
                           'd2h_result': 'the whole combined bf16 tensor and the combined top-k weights, into pinned host memory',
                           'step_ms': round(e2e_ms_max, 4), 'step_gbs_dispatch_plus_combine': round(step_bytes / (e2e_ms_max * 1e6), 2),
                           'h2d_bytes_per_step': h2d_bytes, 'd2h_bytes_per_step': e2e['full'][1],
                           'input_pipeline': 'pinned host buffers on the NUMA node of the GPU (node %s of rank 0); the copy of step i + 1 '
                                             'and the read-back of step i - 1 overlap the kernels of step i' % numa_node}
            if 'metric' in e2e:
                line['e2e']['metric_only'] = {'value': round(sum_dispatch_bytes / (e2e_metric_ms_max * 1e6), 2),
                                              'step_ms': round(e2e_metric_ms_max, 4), 'd2h_bytes_per_step': e2e['metric'][1],
                                              'what': 'same loop, but only two reduced scalars (a checksum of the result) are read '
                                                      'back each step, with a host synchronisation per step'}
        elif not args.skip_e2e and e2e_error is not None:
            line['e2e_error'] = e2e_error
        print(json.dumps(line))
    buffer.destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
