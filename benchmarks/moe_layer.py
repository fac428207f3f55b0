"""MoE layer forward+backward: this library (EPBuffer dispatch/combine + tcgen05 grouped GEMMs) against the
conventional NCCL `all_to_all_single` + per-expert library-GEMM layer, same shapes, same box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/moe_layer.py

DeepSeek-V3-like expert FFN: 4096 tokens per rank, hidden 7168, intermediate 2048, SwiGLU, 256 routed experts,
top-8, one shared expert; random-init weights ~ N(0, 0.02), BF16 compute with fp32 weight-gradient accumulation.
A step is forward + backward of the layer (no optimizer: the layer is a communication+GEMM benchmark).
Times are CUDA events per step, maximum over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.distributed.nn.functional as dist_fn
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import deep_ep  # noqa: E402
from deep_ep.models.moe_layer import MoEConfig, MoELayer  # noqa: E402


class BaselineMoELayer(nn.Module):
    """Permute by expert, `all_to_all_single` the (token, expert) copies, per-expert `F.linear`, exchange back, weighted sum."""

    def __init__(self, ours: MoELayer, use_grouped_mm: bool = False):
        super().__init__()
        # expert GEMMs: one cuBLAS call per expert (default) or the library's grouped GEMM, `F.grouped_mm`, one per layer
        self.use_grouped_mm = use_grouped_mm
        self.group, self.config = ours.group, ours.config
        self.world = ours.num_ranks
        self.num_local_experts = ours.num_local_experts
        self.gate = ours.gate
        self.w_gate_up = nn.Parameter(ours.w_gate_up.detach().clone())
        self.w_down = nn.Parameter(ours.w_down.detach().clone())
        self.shared_gate_up = nn.Parameter(ours.shared_gate_up.detach().clone()) if ours.config.num_shared_experts else None
        self.shared_down = nn.Parameter(ours.shared_down.detach().clone()) if ours.config.num_shared_experts else None

    def route(self, x):
        # library GEMM (cuBLAS) for the router of the baseline, same arithmetic as the layer's own kernel
        # the operands of the layer's own kernel (bf16 activations, gate matrix rounded to bf16) in an fp32 library GEMM
        logits = F.linear(x.float(), self.gate.to(torch.bfloat16).float())
        topk_weights, topk_idx = torch.softmax(logits, dim=-1).topk(self.config.num_topk, dim=-1)
        return topk_idx, topk_weights / topk_weights.sum(dim=-1, keepdim=True)

    def forward(self, x):
        cfg = self.config
        topk_idx, topk_w = self.route(x)
        t, k = topk_idx.shape
        flat_expert = topk_idx.reshape(-1)
        order = torch.argsort(flat_expert, stable=True)                      # (token, slot) pairs grouped by expert
        send = x[order // k]
        per_expert = torch.bincount(flat_expert, minlength=cfg.num_experts)
        send_counts = per_expert.view(self.world, self.num_local_experts).sum(1)
        recv_per_expert = torch.empty_like(per_expert)
        dist.all_to_all_single(recv_per_expert, per_expert, group=self.group)   # [src rank, local expert]
        recv_counts = recv_per_expert.view(self.world, self.num_local_experts).sum(1)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv = dist_fn.all_to_all_single(torch.empty((sum(rc), x.size(1)), dtype=x.dtype, device=x.device), send, rc, sc,
                                         group=self.group)
        # received rows are (src rank, local expert) ordered: regroup by local expert
        counts = recv_per_expert.view(self.world, self.num_local_experts)
        expert_of_row = torch.repeat_interleave(torch.arange(self.num_local_experts, device=x.device).repeat(self.world),
                                                counts.reshape(-1))
        by_expert = torch.argsort(expert_of_row, stable=True)
        rows = recv[by_expert]
        if self.use_grouped_mm:
            offs = counts.sum(0).cumsum(0).int()
            g, u = F.grouped_mm(rows, self.w_gate_up.transpose(-2, -1), offs=offs).chunk(2, dim=-1)
            out = F.grouped_mm(F.silu(g) * u, self.w_down.transpose(-2, -1), offs=offs)
            return self._finish(x, out, by_expert, sc, rc, topk_w, order, k)
        outs, start = [], 0
        # unbind once: indexing the stacked parameter per expert would make autograd materialise a full-size
        # gradient of all experts for every expert
        w1s, w2s = self.w_gate_up.unbind(0), self.w_down.unbind(0)
        for e, c in enumerate(counts.sum(0).tolist()):
            if c:
                g, u = F.linear(rows[start:start + c], w1s[e]).chunk(2, dim=-1)
                outs.append(F.linear(F.silu(g) * u, w2s[e]))
            start += c
        out = torch.cat(outs) if outs else torch.empty_like(rows)
        return self._finish(x, out, by_expert, sc, rc, topk_w, order, k)

    def _finish(self, x, out, by_expert, sc, rc, topk_w, order, k):
        back_rows = torch.empty_like(out)
        back_rows[by_expert] = out
        back = dist_fn.all_to_all_single(torch.empty((sum(sc), x.size(1)), dtype=x.dtype, device=x.device), back_rows, sc, rc,
                                         group=self.group)
        weighted = back * topk_w.reshape(-1)[order].unsqueeze(1).to(back.dtype)
        y = torch.zeros_like(x).index_add_(0, order // k, weighted)
        if self.shared_gate_up is not None:
            g, u = F.linear(x, self.shared_gate_up).chunk(2, dim=-1)
            y = y + F.linear(F.silu(g) * u, self.shared_down)
        return y


def time_layer(layer, x, steps, warmup, accumulate_into=None):
    """Forward + backward per step. Gradients are dropped after every step (`zero_grad(set_to_none=True)` of a training
    loop), for both layers alike: otherwise every step after the first would also pay an elementwise accumulation pass
    over all expert weight gradients, which belongs to neither layer."""
    grad = torch.randn_like(x)
    params = list(layer.parameters())

    def step():
        layer(x).backward(grad)
        if accumulate_into is not None:
            # a layer whose weight-gradient GEMMs cannot add into fp32 buffers themselves does it in a pass of its own
            for p, main_grad in accumulate_into:
                main_grad.add_(p.grad)
        for p in params:
            p.grad = None
        x.grad = None

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in ev) / steps
    t = torch.tensor([ms], device=x.device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def time_forward(fn, x, steps, warmup):
    """Inference forward only (no autograd), device-timed, maximum over ranks."""
    with torch.no_grad():
        for _ in range(warmup):
            fn(x)
        torch.cuda.synchronize()
        dist.barrier()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in ev:
            a.record()
            fn(x)
            b.record()
        torch.cuda.synchronize()
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev) / steps], device=x.device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--num-tokens', type=int, default=4096)
    p.add_argument('--hidden', type=int, default=7168)
    p.add_argument('--intermediate', type=int, default=2048)
    p.add_argument('--num-experts', type=int, default=256)
    p.add_argument('--num-topk', type=int, default=8)
    p.add_argument('--steps', type=int, default=10)
    p.add_argument('--warmup', type=int, default=3)
    p.add_argument('--skip-baseline', action='store_true')
    p.add_argument('--baseline-grouped-mm', action='store_true',
                   help='baseline expert GEMMs through torch.nn.functional.grouped_mm instead of one cuBLAS call per expert')
    p.add_argument('--baseline-both', action='store_true', help='time both baselines (per-expert loop and F.grouped_mm)')
    p.add_argument('--overlap-shared-expert', action='store_true', help='run the shared expert on a side stream')
    p.add_argument('--fuse-combine', action='store_true',
                   help='let the second expert GEMM store single-row tokens straight into the combine landing slots of their owners')
    p.add_argument('--fp8-training', action='store_true',
                   help='also time forward + backward with the routed experts\' forward and data-gradient GEMMs in FP8 '
                        '(power-of-two block scales applied by the tensor core; weight gradients stay bf16)')
    p.add_argument('--main-grad', action='store_true',
                   help='expert weight gradients accumulate in persistent fp32 `main_grad` buffers (read-modify-write in the '
                        'weight-gradient kernel) instead of being stored once in bf16')
    p.add_argument('--decode-graph', type=int, default=0, metavar='TOKENS',
                   help='also time a decode-sized inference forward (this many tokens per rank, FP8 with power-of-two scales, '
                        'no host synchronisation) launched eagerly and replayed as ONE CUDA graph of the whole layer')
    p.add_argument('--kernel-breakdown', action='store_true',
                   help='print the device time of every kernel of one forward + backward step of our layer (activity records)')
    p.add_argument('--forward-fp8', action='store_true',
                   help='also time the inference forward: BF16 path against the FP8 path (e4m3 dispatch + block-scaled FP8 GEMMs)')
    args = p.parse_args()
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    local_rank = int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29551')
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(7 + rank)
    cfg = MoEConfig(hidden=args.hidden, intermediate=args.intermediate, num_experts=args.num_experts, num_topk=args.num_topk,
                    num_shared_experts=1, num_max_tokens_per_rank=args.num_tokens, expert_alignment=128,
                    fuse_combine=args.fuse_combine, overlap_shared_expert=args.overlap_shared_expert)
    ours = MoELayer(dist.group.WORLD, cfg, device=dev)
    x = torch.randn(args.num_tokens, args.hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)

    result = {'bench': 'moe_layer_fwd_bwd', 'n_gpus': world, 'tokens_per_rank': args.num_tokens, 'hidden': args.hidden,
              'intermediate': args.intermediate, 'experts': args.num_experts, 'topk': args.num_topk, 'dtype': 'bf16', 'fuse_combine': args.fuse_combine}
    if not args.skip_baseline:
        kinds = [False, True] if args.baseline_both else [args.baseline_grouped_mm]
        for use_grouped_mm in kinds:
            name = 'F.grouped_mm' if use_grouped_mm else 'per-expert F.linear'
            key = 'baseline_grouped_mm_ms' if use_grouped_mm else 'baseline_loop_ms'
            base = BaselineMoELayer(ours, use_grouped_mm=use_grouped_mm).to(dev)
            with torch.no_grad():                      # same function, different plumbing: outputs must agree
                y_ours, y_base = ours(x), base(x)
            rel = ((y_ours.float() - y_base.float()).norm() / y_base.float().norm()).item()
            result['rel_diff_vs_baseline'] = round(rel, 5)
            accumulate = None
            if args.main_grad:        # same work as our layer: expert weight gradients end up added into fp32 buffers
                accumulate = [(w, torch.zeros(w.shape, dtype=torch.float32, device=dev)) for w in (base.w_gate_up, base.w_down)]
                result['baseline_wgrad'] = 'bf16 gradients, then one fp32 accumulation pass per step (main_grad += grad)'
            result[key] = round(time_layer(base, x, args.steps, args.warmup, accumulate), 3)
            del accumulate
            result['baseline_gemm'], result['baseline_ms'] = name, result[key]       # the last (strongest) one
            del base
            torch.cuda.empty_cache()
    if args.main_grad:
        for w in (ours.w_gate_up, ours.w_down):
            w.main_grad = torch.zeros(w.shape, dtype=torch.float32, device=dev)
        result['wgrad'] = 'fp32 accumulation into main_grad'
    result['ours_ms'] = round(time_layer(ours, x, args.steps, args.warmup), 3)
    # useful FLOPs: 3 GEMMs (gate, up, down) x (fwd + dgrad + wgrad) over routed + shared expert rows
    rows = args.num_tokens * (args.num_topk + 1)
    flops = 3 * 2 * rows * args.hidden * args.intermediate * 3
    result['ours_tflops_per_gpu'] = round(flops / (result['ours_ms'] * 1e-3) / 1e12, 1)
    result['tokens_per_s_total'] = round(args.num_tokens * world / (result['ours_ms'] * 1e-3))
    if args.fp8_training:
        assert args.hidden % 512 == 0 and args.intermediate % 512 == 0
        x.grad = None
        ours(x).backward(torch.ones_like(x))
        gx16 = x.grad.clone()
        ours.config.fp8_training = True
        x.grad = None
        ours(x).backward(torch.ones_like(x))
        result['fp8_training_dx_rel_diff_vs_bf16'] = round(((x.grad.float() - gx16.float()).norm() / gx16.float().norm()).item(), 5)
        for p_ in ours.parameters():
            p_.grad = None
        result['ours_fp8_training_ms'] = round(time_layer(ours, x, args.steps, args.warmup), 3)
        ours.config.fp8_training = False
        ours._fp8_cache = None
        torch.cuda.empty_cache()
    if args.kernel_breakdown:
        from deep_ep.utils.testing import bench_kineto
        g = torch.randn_like(x)

        def one_step():
            ours(x).backward(g)
            for p_ in ours.parameters():
                p_.grad = None
            x.grad = None
        ours.config.fp8_training = args.fp8_training
        profiles = bench_kineto(one_step, return_all_kernels=True, num_warmups=2, num_tests=3, flush_l2=False)
        ours.config.fp8_training = False
        top = sorted(profiles.values(), key=lambda k: -k.dur_ns * k.num_calls)[:24]
        result['kernel_breakdown_us'] = [[k.name[:70], k.num_calls, round(k.dur_us, 1)] for k in top]
    if args.forward_fp8:
        ours.quantize_weights()
        with torch.no_grad():
            y16, y8 = ours(x), ours.forward_fp8(x)
        result['fp8_forward_rel_diff_vs_bf16'] = round(((y8.float() - y16.float()).norm() / y16.float().norm()).item(), 5)
        result['forward_bf16_ms'] = round(time_forward(ours, x, args.steps, args.warmup), 3)
        result['forward_fp8_ms'] = round(time_forward(ours.forward_fp8, x, args.steps, args.warmup), 3)
        if args.hidden % 512 == 0 and args.intermediate % 512 == 0:
            # power-of-two scales: quantised that way by the dispatch kernel, applied by the tensor core in the GEMMs
            ours.config.fp8_scales = 'ue8m0'
            ours.quantize_weights()
            with torch.no_grad():
                y8h = ours.forward_fp8(x)
            result['fp8_ue8m0_forward_rel_diff_vs_bf16'] = round(((y8h.float() - y16.float()).norm() / y16.float().norm()).item(), 5)
            result['forward_fp8_ue8m0_ms'] = round(time_forward(ours.forward_fp8, x, args.steps, args.warmup), 3)
    if args.decode_graph > 0:
        # decode: route -> FP8 dispatch -> FP8 expert GEMMs -> combine (+ shared expert) without touching the host, so the
        # whole layer is one CUDA graph; the weights are shared with the layer above, only the buffer is decode-sized
        assert args.hidden % 512 == 0 and args.intermediate % 512 == 0
        tokens = args.decode_graph
        dcfg = MoEConfig(hidden=args.hidden, intermediate=args.intermediate, num_experts=args.num_experts, num_topk=args.num_topk,
                         num_shared_experts=1, num_max_tokens_per_rank=tokens, expert_alignment=128, fp8_scales='ue8m0',
                         host_sync=False)
        ours.config.fp8_scales = 'ue8m0'
        ours.quantize_weights()
        decode_buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=tokens, hidden=args.hidden,
                                         num_topk=args.num_topk, explicitly_destroy=True)
        saved = ours.config, ours.buffer
        ours.config, ours.buffer = dcfg, decode_buffer
        xd = torch.randn(tokens, args.hidden, device=dev, dtype=torch.bfloat16)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(3):
                y_eager = ours.forward_fp8(xd)
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                y_graph = ours.forward_fp8(xd)
        torch.cuda.synchronize()
        dist.barrier()

        def timed(fn):
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps + 3)]
            for a, b in ev:
                a.record()
                fn()
                b.record()
            torch.cuda.synchronize()
            t = torch.tensor([sum(a.elapsed_time(b) for a, b in ev[3:]) / args.steps], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return round(t.item() * 1e3, 1)
        result['decode_tokens_per_rank'] = tokens
        result['decode_forward_fp8_eager_us'] = timed(lambda: ours.forward_fp8(xd))
        result['decode_forward_fp8_one_graph_us'] = timed(graph.replay)
        decode_buffer.runtime.check_status()
        result['decode_graph_matches_eager'] = bool(torch.equal(y_graph, y_eager))
        ours.config, ours.buffer = saved
        ours.config.fp8_scales, ours._w1_fp8 = 'fp32', None         # the next section quantises for itself
        decode_buffer.destroy()
    if 'baseline_ms' in result:
        result['speedup'] = round(result['baseline_ms'] / result['ours_ms'], 3)
        if 'ours_fp8_training_ms' in result:
            result['speedup_fp8_training'] = round(result['baseline_ms'] / result['ours_fp8_training_ms'], 3)
    if 'ours_fp8_training_ms' in result:
        result['fp8_training_tflops_per_gpu'] = round(flops / (result['ours_fp8_training_ms'] * 1e-3) / 1e12, 1)
    if rank == 0:
        print(json.dumps(result))
    ours.destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
