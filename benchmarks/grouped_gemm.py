"""Throughput of the tcgen05 grouped GEMM kernels against the per-expert library-GEMM loop (single GPU).

    python benchmarks/grouped_gemm.py [--experts 32 --rows 1024 --hidden 7168 --inter 2048]

Shapes follow one rank of an EP8 DeepSeek-V3-like layer: 32 local experts, about 1024 rows each, GEMM1
[rows, 7168] x [4096, 7168]^T and GEMM2 [rows, 2048] x [7168, 2048]^T. Inputs exceed the 126 MB L2. Times are
CUDA events after warm-up; fractions are relative to the measured cuBLAS BF16 burst peak in MEASURED_PEAKS.json.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from deep_ep.ops import grouped_gemm as gg  # noqa: E402


def bench(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return min(a.elapsed_time(b) for a, b in ev), sum(a.elapsed_time(b) for a, b in ev) / iters


def main():
    p = argparse.ArgumentParser()
    p.add_argument('--experts', type=int, default=32)
    p.add_argument('--rows', type=int, default=1024)
    p.add_argument('--hidden', type=int, default=7168)
    p.add_argument('--inter', type=int, default=2048)
    p.add_argument('--iters', type=int, default=10)
    p.add_argument('--skip-torch', action='store_true')
    p.add_argument('--skip-fp8', action='store_true')
    p.add_argument('--only', type=str, default='', help='comma-separated case names to run')
    p.add_argument('--fp8-training', action='store_true',
                   help='also time the pieces of the FP8 training path: data-gradient GEMMs on transposed FP8 weights and the '
                        'three quantiser kernels (reported in GB/s of bytes read + written)')
    args = p.parse_args()
    dev = torch.device('cuda')
    torch.manual_seed(0)
    g, h, i = args.experts, args.hidden, args.inter
    counts = torch.randint(int(args.rows * 0.7), int(args.rows * 1.3), (g,)).clamp(min=1)
    aligned = (counts + 127) // 128 * 128
    starts = torch.cumsum(aligned, 0) - aligned
    psum, count = (starts + counts).int().to(dev), counts.int().to(dev)
    rows, useful = int(aligned.sum()), int(counts.sum())
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    w1 = (torch.randn(g, 2 * i, h, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(g, h, i, device=dev) * 0.02).to(torch.bfloat16)
    dy1 = torch.randn(rows, 2 * i, device=dev, dtype=torch.bfloat16)
    act = torch.randn(rows, i, device=dev, dtype=torch.bfloat16)
    dw1 = torch.zeros(g, 2 * i, h, device=dev, dtype=torch.float32)
    peak = 1658.2
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        peak = json.load(open(path)).get('bf16_tflops', peak)
    ranges = [(int(s), int(c)) for s, c in zip(starts, counts)]

    def torch_fwd(a, w):
        for e, (s, c) in enumerate(ranges):
            torch.mm(a[s:s + c], w[e].t())

    # library grouped GEMM (`torch.nn.functional.grouped_mm`, one launch for all experts) as a second baseline for the
    # forward GEMMs; group e spans its aligned region, i.e. it also multiplies the zero padding rows
    region_ends = (starts + aligned).int().to(dev)
    grouped_mm = getattr(torch.nn.functional, 'grouped_mm', None)

    def library_grouped(a, w):
        return grouped_mm(a, w.transpose(-2, -1), offs=region_ends)

    cases = {
        'gemm1_forward': (lambda: gg.grouped_gemm_forward(x, w1, psum, count), lambda: torch_fwd(x, w1), 2 * useful * h * 2 * i),
        'gemm1_forward_swiglu': (lambda: gg.grouped_gemm_forward(x, w1, psum, count, swiglu=True), None, 2 * useful * h * 2 * i),
        'gemm2_forward': (lambda: gg.grouped_gemm_forward(act, w2, psum, count), lambda: torch_fwd(act, w2), 2 * useful * h * i),
        'gemm1_dgrad': (lambda: gg.grouped_gemm_dgrad(dy1, w1, psum, count),
                        lambda: [torch.mm(dy1[s:s + c], w1[e]) for e, (s, c) in enumerate(ranges)], 2 * useful * h * 2 * i),
        'gemm1_wgrad_store': (lambda: gg.grouped_gemm_wgrad(dy1, x, dw1, psum, count, accumulate=False), None, 2 * useful * h * 2 * i),
        'gemm1_wgrad': (lambda: gg.grouped_gemm_wgrad(dy1, x, dw1, psum, count),
                        lambda: [torch.mm(dy1[s:s + c].t(), x[s:s + c]) for e, (s, c) in enumerate(ranges)], 2 * useful * h * 2 * i),
    }
    if not args.skip_fp8:
        # FP8 forward path: e4m3 rows with 1 x 128 scales (what the FP8 dispatch delivers), weights with 128 x 128 scales
        from deep_ep.ops.quant import per_token_cast_to_fp8
        x8, x8_sf = per_token_cast_to_fp8(x)
        a8, a8_sf = per_token_cast_to_fp8(act)
        w1_8, w1_sf = gg.per_block_cast_to_fp8(w1)
        w2_8, w2_sf = gg.per_block_cast_to_fp8(w2)
        cases.update({
            'fp8_gemm1_forward': (lambda: gg.grouped_gemm_fp8_forward(x8, x8_sf, w1_8, w1_sf, psum, count), None, 2 * useful * h * 2 * i),
            'fp8_gemm1_forward_swiglu_quant': (lambda: gg.grouped_gemm_fp8_forward(x8, x8_sf, w1_8, w1_sf, psum, count, swiglu=True,
                                                                                   quantize_output=True), None, 2 * useful * h * 2 * i),
            'fp8_gemm2_forward': (lambda: gg.grouped_gemm_fp8_forward(a8, a8_sf, w2_8, w2_sf, psum, count), None, 2 * useful * h * i),
        })
    if not args.skip_fp8:
        # hardware-scaled FP8: the same operands with power-of-two (UE8M0) scales applied by the tensor core
        x8h, x8h_sf = gg.per_token_cast_to_fp8_ue8m0(x)
        a8h, a8h_sf = gg.per_token_cast_to_fp8_ue8m0(act)
        w1_8h, w1h_sf = gg.per_block_cast_to_fp8_ue8m0(w1)
        w2_8h, w2h_sf = gg.per_block_cast_to_fp8_ue8m0(w2)
        cases.update({
            'fp8hw_gemm1_forward': (lambda: gg.grouped_gemm_fp8_forward(x8h, x8h_sf, w1_8h, w1h_sf, psum, count), None, 2 * useful * h * 2 * i),
            'fp8hw_gemm1_forward_swiglu_quant': (lambda: gg.grouped_gemm_fp8_forward(x8h, x8h_sf, w1_8h, w1h_sf, psum, count, swiglu=True,
                                                                                     quantize_output=True), None, 2 * useful * h * 2 * i),
            'fp8hw_gemm2_forward': (lambda: gg.grouped_gemm_fp8_forward(a8h, a8h_sf, w2_8h, w2h_sf, psum, count), None, 2 * useful * h * i),
        })
    bandwidth_cases = {}
    if args.fp8_training:
        from deep_ep.ops import fp8_training as ft
        _, _, w1t_8, w1t_sf = ft.block_quant(w1, transposed=True)
        _, _, w2t_8, w2t_sf = ft.block_quant(w2, transposed=True)
        dy = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
        dy8, dy8_sf = ft.row_quant(dy)
        dh8, dh8_sf = ft.row_quant(dy1)
        cases.update({
            'fp8hw_gemm2_dgrad': (lambda: ft.fp8_gemm(dy8, dy8_sf, w2t_8, w2t_sf, psum, count, 128), None, 2 * useful * h * i),
            'fp8hw_gemm1_dgrad': (lambda: ft.fp8_gemm(dh8, dh8_sf, w1t_8, w1t_sf, psum, count, 128), None, 2 * useful * h * 2 * i),
        })
        bandwidth_cases = {
            'row_quant_hidden': (lambda: ft.row_quant(x), rows * h * 3 + rows * h // 128),
            'row_quant_2inter': (lambda: ft.row_quant(dy1), rows * 2 * i * 3 + rows * 2 * i // 128),
            'swiglu_quant': (lambda: ft.swiglu_quant(dy1, None), rows * 2 * i * 2 + rows * i * 3 + rows * i // 128),
            'block_quant_w1_with_transpose': (lambda: ft.block_quant(w1, transposed=True), g * 2 * i * h * 4),
        }
    out = {'bench': 'grouped_gemm', 'experts': g, 'rows_total': rows, 'rows_useful': useful, 'hidden': h, 'inter': i,
           'peak_tflops_measured': peak, 'results': {}}
    for name, (ours, ref, flops) in cases.items():
        if args.only and name not in args.only.split(','):
            continue
        t_min, t_avg = bench(ours, args.iters)
        entry = {'ours_ms': round(t_avg, 4), 'ours_tflops': round(flops / (t_avg * 1e-3) / 1e12, 1),
                 'ours_frac_of_measured_peak': round(flops / (t_avg * 1e-3) / 1e12 / peak, 3)}
        if ref is not None and not args.skip_torch:
            r_min, r_avg = bench(ref, args.iters)
            entry.update({'torch_loop_ms': round(r_avg, 4), 'torch_loop_tflops': round(flops / (r_avg * 1e-3) / 1e12, 1)})
        if name in ('gemm1_forward', 'gemm2_forward') and grouped_mm is not None and not args.skip_torch:
            operands = (x, w1) if name == 'gemm1_forward' else (act, w2)
            try:
                g_min, g_avg = bench(lambda: library_grouped(*operands), args.iters)
                entry.update({'torch_grouped_mm_ms': round(g_avg, 4),
                              'torch_grouped_mm_tflops': round(flops / (g_avg * 1e-3) / 1e12, 1)})
            except Exception as e:      # not available for this architecture / build
                entry['torch_grouped_mm_error'] = str(e).splitlines()[0][:200]
        out['results'][name] = entry
    hbm = 6543.7
    if os.path.exists(path):
        hbm = json.load(open(path)).get('hbm_gbs', hbm)
    for name, (fn, num_bytes) in bandwidth_cases.items():
        if args.only and name not in args.only.split(','):
            continue
        t_min, t_avg = bench(fn, args.iters)
        out['results'][name] = {'ours_ms': round(t_avg, 4), 'gbs': round(num_bytes / (t_avg * 1e6), 1),
                                'frac_of_measured_copy_bandwidth': round(num_bytes / (t_avg * 1e6) / hbm, 3)}
    print(json.dumps(out))


if __name__ == '__main__':
    main()
