"""Compute operators next to the communication buffers.

* `grouped_gemm`: tcgen05 grouped GEMMs of the expert FFNs (bf16 forward / data gradient / weight gradient, FP8 forward with
  fp32 or power-of-two block scales), the fused SwiGLU FFN autograd node, weight quantisers.
* `fp8_training`: opt-in FP8 training path of the expert FFN (FP8 forward and data-gradient GEMMs, bf16 weight gradients).
* `quant`, `jit`: run-time specialised kernels (per-token FP8 quantiser compiled for the hidden size in use).
* `layout`: routing layout of a batch (`get_dispatch_layout`).
* `dense`: the router's and the shared expert's dense products on the same tcgen05 kernels (one group).
"""
__all__ = ['dense', 'fp8_training', 'grouped_gemm', 'jit', 'layout', 'quant']
