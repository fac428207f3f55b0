"""An expert-parallel MoE layer built on `EPBuffer`: gate -> dispatch -> per-expert SwiGLU FFN -> combine,
with a backward pass that reuses the routing handle (the gradient of dispatch is a combine and the
gradient of combine is a cached dispatch). The router trains too: the expert FFN returns the gradient of every
expanded row's routing weight, and the combine that is the backward of dispatch carries those scalars back to their
(token, top-k position) through its positional weight channel, from where autograd reaches the gate matrix.
This is the "one model" of a communication library: the layer shape follows the DeepSeek-V3 expert FFN (hidden 7168,
intermediate 2048, 256 routed experts, top-8, one shared expert), cf. the usage sketch in the reference's
`README.md:178-194`.
"""
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..buffers.ep import EPBuffer, EPHandle


@dataclass
class MoEConfig:
    hidden: int = 7168
    intermediate: int = 2048
    num_experts: int = 256
    num_topk: int = 8
    num_shared_experts: int = 0
    num_max_tokens_per_rank: int = 4096
    expert_alignment: int = 128
    fp8_scales: str = 'fp32'            # inference (`forward_fp8`: e4m3 dispatch quantised inside the dispatch kernel feeding
                                        # block-scaled FP8 expert GEMMs). 'fp32': scales amax / 448, promoted in registers by the
                                        # GEMM; 'ue8m0': powers of two, applied by the tensor core (hidden and intermediate
                                        # must be multiples of 512)
    fp8_training: bool = False          # training: forward and data-gradient GEMMs of the routed experts in FP8 (e4m3, power-of-two
                                        # 1x128 / 128x128 scales applied by the tensor core), weight gradients in bf16;
                                        # hidden and intermediate must be multiples of 512
    host_sync: bool = True              # dispatch waits on the host for the received-token counts and sizes its outputs exactly;
                                        # False: outputs get their worst-case size and nothing touches the host, so a whole
                                        # forward pass can be captured in one CUDA graph (decode); consumers read the counts
                                        # from the handle's device tensors, as the grouped GEMMs do
    overlap_shared_expert: bool = False # run the shared expert on a side stream next to dispatch / routed experts / combine
    fuse_combine: bool = False          # the second expert GEMM stores the rows of single-row tokens straight into their
                                        # owners' combine landing slots (over NVLink, tile by tile); combine sends the rest
    expert_backend: str = 'grouped'     # 'grouped': hand-written grouped GEMM kernels, 'torch': per-expert torch.mm
    num_sms: int = 0
    init_std: float = 0.02


class _Dispatch(torch.autograd.Function):
    """recv_x, recv_w = dispatch(x, topk_weights). Backward: one combine with the same handle returns both gradients:
    grad_x is the sum of the rows' gradients, and the gradient of every expanded row's routing weight travels back to
    its (token, top-k position) through the combine's positional weight channel."""

    @staticmethod
    def forward(ctx, x, topk_idx, topk_weights, layer):
        cfg = layer.config
        recv_x, _, recv_w, handle, _ = layer.buffer.dispatch(
            x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=cfg.num_experts,
            expert_alignment=cfg.expert_alignment, num_sms=cfg.num_sms, do_expand=True, do_zero_padding=True,
            do_cpu_sync=cfg.host_sync)
        ctx.layer, ctx.handle = layer, handle
        layer._handle = handle
        return recv_x, recv_w

    @staticmethod
    def backward(ctx, grad_recv_x, grad_recv_w):
        # with `fuse_combine` the data-gradient GEMM that produced `grad_recv_x` has already stored the rows of
        # single-row tokens into their owners' landing slots
        want_w = grad_recv_w is not None and ctx.needs_input_grad[2]
        grad_x, grad_topk_w, _ = ctx.layer.buffer.combine(
            grad_recv_x.contiguous(), ctx.handle, topk_weights=grad_recv_w.float().contiguous() if want_w else None,
            fused_single_rows=ctx.layer._backward_route_used)
        ctx.layer._backward_route_used = False
        return grad_x, None, (grad_topk_w if want_w else None), None


class _Combine(torch.autograd.Function):
    """y = combine(x). Backward: grad_x = cached dispatch(grad_y) (every expanded row receives its token's gradient)."""

    @staticmethod
    def forward(ctx, x, layer, handle, fused_single_rows=False):
        ctx.layer, ctx.handle = layer, handle
        combined, _, _ = layer.buffer.combine(x, handle, fused_single_rows=fused_single_rows)
        return combined

    @staticmethod
    def backward(ctx, grad_y):
        grad_x, _, _, _, _ = ctx.layer.buffer.dispatch(grad_y.contiguous(), handle=ctx.handle, do_expand=True,
                                                       do_zero_padding=True)
        return grad_x, None, None, None


class MoELayer(nn.Module):
    """Expert-parallel MoE FFN. Experts `[rank * E_local, (rank + 1) * E_local)` live on this rank."""

    def __init__(self, group: dist.ProcessGroup, config: MoEConfig, buffer: Optional[EPBuffer] = None,
                 device: Optional[torch.device] = None):
        """`device`: where the parameters are created (default: CPU, to be moved with `.to()`); creating them on the GPU
        avoids generating gigabytes of random numbers on the host for layers with many local experts."""
        super().__init__()
        self.group, self.config = group, config
        self.num_ranks, self.rank = group.size(), group.rank()
        assert config.num_experts % self.num_ranks == 0
        self.num_local_experts = config.num_experts // self.num_ranks
        h, i, e = config.hidden, config.intermediate, self.num_local_experts
        std = config.init_std
        self.gate = nn.Parameter(torch.randn(config.num_experts, h, dtype=torch.float32, device=device) * std)
        self.w_gate_up = nn.Parameter(torch.randn(e, 2 * i, h, dtype=torch.bfloat16, device=device) * std)   # [gate; up] rows
        self.w_down = nn.Parameter(torch.randn(e, h, i, dtype=torch.bfloat16, device=device) * std)
        if config.num_shared_experts > 0:
            si = i * config.num_shared_experts
            self.shared_gate_up = nn.Parameter(torch.randn(2 * si, h, dtype=torch.bfloat16, device=device) * std)
            self.shared_down = nn.Parameter(torch.randn(h, si, dtype=torch.bfloat16, device=device) * std)
        self._own_buffer = buffer is None
        self.buffer = buffer if buffer is not None else EPBuffer(
            group, num_max_tokens_per_rank=config.num_max_tokens_per_rank, hidden=h, num_topk=config.num_topk,
            explicitly_destroy=True)
        self._handle: Optional[EPHandle] = None
        self._backward_route_used = False
        self._side_stream = None
        self._fp8_cache = None

    def destroy(self) -> None:
        if self._own_buffer and self.buffer is not None:
            self.buffer.destroy()
        self.buffer = None

    def route(self, x: torch.Tensor):
        """Top-k routing of `x`. The logits are an fp32-accumulated product of the bf16 activations with the gate matrix
        rounded to bf16 (the fp32 parameter stays the master copy), computed by the layer's own tensor-core kernel."""
        from ..ops.dense import dense_linear
        if x.is_cuda and x.dtype == torch.bfloat16:
            logits = dense_linear(x, self.gate.to(torch.bfloat16), out_fp32=True)
        else:
            logits = F.linear(x.float(), self.gate)
        scores = torch.softmax(logits, dim=-1)
        topk_weights, topk_idx = scores.topk(self.config.num_topk, dim=-1)
        topk_weights = topk_weights / topk_weights.sum(dim=-1, keepdim=True)
        return topk_idx, topk_weights

    def experts(self, recv_x: torch.Tensor, recv_w: torch.Tensor, handle: EPHandle,
                route: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Expert FFN on the expanded rows, already multiplied by each row's routing weight."""
        from ..ops.grouped_gemm import grouped_swiglu_ffn
        backward_route = None
        if route is not None and torch.is_grad_enabled() and recv_x.requires_grad:
            def barrier_then_mark():
                self.buffer.barrier()
                self._backward_route_used = True
            backward_route = (route, barrier_then_mark)
        if self.config.fp8_training:
            from ..ops.fp8_training import Fp8WeightCache, grouped_swiglu_ffn_fp8_training
            if self._fp8_cache is None:
                self._fp8_cache = Fp8WeightCache()
            return grouped_swiglu_ffn_fp8_training(recv_x, self.w_gate_up, self.w_down, handle.psum_num_recv_tokens_per_expert,
                                                   handle.num_unaligned_recv_tokens_per_expert, self.config.expert_alignment,
                                                   self._fp8_cache, row_scale=recv_w, route=route, backward_route=backward_route)
        return grouped_swiglu_ffn(recv_x, self.w_gate_up, self.w_down, handle.psum_num_recv_tokens_per_expert,
                                  handle.num_unaligned_recv_tokens_per_expert, handle.num_recv_tokens_per_expert_list,
                                  self.config.expert_alignment, backend=self.config.expert_backend, row_scale=recv_w,
                                  route=route, backward_route=backward_route)

    # ------------------------------------------------------------------------------------------ FP8 inference
    def quantize_weights(self) -> None:
        """Store the routed experts' weights as e4m3 with one fp32 scale per 128 x 128 block (used by `forward_fp8`)."""
        from ..ops.grouped_gemm import per_block_cast_to_fp8, per_block_cast_to_fp8_ue8m0
        assert self.config.fp8_scales in ('fp32', 'ue8m0')
        cast = per_block_cast_to_fp8_ue8m0 if self.config.fp8_scales == 'ue8m0' else per_block_cast_to_fp8
        with torch.no_grad():
            self._w1_fp8, self._w1_sf = cast(self.w_gate_up)
            self._w2_fp8, self._w2_sf = cast(self.w_down)

    @torch.no_grad()
    def forward_fp8(self, x: torch.Tensor) -> torch.Tensor:
        """Forward pass for inference with FP8 on the wire and on the tensor cores: the dispatch kernel quantises the
        bf16 tokens to e4m3 (fp32 1 x 128 scales), GEMM1 consumes the received rows as they are and re-quantises the
        SwiGLU output in its epilogue, GEMM2 writes bf16 for the combine. Needs `quantize_weights()` once."""
        from ..ops.grouped_gemm import grouped_swiglu_ffn_fp8
        cfg = self.config
        assert cfg.expert_alignment % 128 == 0, 'the FP8 path needs an expert alignment that is a multiple of 128'
        if getattr(self, '_w1_fp8', None) is None:
            self.quantize_weights()
        topk_idx, topk_weights = self.route(x)
        (recv_x, recv_sf), _, recv_w, handle, _ = self.buffer.dispatch(
            x, topk_idx=topk_idx, topk_weights=topk_weights.float().contiguous(), num_experts=cfg.num_experts,
            expert_alignment=cfg.expert_alignment, num_sms=cfg.num_sms, do_expand=True, do_zero_padding=True,
            do_cpu_sync=cfg.host_sync, fused_fp8_quant='ue8m0' if cfg.fp8_scales == 'ue8m0' else True)
        route = None
        if cfg.fuse_combine and cfg.fp8_scales == 'ue8m0':
            route = self.buffer.build_combine_route(handle, cfg.hidden)
            self.buffer.barrier()
        y = grouped_swiglu_ffn_fp8(recv_x, recv_sf, self._w1_fp8, self._w1_sf, self._w2_fp8, self._w2_sf,
                                   handle.psum_num_recv_tokens_per_expert, handle.num_unaligned_recv_tokens_per_expert,
                                   alignment=cfg.expert_alignment, row_scale=recv_w, route=route)
        out, _, _ = self.buffer.combine(y, handle, fused_single_rows=route is not None)
        if cfg.num_shared_experts > 0:
            out = out + self._shared_expert(x)
        return out

    def _shared_expert(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops.dense import dense_swiglu_ffn
        return dense_swiglu_ffn(x, self.shared_gate_up, self.shared_down)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shared = None
        if self.config.num_shared_experts > 0 and self.config.overlap_shared_expert and x.is_cuda:
            # the shared expert only needs `x`: it runs on its own stream while the routed path communicates
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream()
            self._side_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side_stream):
                shared = self._shared_expert(x)
        topk_idx, topk_weights = self.route(x)
        recv_x, recv_w = _Dispatch.apply(x, topk_idx, topk_weights.float().contiguous(), self)
        handle = self._handle
        route = None
        if self.config.fuse_combine:
            # landing addresses of the rows the second GEMM may deliver itself; the barrier makes sure every rank has
            # finished reading the landing area (its dispatch epilogue) before the first such store
            route = self.buffer.build_combine_route(handle, self.config.hidden)
            self.buffer.barrier()
        y = self.experts(recv_x, recv_w, handle, route)
        out = _Combine.apply(y, self, handle, route is not None)
        if shared is not None:
            torch.cuda.current_stream().wait_stream(self._side_stream)
            shared.record_stream(torch.cuda.current_stream())
            out = out + shared
        elif self.config.num_shared_experts > 0:
            out = out + self._shared_expert(x)
        return out
