"""GPU tests of the expert-parallel kernels (one process per GPU; a single GPU runs as a 1-rank group)."""
import pytest
import torch

from dist_utils import run_distributed


def _ep_worker(rank, world_size, num_tokens, hidden, num_topk, num_experts, do_cpu_sync, defer, masked, ratio, num_sms, quick=True):
    import torch.distributed as dist
    import deep_ep
    from deep_ep.utils.envs import init_seed
    from ep_check import check_dispatch_combine, check_fused_quant
    init_seed(11)
    with torch.inference_mode():
        buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=num_tokens, hidden=hidden, num_topk=num_topk,
                                  explicitly_destroy=True, num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        assert not buffer.is_simulated
        check_dispatch_combine(buffer, num_tokens, hidden, num_topk, num_experts, do_cpu_sync=do_cpu_sync, defer=defer,
                               masked_ratio=masked, unbalanced_ratio=ratio, quick=quick, num_sms=num_sms)
        if hidden % 128 == 0:
            check_fused_quant(buffer, num_tokens, hidden, num_topk, num_experts)
        buffer.destroy()


CASES = [
    # tokens, hidden, topk, experts, cpu_sync, defer, masked, ratio, num_sms
    (257, 512, 6, 64, True, True, 0.0, 1.0, 0),
    (130, 1024, 8, 32, False, False, 0.2, 2.0, 3),
    (1024, 7168, 6, 256, True, True, 0.0, 1.0, 24),
]


@pytest.mark.gpu
@pytest.mark.parametrize('case', CASES)
def test_ep_single_gpu(master_port, case):
    run_distributed(_ep_worker, 1, master_port, 'nccl', case)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize('case', CASES)
def test_ep_multi_gpu(master_port, case):
    world = min(torch.cuda.device_count(), 8)
    world -= world % 2
    if case[3] % world:
        pytest.skip('experts not divisible')
    run_distributed(_ep_worker, world, master_port, 'nccl', case)


@pytest.mark.gpu
def test_ep_full_mode_matrix(master_port):
    """Every mode of the reference's sweep (`tests/ep/test_ep.py:25-30`): alignment {128, 1} x FP8 / BF16 x 0, 1 or 2 biases x
    row- or column-major scale factors, on all visible GPUs (an even number of them, or one)."""
    world = min(torch.cuda.device_count(), 8)
    world = world - world % 2 if world > 1 else 1
    run_distributed(_ep_worker, world, master_port, 'nccl', (190, 512, 4, 8 * world, True, True, 0.1, 1.5, 0, False))


def _recreate_worker(rank, world_size):
    import torch.distributed as dist
    import deep_ep
    # buffers are created, used once and destroyed again and again: allocation, peer mapping and release must not leak
    # or leave a stale mapping behind (the reference's pressure loop, `tests/ep/test_ep.py:538-547`)
    free_after_first = None
    for i in range(6):
        buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=64 + i, hidden=512, num_topk=2, explicitly_destroy=True,
                                  num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        x = torch.full((32, 512), float(rank + i), device='cuda', dtype=torch.bfloat16)
        idx = torch.rand(32, 4 * world_size, device='cuda').topk(2, dim=-1).indices
        recv_x, _, _, handle, _ = buffer.dispatch(x, topk_idx=idx, num_experts=4 * world_size, expert_alignment=1, do_expand=True)
        combined, _, _ = buffer.combine(recv_x, handle)
        torch.cuda.synchronize()
        # both copies of a token come back and are summed: small integers, exact in bf16 whatever the split over ranks
        assert torch.equal(combined.float(), torch.full((32, 512), 2.0 * (rank + i), device='cuda')), i
        buffer.destroy()
        if free_after_first is None:
            # the first lifetime also pays for one-off allocations (communicator buffers, the caching allocator's pools)
            torch.cuda.synchronize()
            free_after_first = torch.cuda.mem_get_info()[0]
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_after_first - (64 << 20), 'device memory leaked across buffer lifetimes'


def _pending_worker(rank, world_size):
    from test_ep_gloo import _pending_epilogue_worker
    with torch.cuda.device(rank):
        torch.set_default_device('cuda')
        try:
            _pending_epilogue_worker(rank, world_size)
        finally:
            torch.set_default_device('cpu')
    torch.cuda.synchronize()


@pytest.mark.gpu
def test_second_operation_is_refused_while_a_deferred_epilogue_is_pending_gpu(master_port):
    run_distributed(_pending_worker, min(torch.cuda.device_count(), 2), master_port, 'nccl')


@pytest.mark.gpu
def test_ep_buffer_recreation(master_port):
    world = min(torch.cuda.device_count(), 2)
    run_distributed(_recreate_worker, world, master_port, 'nccl')


@pytest.mark.gpu
@pytest.mark.parametrize('num_tokens,num_topk,num_experts,num_ranks', [(1, 4, 16, 2), (1000, 6, 256, 8), (16384, 8, 256, 8), (333, 32, 64, 64)])
def test_dispatch_layout_matches_cpu_rule(num_tokens, num_topk, num_experts, num_ranks):
    from deep_ep.ops.layout import get_dispatch_layout
    torch.manual_seed(3)
    idx = torch.rand(num_tokens, num_experts).topk(num_topk, dim=-1).indices
    idx = idx.masked_fill(torch.rand(idx.shape) < 0.1, -1)
    ref_slots, ref_rank, ref_expert = get_dispatch_layout(idx, num_experts, num_ranks)
    for _ in range(2):        # scratch state must not leak between launches
        slots, per_rank, per_expert = get_dispatch_layout(idx.cuda(), num_experts, num_ranks)
        assert torch.equal(slots.cpu(), ref_slots) and torch.equal(per_rank.cpu(), ref_rank)
        assert torch.equal(per_expert.cpu(), ref_expert)
