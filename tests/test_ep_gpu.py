"""GPU tests of the expert-parallel kernels (one process per GPU; a single GPU runs as a 1-rank group)."""
import pytest
import torch

from dist_utils import run_distributed


def _ep_worker(rank, world_size, num_tokens, hidden, num_topk, num_experts, do_cpu_sync, defer, masked, ratio, num_sms):
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
                               masked_ratio=masked, unbalanced_ratio=ratio, quick=True, num_sms=num_sms)
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
