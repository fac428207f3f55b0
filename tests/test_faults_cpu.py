"""Failure detection, injected on the host among CPU (gloo) ranks: no GPU is involved and nothing faults a device.

A rank that never joins a collective, ranks that disagree on the buffer configuration, a routing tensor edited behind
a live handle, and misuse of the API must all surface as Python exceptions on the healthy ranks.
"""
import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed


def _rank1_never_joins(rank, world):
    import deep_ep
    if rank == 1:
        return                                    # leaves before the collective constructor
    # the healthy rank's bootstrap collective must end with an error once the short group timeout runs out
    with pytest.raises(Exception):
        deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=8, hidden=64, num_topk=2)


def test_missing_rank_times_out(master_port):
    run_distributed(_rank1_never_joins, 2, master_port, 'gloo', timeout_s=5)


def _mismatched_config(rank, world):
    import deep_ep
    with pytest.raises(AssertionError, match='differ across ranks'):
        deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=8 + rank, hidden=64, num_topk=2)


def test_mismatched_buffer_config_is_rejected(master_port):
    run_distributed(_mismatched_config, 2, master_port, 'gloo', timeout_s=30)


def _api_misuse(rank, world):
    import deep_ep
    buf = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=16, hidden=32, num_topk=2, explicitly_destroy=True)
    x = torch.randn(16, 32)
    idx = torch.rand(16, 4).topk(2, dim=-1).indices
    with pytest.raises(AssertionError):
        buf.dispatch(x, topk_idx=idx, num_experts=4)                       # do_expand is mandatory
    with pytest.raises(NotImplementedError):
        buf.dispatch(x, topk_idx=idx, num_experts=4, do_expand=True, num_qps=3)
    recv_x, _, _, handle, _ = buf.dispatch(x, topk_idx=idx, num_experts=4, do_expand=True)
    with pytest.raises(AssertionError):
        buf.dispatch(x, topk_idx=idx, handle=handle, do_expand=True)       # cached dispatch takes no topk_idx
    with pytest.raises(AssertionError):
        buf.dispatch(x, handle=handle, do_expand=True, do_cpu_sync=True)   # nor a host sync
    idx.add_(0)                                                            # edits the routing behind the handle
    with pytest.raises(AssertionError, match='must not be modified'):
        buf.combine(recv_x, handle)
    with pytest.raises(NotImplementedError):
        deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=16, hidden=32, num_topk=2, sl_idx=1)
    buf.destroy()
    not_explicit = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=16, hidden=32, num_topk=2)
    with pytest.raises(AssertionError):
        not_explicit.destroy()                                             # needs explicitly_destroy=True


def test_api_misuse_raises(master_port):
    run_distributed(_api_misuse, 2, master_port, 'gloo', timeout_s=60)
