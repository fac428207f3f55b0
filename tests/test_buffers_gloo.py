"""`BucketBuffer`, `PPBuffer` and `EngramBuffer` over CPU process groups (gloo): the Python layer of the three buffers
(sessions, alias rules, argument checks, hooks) on top of the simulated runtimes, with the checks of the reference's
`tests/bucket/test_all_gather.py`, `tests/bucket/test_session.py`, `tests/pp/test_pp.py` and `tests/engram/test_engram.py`."""
import pytest
import torch

from dist_utils import run_distributed


def _bucket_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    sub = dist.new_group(list(range(world)))
    bucket = deep_ep.BucketBuffer([group, sub], 4 << 20, explicitly_destroy=True)
    assert bucket.is_simulated and bucket.get_context_idx(sub) == 1
    with pytest.raises(AssertionError):
        bucket.get_context_idx(None)                      # several groups: the group must be named

    # in place: my shard already sits inside the gathered tensor
    n = 1000
    full = bucket.storage.narrow(0, 0, world * n * 4).view(torch.float32).view(world, n)
    full.fill_(float('nan'))
    full[rank] = rank + 0.5
    out = bucket.all_gather(full[rank], group=group).wait()
    assert torch.equal(out.view(world, n)[:, 7], torch.arange(world).float() + 0.5)
    # out of place into a registered destination, odd size, second group
    src = torch.arange(37, dtype=torch.int16) + 100 * rank
    dst = bucket.storage.narrow(0, 1 << 20, world * src.nbytes).view(torch.int16)
    out2 = bucket.all_gather(src, dst, group=sub).wait()
    assert torch.equal(out2.view(world, 37)[:, 0], (torch.arange(world) * 100).to(torch.int16))
    # a full batch of 64 tensors at once
    srcs = [torch.full((16,), float(rank * 100 + i)) for i in range(64)]
    dsts = [bucket.storage.narrow(0, (2 << 20) + i * world * 64, world * 64).view(torch.float32) for i in range(64)]
    outs = bucket.all_gather(srcs, dsts, group=group).wait()
    for i, o in enumerate(outs):
        assert torch.equal(o.view(world, 16)[:, 0], torch.arange(world).float() * 100 + i)
    # outputs outside the storage are rejected
    with pytest.raises(AssertionError):
        bucket.all_gather(src, torch.empty(world * 37, dtype=torch.int16), group=group)

    # sessions: unregistered tensors, exclusivity, cleanup on exceptions
    original = bucket.all_gather
    with bucket.session() as session:
        user_dst = torch.empty(world * 50)
        got = bucket.all_gather(torch.full((50,), float(rank)), user_dst, group=group).wait()
        assert got is user_dst and torch.equal(got.view(world, 50)[:, 3], torch.arange(world).float())
        reg = session.allocate((world, 64), torch.bfloat16, group=group)
        reg[rank] = rank + 1
        got2 = bucket.all_gather(reg[rank], group=group).wait()
        assert torch.equal(got2.view(world, 64)[:, 0].float(), torch.arange(world).float() + 1)
        with pytest.raises(AssertionError):
            bucket.all_gather(torch.zeros(8), group=sub)          # a session is bound to its first group
        with pytest.raises(AssertionError):
            with bucket.session():
                pass
    assert bucket.all_gather == original
    with pytest.raises(RuntimeError):
        with bucket.session():
            raise RuntimeError('boom')
    assert bucket.all_gather == original and bucket._active_session is None

    # randomised schedule (reference: `tests/bucket/test_session.py:65-185`): 64 gathers with at most 4 in flight, sizes
    # and forms mixed (outside destination, no destination, in place inside a session allocation, batches of two);
    # when the arena runs low the ranks meet at a barrier and the session starts again at offset 0
    import random
    rng = random.Random(5)
    with bucket.session() as session:
        inflight = []

        def drain():
            for tag, count, handle in inflight:
                outs = handle.wait()
                outs = [outs] if isinstance(outs, torch.Tensor) else outs
                assert len(outs) == count
                for k, out in enumerate(outs):
                    assert torch.equal(out.view(world, -1)[:, -1].float(), torch.arange(world).float() + tag + k)
            inflight.clear()
        for i in range(64):
            n, form = rng.choice([7, 256, 4099]), rng.randrange(4)
            src = torch.full((n,), float(rank + i), dtype=torch.bfloat16)
            if form == 0:
                inflight.append((i, 1, bucket.all_gather(src, torch.empty(world * n, dtype=torch.bfloat16), group=group)))
            elif form == 1:
                inflight.append((i, 1, bucket.all_gather(src, group=group)))
            elif form == 2:
                full = session.allocate((world, n), torch.bfloat16, group=group)
                full[rank] = src
                inflight.append((i, 1, bucket.all_gather(full[rank], group=group)))
            else:
                pair = [src, torch.full((n + 3,), float(rank + i + 1), dtype=torch.bfloat16)]
                inflight.append((i, 2, bucket.all_gather(pair, [torch.empty(world * t.numel(), dtype=torch.bfloat16) for t in pair], group=group)))
            if len(inflight) >= 4 or session.offset > (3 << 20):
                drain()
                if session.offset > (3 << 20):
                    bucket.barrier(group=group)
                    session.offset = 0
        drain()

    # reduce-scatter and all-reduce: fp32 sum in rank order, scaled, one rounding
    with bucket.session() as session:
        t = session.allocate((world * 8 * 25,), torch.bfloat16, group=group)
        mine = (torch.arange(t.numel()).float() * 0.01 + rank).to(torch.bfloat16)
        expect = torch.zeros(t.numel())
        for r in range(world):
            expect += (torch.arange(t.numel()).float() * 0.01 + r).to(torch.bfloat16).float()
        t.copy_(mine)
        out = bucket.all_reduce(t, scale=0.5, group=group).wait()
        assert out.data_ptr() == t.data_ptr() and torch.equal(out, (expect * 0.5).to(torch.bfloat16))
        t.copy_(mine)
        shard = bucket.reduce_scatter(t, group=group).wait()
        m = t.numel() // world
        assert torch.equal(shard, expect.to(torch.bfloat16)[rank * m:(rank + 1) * m])
        keep = torch.ones(t.numel(), dtype=torch.bool)
        keep[rank * m:(rank + 1) * m] = False
        assert torch.equal(t[keep], mine[keep])
        # inside a session tensors outside the storage are staged: all-reduce stays in place for the caller,
        # reduce-scatter hands back the reduced shard
        user = mine.clone()
        out = bucket.all_reduce(user, scale=0.5, group=group).wait()
        assert out is user and torch.equal(user, (expect * 0.5).to(torch.bfloat16))
        user2, user3 = mine.clone(), mine.clone().float()
        expect3 = torch.zeros(t.numel())
        for r in range(world):
            expect3 += (torch.arange(t.numel()).float() * 0.01 + r).to(torch.bfloat16).float()
        shards = bucket.reduce_scatter([user2, user3], group=group).wait()
        assert torch.equal(shards[0], expect.to(torch.bfloat16)[rank * m:(rank + 1) * m])
        assert torch.equal(shards[1], expect3[rank * m:(rank + 1) * m])
        assert torch.equal(user2, mine)                                  # the caller's tensor is only read
    with pytest.raises((AssertionError, deep_ep.EPException)):
        bucket.all_reduce(torch.zeros(world * 16), group=group)          # outside a session: not registered
    bucket.destroy()


def _pp_worker(rank, world, transport='nvlink'):
    import torch.distributed as dist
    import deep_ep
    pp = deep_ep.PPBuffer(dist.group.WORLD, 1 << 16, 3, explicitly_destroy=True, transport=transport)
    assert pp.is_simulated and pp.transport == transport
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    # several sends run ahead of their receives (up to the in-flight limit), FIFO per pair
    for i in range(3):
        pp.send(torch.full((100,), float(10 * rank + i)), nxt)
    for i in range(3):
        got = torch.empty(100)
        pp.recv(got, prv)
        assert torch.all(got == 10 * prv + i)
    # mixed sizes and dtypes, both directions when the ring has more than two ranks
    if world > 2:
        pp.send(torch.arange(33, dtype=torch.int32) + rank, prv)
        got = torch.empty(33, dtype=torch.int32)
        pp.recv(got, nxt)
        assert torch.equal(got, torch.arange(33, dtype=torch.int32) + nxt)
    # both directions at once, random schedule honouring the in-flight limit (same seed on every rank), as the
    # reference's `tests/pp/test_pp.py:16-47,96-111` does with timestamps
    import random
    rng = random.Random(11)
    sent, received = {0: 0, 1: 0}, {0: 0, 1: 0}

    def receive(d):
        src = prv if d == 0 else nxt
        got = torch.empty(64 + 5 * (received[d] % 7), dtype=torch.bfloat16)
        pp.recv(got, src)
        assert torch.all(got == float(100 * d + received[d] % 50 + src))
        received[d] += 1
    for _ in range(80):
        d = rng.randrange(2) if world > 2 else 0                     # with two ranks both directions are one channel
        if sent[d] - received[d] < 3 and rng.random() < 0.6:
            pp.send(torch.full((64 + 5 * (sent[d] % 7),), float(100 * d + sent[d] % 50 + rank), dtype=torch.bfloat16), nxt if d == 0 else prv)
            sent[d] += 1
        elif received[d] < sent[d]:
            receive(d)
    for d in (0, 1):
        while received[d] < sent[d]:
            receive(d)
    with pytest.raises(AssertionError):
        pp.send(torch.zeros(1 << 20), nxt)                           # larger than the slot
    if world > 3:
        with pytest.raises(AssertionError):
            pp.send(torch.zeros(4), (rank + 2) % world)              # not a ring neighbour
    pp.destroy()


def _engram_worker(rank, world, use_fp8):
    import torch.distributed as dist
    import deep_ep
    from deep_ep.utils.math import per_token_cast_to_fp8
    group = dist.group.WORLD
    entries, hidden, per_token, num_tokens = [40, 24], 256, 6, 20
    dtype = torch.float8_e4m3fn if use_fp8 else torch.bfloat16
    packs = hidden // 128 * 2 if use_fp8 else 0
    recv, storage = deep_ep.EngramBuffer.get_storage_size_hint(group, entries, hidden, num_tokens, per_token, dtype, packs)
    buf = deep_ep.EngramBuffer(group, recv, storage, explicitly_destroy=True)
    assert buf.is_simulated
    buf.set_config(entries, hidden, num_tokens, per_token, dtype, packs)
    torch.manual_seed(50 + rank)
    tables = [torch.randn(n, hidden).to(torch.bfloat16) for n in entries]

    def gather(t):
        out = [torch.empty_like(t.view(torch.uint8)) for _ in range(world)]
        dist.all_gather(out, t.contiguous().view(torch.uint8))
        return torch.cat(out)
    if use_fp8:
        quant = [per_token_cast_to_fp8(t) for t in tables]
        local = [q for q, _ in quant]
        full_sf = [gather(s.contiguous().view(torch.int16)).view(torch.int16).view(world * n, packs) for (_, s), n in zip(quant, entries)]
    else:
        local, full_sf = tables, None
    full = [gather(t).view(world * n, -1) for t, n in zip(local, entries)]
    buf.write(local, full_sf)
    torch.manual_seed(7)
    idx = torch.stack([torch.randint(0, world * n, (num_tokens, per_token), dtype=torch.int32) for n in entries])
    idx[0, 3, 5] = -1
    for col_major in ((False, True) if use_fp8 else (False,)):
        hooks = buf.fetch(idx, use_tma_aligned_col_major_sf=col_major)
        for layer in (1, 0):
            out = hooks[layer]()
            fetched, sf = out if use_fp8 else (out, None)
            flat = idx[layer].long().clamp(min=0).view(-1)
            ref = full[layer][flat].view(num_tokens, -1)
            got = fetched.view(torch.uint8).view(num_tokens, -1)
            keep = torch.ones(num_tokens, per_token, dtype=torch.bool)
            if layer == 0:
                keep[3, 5] = False
            keep_b = keep.repeat_interleave(got.size(1) // per_token, dim=1)
            assert torch.equal(got[keep_b], ref[keep_b])
            if use_fp8:
                assert sf.stride() == ((1, num_tokens) if col_major else (per_token * packs, 1))
                assert torch.equal(sf[keep.repeat_interleave(packs, dim=1)],
                                   full_sf[layer][flat].view(num_tokens, per_token * packs)[keep.repeat_interleave(packs, dim=1)])
    buf.destroy()


def test_bucket_buffer_two_cpu_ranks(master_port):
    run_distributed(_bucket_worker, 2, master_port, 'gloo', timeout_s=120)


@pytest.mark.parametrize('world', [2, 4])
def test_pp_buffer_cpu_ranks(master_port, world):
    run_distributed(_pp_worker, world, master_port, 'gloo', timeout_s=120)


@pytest.mark.parametrize('world', [2, 3])
def test_pp_buffer_library_transport_cpu_ranks(master_port, world):
    """`transport='nccl'`: the process group's own send / recv behind staging slots (over gloo on CPU ranks), with the
    same buffered semantics: sends run ahead of their receives, also when both ranks of a pair send first."""
    run_distributed(_pp_worker, world, master_port, 'gloo', ('nccl',), timeout_s=120)


@pytest.mark.parametrize('use_fp8', [False, True])
def test_engram_buffer_two_cpu_ranks(master_port, use_fp8):
    run_distributed(_engram_worker, 2, master_port, 'gloo', (use_fp8,), timeout_s=120)


def _mesh_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    from deep_ep.parallel import ParallelMesh
    mesh = ParallelMesh(ep_size=2, pp_size=2)                    # 4 ranks: pp x dp x ep = 2 x 1 x 2, ep innermost
    assert mesh.coords == {'pp': rank // 2, 'dp': 0, 'ep': rank % 2}
    assert mesh.groups_of('ep') == [(0, 1), (2, 3)] and mesh.groups_of('pp') == [(0, 2), (1, 3)]
    assert mesh.group('ep').size() == 2 and mesh.group('pp').size() == 2 and mesh.group('dp').size() == 1
    assert mesh.pp_next() == (rank + 2) % 4 == mesh.pp_prev()
    assert mesh.rank_of(ep=1 - rank % 2) == rank ^ 1
    # an expert-parallel exchange inside each EP group and a pipeline hop across them
    buffer = mesh.ep_buffer(num_max_tokens_per_rank=8, hidden=64, num_topk=2, explicitly_destroy=True)
    x = torch.full((8, 64), float(rank)).to(torch.bfloat16)
    idx = torch.stack([torch.arange(8) % 4, (torch.arange(8) + 1) % 4], dim=1)
    recv_x, _, _, handle, _ = buffer.dispatch(x, topk_idx=idx, num_experts=4, expert_alignment=1, do_expand=True)
    combined, _, _ = buffer.combine(recv_x, handle)
    assert torch.equal(combined.float(), torch.full((8, 64), 2.0 * rank))
    assert set(recv_x.float().unique().tolist()) <= {float(r) for r in mesh.axes['ep'].ranks}
    buffer.destroy()
    pp = mesh.pp_buffer(1 << 12, 2, explicitly_destroy=True)
    peer = mesh.group('pp').rank() ^ 1                            # the other rank of this two-stage pipeline
    pp.send(torch.full((16,), float(rank)), peer)
    got = torch.empty(16)
    pp.recv(got, peer)
    assert torch.all(got == mesh.pp_next())
    pp.destroy()


def test_parallel_mesh_builds_groups_and_buffers(master_port):
    run_distributed(_mesh_worker, 4, master_port, 'gloo', timeout_s=180)
