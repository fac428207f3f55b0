"""GPU tests of the non-EP buffers: barrier, events/streams, allocation plans, bucket all-gather and sessions,
pipeline send/recv, Engram fetch, and bounded device waits. A single GPU runs them as a 1-rank group; with more
GPUs the same bodies run with one process per GPU."""
import pytest
import torch

from dist_utils import run_distributed


def _world():
    n = torch.cuda.device_count()
    return 1 if n < 2 else min(n - n % 2, 8)


# ---------------------------------------------------------------------------------------------------- barrier
def _barrier_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    for _ in range(3):                      # construct / destroy loop
        buf = deep_ep.PPBuffer(group, 1 << 20, 2, explicitly_destroy=True, num_gpu_timeout_secs=10)
        for _ in range(101):                # odd count: both phases and both signs of the counter are used
            buf.barrier()
        buf.barrier(with_cpu_sync=True)
        assert buf.context.status_code() == 0
        buf.destroy()


@pytest.mark.gpu
def test_barrier(master_port):
    run_distributed(_barrier_worker, _world(), master_port, 'nccl')


# ---------------------------------------------------------------------------------------------------- bounded wait
def _timeout_worker(rank, world):
    import time
    import torch.distributed as dist
    import deep_ep
    buf = deep_ep.PPBuffer(dist.group.WORLD, 1 << 20, 2, explicitly_destroy=True, num_gpu_timeout_secs=10)
    t0 = time.time()
    buf.context.bounded_wait_probe(0.2)     # waits 0.2 s for a flag that nothing sets, then gives up
    assert time.time() - t0 < 5
    assert buf.context.status_code() == 2
    with pytest.raises(deep_ep.EPException):
        buf.context.check_status()
    # the context of the process is still usable: clear the sticky status and run a collective
    buf.context.clear_status()
    buf.barrier(with_cpu_sync=True)
    x = torch.ones(4, device='cuda')
    assert x.sum().item() == 4
    buf.destroy()


@pytest.mark.gpu
def test_bounded_wait_reports_status(master_port):
    run_distributed(_timeout_worker, 1, master_port, 'nccl')


def _absent_peer_worker(rank, world):
    """One rank never enters a barrier: the other one's wait gives up after its one-second budget, the exception names
    the absent rank and the site, and both ranks then release their buffers without a device-side barrier. Nothing
    faults, traps or spins past its budget; the failure is a rank that stays away, made on the host."""
    import time
    import torch.distributed as dist
    import deep_ep
    buf = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=64, hidden=256, num_topk=2, explicitly_destroy=True,
                           num_gpu_timeout_secs=1, num_cpu_timeout_secs=5)
    assert not buf.is_simulated
    buf.barrier(with_cpu_sync=True)                 # a healthy barrier first
    if rank == 0:
        t0 = time.time()
        with pytest.raises(deep_ep.EPException) as info:
            buf.barrier(with_cpu_sync=True)         # rank `world - 1` does not come
        took = time.time() - t0
        text = str(info.value)
        assert f'waiting for rank {world - 1}' in text and 'site 1' in text and 'rank barrier timeout' in text, text
        assert 0.5 < took < 5, took
    elif rank != world - 1:
        with pytest.raises(deep_ep.EPException):
            buf.barrier(with_cpu_sync=True)
    # the absent rank learns on the host that the others are done; no kernel of this buffer is in flight anywhere now
    torch.cuda.synchronize()
    dist.barrier()
    buf.abort(dist.group.WORLD)
    # the process and its CUDA context are still healthy: a new buffer over the same group works
    buf2 = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=64, hidden=256, num_topk=2, explicitly_destroy=True,
                            num_gpu_timeout_secs=10)
    buf2.barrier(with_cpu_sync=True)
    buf2.destroy()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_barrier_names_the_absent_rank_and_buffers_are_released_without_a_barrier(master_port, monkeypatch):
    monkeypatch.setenv('NCCL_NVLS_ENABLE', '0')     # plain peer loads and stores everywhere in a failure test
    run_distributed(_absent_peer_worker, 2, master_port, 'nccl', timeout_s=60)


# ---------------------------------------------------------------------------------------------------- events / streams
def _stream_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    calls = []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        a = torch.ones(1 << 20, device='cuda')
        torch.cuda._sleep(20_000_000)
        a.add_(1)
        ev = deep_ep.EventOverlap(deep_ep.EventHandle())
    ev.register_hook_after_wait(lambda: calls.append(torch.cuda.current_stream()) or a.sum())
    total = ev.current_stream_wait()
    assert total.item() == 2 * (1 << 20) and calls == [torch.cuda.current_stream()]
    assert ev.current_stream_wait() is None
    s1, s2 = deep_ep.comm.get_comm_stream(None), deep_ep.EPBuffer.get_comm_stream(None)
    assert s1.stream_id == s2.stream_id and s1 != torch.cuda.current_stream()

    # dispatch on a non-default stream, deferred, with the input freed and the allocator stressed in between
    group = dist.group.WORLD
    buf = deep_ep.EPBuffer(group, num_max_tokens_per_rank=256, hidden=512, num_topk=4, explicitly_destroy=True,
                           num_gpu_timeout_secs=10)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        x = torch.randn(256, 512, device='cuda', dtype=torch.bfloat16)
        expect = x.clone()
        idx = torch.rand(256, 8 * world, device='cuda').topk(4, dim=-1).indices
        ev = buf.dispatch(x, topk_idx=idx, num_experts=8 * world, do_expand=True, async_with_compute_stream=True,
                          defer_epilogue=True)
        del x
        junk = [torch.full((256, 512), float('nan'), device='cuda', dtype=torch.bfloat16) for _ in range(8)]
        recv_x, _, recv_w, handle = ev.current_stream_wait()
        assert recv_w is None
        stream.synchronize()
    meta = handle.recv_src_metadata
    mine = (meta[:, -2] // 256) == rank
    slots = meta[mine][:, :-2]
    tokens = (meta[mine][:, -2] % 256).long()
    for j in range(4):
        ok = slots[:, j] >= 0
        assert torch.equal(recv_x[slots[ok, j].long()], expect[tokens[ok]])
    del junk
    buf.destroy()


@pytest.mark.gpu
def test_events_and_streams(master_port):
    run_distributed(_stream_worker, _world(), master_port, 'nccl')


# ---------------------------------------------------------------------------------------------------- allocation
def _allocation_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    plan = deep_ep.BufferAllocator()
    a = plan.allocate((1024, 64), torch.bfloat16)
    b = plan.allocate((333,), torch.int32)
    groups = [group]
    if world >= 4:                      # the same storage registered with a second group
        pairs = [dist.new_group([i, i + 1]) for i in range(0, world, 2)]
        groups.append(pairs[rank // 2])
    bucket = deep_ep.BucketBuffer(groups, plan, explicitly_destroy=True, num_gpu_timeout_secs=10)
    assert a.is_cuda and b.is_cuda and a.shape == (1024, 64)
    base = bucket.storage.data_ptr()
    assert a.data_ptr() == base and b.data_ptr() == base + (2 << 20)
    a.fill_(rank)
    assert bucket.storage[:16].view(torch.bfloat16)[0].item() == rank
    bucket.destroy()

    lb_plan = deep_ep.BufferAllocator()
    w = lb_plan.allocate((2, 128, 128), torch.bfloat16)
    ep = deep_ep.EPBuffer(group, num_max_tokens_per_rank=64, hidden=256, num_topk=2,
                          lb_allocation_plan_or_num_bytes=lb_plan, explicitly_destroy=True)
    assert w.is_cuda and ep.num_lb_bytes == 2 << 20
    assert w.data_ptr() == ep.runtime.lb_storage.data_ptr()
    ep.print_memory_usage()
    ep.destroy()


@pytest.mark.gpu
def test_allocation_plans(master_port):
    run_distributed(_allocation_worker, _world(), master_port, 'nccl')


# ---------------------------------------------------------------------------------------------------- bucket all-gather
def _all_gather_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    groups = [group]
    if world >= 4:
        pairs = [dist.new_group([i, i + 1]) for i in range(0, world, 2)]
        groups.append(pairs[rank // 2])
    bucket = deep_ep.BucketBuffer(groups, 64 << 20, explicitly_destroy=True, num_gpu_timeout_secs=10)
    torch.manual_seed(5)
    for g in groups:
        size, grank = g.size(), g.rank()
        kw = dict(group=g) if len(groups) > 1 else {}
        # out-of-place, NaN-poisoned destination, odd sizes and unaligned addresses
        for numel, dtype, offset in [(4096, torch.bfloat16, 0), (1001, torch.float32, 4), (777, torch.uint8, 3), (1 << 20, torch.bfloat16, 128)]:
            src = (torch.arange(numel, device='cuda') % 251 + grank).to(dtype)
            nbytes = numel * src.element_size()
            dst = bucket.storage.narrow(0, 1 << 20, 0)   # placeholder to keep names local
            region = bucket.storage.narrow(0, (1 << 20) + offset, size * nbytes)
            region.fill_(255)
            dst = region.view(dtype)
            out = bucket.all_gather(src, dst, **kw).wait()
            torch.cuda.synchronize()
            assert out.data_ptr() == dst.data_ptr() and out.dim() == 1
            expect = torch.cat([(torch.arange(numel, device='cuda') % 251 + r).to(dtype) for r in range(size)])
            assert torch.equal(out, expect)
        # in-place: my shard already sits in the gathered tensor
        numel = 2048
        whole = bucket.storage.narrow(0, 8 << 20, size * numel * 4).view(torch.float32)
        whole.fill_(float('nan'))
        whole[grank * numel:(grank + 1) * numel] = grank + 0.5
        out = bucket.all_gather(whole[grank * numel:(grank + 1) * numel], **kw).wait()
        torch.cuda.synchronize()
        assert torch.equal(out, torch.arange(size, device='cuda').repeat_interleave(numel) + 0.5)
        # a full batch of 64 buckets of different sizes
        srcs, dsts, off = [], [], 16 << 20
        for i in range(64):
            n = 64 * (i + 1)
            srcs.append(torch.full((n,), float(grank * 100 + i), device='cuda', dtype=torch.bfloat16))
            dsts.append(bucket.storage.narrow(0, off, size * n * 2).view(torch.bfloat16))
            off += (size * n * 2 + 255) // 256 * 256
        handle = bucket.all_gather(srcs, dsts, **kw)
        outs = handle.wait()
        torch.cuda.synchronize()
        for i, o in enumerate(outs):
            # (values beyond 256 are not exact in bf16: round the expectation the same way)
            expect = (torch.arange(size, device='cuda').float() * 100 + i).to(torch.bfloat16).float()
            assert torch.equal(o.view(size, -1)[:, 0].float(), expect)
        bucket.barrier(**kw)
    for c in bucket.contexts:
        assert c.status_code() == 0
    bucket.destroy()


@pytest.mark.gpu
def test_bucket_all_gather(master_port):
    run_distributed(_all_gather_worker, _world(), master_port, 'nccl')


def _session_worker(rank, world):
    import random
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    bucket = deep_ep.BucketBuffer(group, 128 << 20, explicitly_destroy=True, num_gpu_timeout_secs=10)
    original = bucket.all_gather
    with bucket.session() as session:
        src = torch.full((1000,), float(rank), device='cuda')
        user_dst = torch.empty(world * 1000, device='cuda')                  # lives outside the storage
        out = bucket.all_gather(src, user_dst).wait()
        assert out is user_dst
        assert torch.equal(out.view(world, -1)[:, 0], torch.arange(world, device='cuda').float())
        reg = session.allocate((world, 512), torch.bfloat16)
        reg[rank] = rank + 1
        out2 = bucket.all_gather(reg[rank]).wait()
        assert torch.equal(out2.view(world, -1)[:, 0].float(), torch.arange(world, device='cuda').float() + 1)
        out3 = bucket.all_gather(src).wait()                                  # unregistered src, no dst
        assert torch.equal(out3.view(world, -1)[:, 5], torch.arange(world, device='cuda').float())
        with pytest.raises(AssertionError):
            with bucket.session():
                pass
    assert bucket.all_gather == original
    try:
        with bucket.session():
            raise RuntimeError('boom')
    except RuntimeError:
        pass
    assert bucket.all_gather == original and bucket._active_session is None

    # randomised schedule: 48 gathers with at most 4 in flight, mixed registered / external outputs
    rng = random.Random(1)
    with bucket.session() as session:
        inflight = []
        for i in range(48):
            n = rng.choice([256, 4096, 65536])
            src = torch.full((n,), float(rank + i), device='cuda', dtype=torch.bfloat16)
            dst = torch.empty(world * n, device='cuda', dtype=torch.bfloat16) if rng.random() < 0.5 else None
            inflight.append((i, bucket.all_gather(src, dst) if dst is not None else bucket.all_gather(src)))
            if len(inflight) >= 4 or session.offset > (96 << 20):
                for j, h in inflight:
                    out = h.wait()
                    assert torch.equal(out.view(world, -1)[:, 0].float(), torch.arange(world, device='cuda').float() + j)
                inflight.clear()
                if session.offset > (96 << 20):
                    bucket.barrier()
                    session.offset = 0
        for j, h in inflight:
            out = h.wait()
            assert torch.equal(out.view(world, -1)[:, 0].float(), torch.arange(world, device='cuda').float() + j)
    torch.cuda.synchronize()
    bucket.destroy()


@pytest.mark.gpu
def test_bucket_sessions(master_port):
    run_distributed(_session_worker, _world(), master_port, 'nccl')


# ---------------------------------------------------------------------------------------------------- pipeline
def _reduce_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    bucket = deep_ep.BucketBuffer(group, 64 << 20, explicitly_destroy=True, num_gpu_timeout_secs=10)

    def data(r, n, dtype):                       # what rank r holds: reproducible on every rank
        g = torch.Generator(device='cuda').manual_seed(1000 + r)
        return torch.randn(n, device='cuda', generator=g).to(dtype)

    def expected(n, dtype, scale):               # fp32 sum in rank order, scaled, rounded once
        acc = torch.zeros(n, device='cuda')
        for r in range(world):
            acc += data(r, n, dtype).float()
        return (acc * scale).to(dtype)

    with bucket.session() as session:
        specs = [(world * 8 * 1000, torch.bfloat16), (world * 4 * 33, torch.float32), (world * 8 * 4096, torch.float16),
                 (world * 8 * 70001, torch.bfloat16)]
        tensors = [session.allocate((n,), dt) for n, dt in specs]
        # ---- all-reduce: every rank ends with the same bits
        for t, (n, dt) in zip(tensors, specs):
            t.copy_(data(rank, n, dt))
        out = bucket.all_reduce(tensors, scale=0.5).wait()
        for o, t, (n, dt) in zip(out, tensors, specs):
            assert o.data_ptr() == t.data_ptr()
            assert torch.equal(o, expected(n, dt, 0.5)), f'all_reduce {dt} {n}'
        # ---- reduce-scatter: my shard is reduced, the rest of my tensor is untouched
        for t, (n, dt) in zip(tensors, specs):
            t.copy_(data(rank, n, dt))
        shards = bucket.reduce_scatter(tensors).wait()
        for sh, t, (n, dt) in zip(shards, tensors, specs):
            m = n // world
            assert sh.numel() == m and sh.data_ptr() == t.data_ptr() + rank * m * t.element_size()
            assert torch.equal(sh, expected(n, dt, 1.0)[rank * m:(rank + 1) * m]), f'reduce_scatter {dt} {n}'
            mine = data(rank, n, dt)
            keep = torch.ones(n, dtype=torch.bool, device='cuda')
            keep[rank * m:(rank + 1) * m] = False
            assert torch.equal(t[keep], mine[keep])
        # ---- a single tensor comes back as a tensor; misaligned sizes are rejected
        tensors[1].copy_(data(rank, specs[1][0], specs[1][1]))
        single = bucket.all_reduce(tensors[1]).wait()
        assert isinstance(single, torch.Tensor) and torch.equal(single, expected(specs[1][0], specs[1][1], 1.0))
        odd = session.allocate((world * 4 + 1,), torch.float32)
        with pytest.raises(deep_ep.EPException):
            bucket.all_reduce(odd)
        # tensors outside the storage are staged by the session: all-reduce stays in place for the caller,
        # reduce-scatter hands back the reduced shard
        n, dt = specs[0]
        user = data(rank, n, dt)
        out = bucket.all_reduce(user, scale=0.5).wait()
        assert out is user and torch.equal(user, expected(n, dt, 0.5))
        user2 = data(rank, n, dt)
        shard = bucket.reduce_scatter(user2).wait()
        assert torch.equal(shard, expected(n, dt, 1.0)[rank * (n // world):(rank + 1) * (n // world)])
        assert torch.equal(user2, data(rank, n, dt))
    outside = torch.zeros(world * 16, device='cuda')
    with pytest.raises(deep_ep.EPException):
        bucket.reduce_scatter(outside)                       # outside a session only registered tensors are accepted
    torch.cuda.synchronize()
    bucket.destroy()


@pytest.mark.gpu
def test_bucket_reduce_scatter_all_reduce(master_port):
    run_distributed(_reduce_worker, _world(), master_port, 'nccl')


def _pp_worker(rank, world, transport='nvlink'):
    import random
    import torch.distributed as dist
    import deep_ep
    inflight = 3
    pp = deep_ep.PPBuffer(dist.group.WORLD, 1 << 20, inflight, explicitly_destroy=True, num_gpu_timeout_secs=10,
                          transport=transport)
    nxt, prv = (rank + 1) % world, (rank + world - 1) % world
    # ring: everybody sends `inflight` messages ahead to the next rank, then receives them from the previous one
    msgs = [torch.full((1000 + 37 * i,), float(rank * 10 + i), device='cuda') for i in range(inflight)]
    for m in msgs:
        pp.send(m, nxt)
    for i in range(inflight):
        out = torch.empty(1000 + 37 * i, device='cuda')
        pp.recv(out, prv)
        assert torch.equal(out, torch.full_like(out, float(prv * 10 + i)))
    # both directions at once, random schedule honouring the in-flight limit (same seed on every rank)
    rng = random.Random(3)
    sent = {0: 0, 1: 0}
    received = {0: 0, 1: 0}
    for _ in range(60):
        # 0: data flows towards next ranks, 1: towards previous ranks (the two are one channel when world <= 2)
        d = rng.randrange(2) if world > 2 else 0
        if sent[d] - received[d] < inflight and rng.random() < 0.6:
            x = torch.full((4096,), float(100 * d + sent[d] + rank), device='cuda', dtype=torch.bfloat16)
            pp.send(x, nxt if d == 0 else prv)
            sent[d] += 1
        elif received[d] < sent[d]:
            src = prv if d == 0 else nxt
            out = torch.empty(4096, device='cuda', dtype=torch.bfloat16)
            pp.recv(out, src)
            assert out[0].item() == float(100 * d + received[d] + src)
            received[d] += 1
    for d in (0, 1):
        while received[d] < sent[d]:
            src = prv if d == 0 else nxt
            out = torch.empty(4096, device='cuda', dtype=torch.bfloat16)
            pp.recv(out, src)
            assert out[0].item() == float(100 * d + received[d] + src)
            received[d] += 1
    torch.cuda.synchronize()
    assert pp.context.status_code() == 0
    with pytest.raises(Exception):
        pp.send(torch.zeros(2 << 20, device='cuda', dtype=torch.uint8), nxt)      # larger than a slot
    if world > 3:
        with pytest.raises(Exception):
            pp.send(msgs[0], (rank + 2) % world)                                   # not a ring neighbour
    pp.destroy()


@pytest.mark.gpu
def test_pp_send_recv(master_port):
    world = _world()
    run_distributed(_pp_worker, world, master_port, 'nccl')


@pytest.mark.gpu
def test_pp_send_recv_over_nccl_point_to_point(master_port):
    """The same schedule through `PPBuffer(transport='nccl')`."""
    run_distributed(_pp_worker, _world(), master_port, 'nccl', ('nccl',), timeout_s=120)


# ---------------------------------------------------------------------------------------------------- engram
def _engram_worker(rank, world, use_fp8):
    import torch.distributed as dist
    import deep_ep
    from deep_ep.utils.math import per_token_cast_to_fp8
    group = dist.group.WORLD
    entries, hidden, max_tokens, per_token = [512, 384], 256, 64, 24
    dtype = torch.float8_e4m3fn if use_fp8 else torch.bfloat16
    packs = (hidden // 128) * 2 if use_fp8 else 0
    recv_bytes, storage_bytes = deep_ep.EngramBuffer.get_storage_size_hint(group, entries, hidden, max_tokens, per_token, dtype, packs)
    buf = deep_ep.EngramBuffer(group, recv_bytes, storage_bytes, explicitly_destroy=True, num_gpu_timeout_secs=10)
    assert deep_ep.EngramBuffer.get_theoretical_config(group, 2, max_tokens, per_token) == (0, 0, False)
    buf.set_config(entries, hidden, max_tokens, per_token, dtype, packs)
    torch.manual_seed(100 + rank)
    tables_bf16 = [torch.randn(n, hidden, device='cuda', dtype=torch.bfloat16) for n in entries]
    if use_fp8:
        quant = [per_token_cast_to_fp8(t) for t in tables_bf16]
        local = [q for q, _ in quant]
        local_sf = [s.view(torch.int16) for _, s in quant]
    else:
        local, local_sf = tables_bf16, None
    # global tables for the oracle
    def gather(t):
        out = [torch.empty_like(t.view(torch.uint8)) for _ in range(world)]
        dist.all_gather(out, t.contiguous().view(torch.uint8))
        return torch.cat(out).view(t.dtype) if t.dtype != torch.float8_e4m3fn else torch.cat(out)
    full = [gather(t) for t in local]
    full_sf = [gather(s) for s in local_sf] if use_fp8 else None
    buf.write(local, full_sf)

    torch.manual_seed(7)
    num_tokens = 50
    idx = torch.stack([torch.randint(0, world * n, (num_tokens, per_token), device='cuda', dtype=torch.int32) for n in entries])
    idx[0, 3, 5] = -1
    for col_major in ((False, True) if use_fp8 else (False,)):
        hooks = buf.fetch(idx, use_tma_aligned_col_major_sf=col_major)
        assert len(hooks) == 2
        for layer in (1, 0):                                   # hooks may be invoked in any order
            out = hooks[layer]()
            fetched, sf = out if use_fp8 else (out, None)
            torch.cuda.synchronize()
            flat = idx[layer].long().clamp(min=0).view(-1)
            ref = full[layer].view(torch.uint8)[flat].view(num_tokens, per_token * hidden * (1 if use_fp8 else 2))
            got = fetched.view(torch.uint8).view(num_tokens, -1)
            keep = torch.ones(num_tokens, per_token, dtype=torch.bool, device='cuda')
            if layer == 0:
                keep[3, 5] = False
            keep_b = keep.repeat_interleave(got.size(1) // per_token, dim=1)
            assert torch.equal(got[keep_b], ref[keep_b])
            if use_fp8:
                assert sf.stride() == ((1, num_tokens) if col_major else (per_token * packs, 1))
                ref_sf = full_sf[layer][flat].view(num_tokens, per_token * packs)
                keep_s = keep.repeat_interleave(packs, dim=1)
                assert torch.equal(sf[keep_s], ref_sf[keep_s])
    buf.destroy()


@pytest.mark.gpu
@pytest.mark.parametrize('use_fp8', [False, True])
def test_engram_fetch(master_port, use_fp8):
    run_distributed(_engram_worker, _world(), master_port, 'nccl', (use_fp8,))


# ---------------------------------------------------------------------------------------------------- load balancing
def _lb_worker(rank, world):
    import torch.distributed as dist
    import deep_ep
    group = dist.group.WORLD
    num_local, num_redundant, hidden = 4, 3, 256
    plan = deep_ep.BufferAllocator()
    red_w = plan.allocate((num_redundant, 8, hidden), torch.bfloat16)
    red_g = plan.allocate((num_redundant, hidden), torch.float32)
    ep = deep_ep.EPBuffer(group, num_max_tokens_per_rank=64, hidden=256, num_topk=2, lb_allocation_plan_or_num_bytes=plan,
                          explicitly_destroy=True, num_gpu_timeout_secs=10)
    torch.manual_seed(0)                                   # the mapping is identical on every rank
    mapping = torch.randint(-1, world * num_local, (world, num_redundant), dtype=torch.int32).cuda()
    weights = torch.stack([torch.full((8, hidden), float(rank * num_local + e)) for e in range(num_local)]).cuda().to(torch.bfloat16)
    red_w.fill_(-5)
    ep.lb_prefetch_weights(red_w, weights, mapping).current_stream_wait()
    torch.cuda.synchronize()
    for c in range(num_redundant):
        e = int(mapping[rank, c])
        assert torch.all(red_w[c] == (e if e >= 0 else -5)), f'slot {c} expected expert {e}'

    red_g.copy_(torch.arange(num_redundant).view(-1, 1).float().cuda() + 10 * rank + 1)
    grads = torch.ones(num_local, hidden, device='cuda')
    ep.lb_reduce_grads(red_g, grads, mapping).current_stream_wait()
    torch.cuda.synchronize()
    for e in range(num_local):
        expect = 1.0
        for r in range(world):
            for c in range(num_redundant):
                if int(mapping[r, c]) == rank * num_local + e:
                    expect += c + 10 * r + 1
        assert torch.all(grads[e] == expect), f'expert {e}: {grads[e, 0].item()} != {expect}'
    ep.destroy()


@pytest.mark.gpu
def test_lb_prefetch_and_reduce(master_port):
    run_distributed(_lb_worker, _world(), master_port, 'nccl')


def _nvls_worker(rank, world):
    """Symmetric allocation through the virtual-memory-management route with an NVLink multicast object (`EP_NVLS=1`):
    all-gather through `multimem.st`, all-reduce through `multimem.ld_reduce` + `multimem.st`."""
    import os
    import torch.distributed as dist
    os.environ['EP_NVLS'] = '1'
    import deep_ep
    group = dist.group.WORLD
    bucket = deep_ep.BucketBuffer(group, 64 << 20, explicitly_destroy=True, num_gpu_timeout_secs=10)
    assert bucket.contexts[0].has_multicast()
    with bucket.session() as session:
        n = 8 * 4096
        gathered = session.allocate((world, n), torch.bfloat16)
        gathered.fill_(float('nan'))
        gathered[rank] = rank + 1
        out = bucket.all_gather(gathered[rank]).wait()
        assert torch.equal(out.view(world, n)[:, 0].float(), torch.arange(world, device='cuda').float() + 1)
        assert torch.equal(out.view(world, n)[:, -1].float(), torch.arange(world, device='cuda').float() + 1)
        for dtype in (torch.float32, torch.bfloat16):
            t = session.allocate((world * 8 * 1000,), dtype)
            g = torch.Generator(device='cuda').manual_seed(7 + rank)
            mine = torch.randn(t.numel(), device='cuda', generator=g).to(dtype)
            t.copy_(mine)
            ref = mine.float().clone()
            dist.all_reduce(ref)
            got = bucket.all_reduce(t, scale=0.5).wait()
            # the switch chooses the order of the additions: equal up to rounding, not bitwise
            assert torch.allclose(got.float(), (ref * 0.5).to(dtype).float(), atol=0.05 * world, rtol=0.02), f'all_reduce {dtype}'
    torch.cuda.synchronize()
    bucket.destroy()


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.skipif(__import__('os').environ.get('EP_TEST_NEW_PATHS', '0') != '1',
                    reason='path that has not run on a GPU yet; set EP_TEST_NEW_PATHS=1 to try it')
def test_nvls_route_all_gather_and_all_reduce(master_port):
    run_distributed(_nvls_worker, _world(), master_port, 'nccl')
