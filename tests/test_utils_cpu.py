"""CPU unit tests of the Python utilities: math, allocator, event overlap, gate generators, parsers."""
import pytest
import torch

import deep_ep
from deep_ep.buffers.allocator import BufferAllocator
from deep_ep.utils.event import EventOverlap
from deep_ep.utils.gate import get_unbalanced_scores
from deep_ep.utils.math import align, calc_diff, ceil_div, count_bytes, per_token_cast_back, per_token_cast_to_fp8, safe_div
from deep_ep.utils.testing import KernelProfile, parse_num_bytes


def test_public_constants():
    assert deep_ep.get_num_allocation_alignment() == 2 << 20
    assert deep_ep.get_num_rdma_alignment() == 32 and deep_ep.get_num_tma_alignment() == 32
    assert deep_ep.topk_idx_t == torch.int64
    assert deep_ep.__version__.split('+')[0] == '1.0.0'      # the build appends '+<source revision>'


def test_math_helpers():
    assert ceil_div(7, 4) == 2 and align(7, 4) == 8 and align(8, 4) == 8
    assert safe_div(0, 0) == 0 and safe_div(3, 2) == 1.5
    with pytest.raises(ZeroDivisionError):
        safe_div(1, 0)
    a, b = torch.randn(4, 8), torch.randn(4, 8, dtype=torch.bfloat16)
    assert count_bytes(a, (b, None), [a]) == 2 * a.numel() * 4 + b.numel() * 2
    assert calc_diff(a, a) < 1e-12


@pytest.mark.parametrize('n', [128, 300, 7168])
def test_fp8_cast_roundtrip(n):
    x = torch.randn(16, n, dtype=torch.bfloat16)
    q, s = per_token_cast_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape and s.shape == (16, ceil_div(n, 128))
    assert s.dtype == torch.float32 and bool((s > 0).all())
    back = per_token_cast_back(q, s)
    assert calc_diff(back, x) < 2e-3
    # |q| never exceeds the e4m3 maximum and every group uses its full range
    assert q.float().abs().max() <= 448


def test_allocator_plan_and_materialize():
    plan = BufferAllocator()
    a = plan.allocate((3, 5), torch.float32)
    b = plan.allocate((7,), torch.int16)
    assert a.device.type == 'meta' and plan.num_bytes == 2 * (2 << 20)
    storage = torch.zeros(plan.num_bytes, dtype=torch.uint8)
    plan.materialize(storage)
    assert a.device.type == 'cpu' and a.shape == (3, 5) and b.shape == (7,)
    a.fill_(1.0)
    assert storage[:60].view(torch.float32).sum() == 15
    assert b.data_ptr() - storage.data_ptr() == 2 << 20
    assert [offset for _, offset in plan.allocations] == [0, 2 << 20] and plan.allocations[1][0] is b
    assert 'materialized' in plan.describe() and '(3, 5)' in plan.describe()
    with pytest.raises(AssertionError):
        plan.materialize(storage)
    with pytest.raises(AssertionError):
        plan.allocate((1,), torch.int8)


def test_event_overlap_hook_runs_once():
    calls = []
    ev = EventOverlap(deep_ep.EventHandle())
    ev.register_hook_after_wait(lambda: calls.append(1) or 'done')
    with pytest.raises(AssertionError):
        ev.register_hook_after_wait(lambda: None)
    assert ev.current_stream_wait() == 'done'
    assert ev.current_stream_wait() is None and calls == [1]
    ev2 = EventOverlap(deep_ep.EventHandle())
    ev2.register_hook_after_wait(lambda: calls.append(2))
    with ev2(release_handle=True):
        pass
    assert calls == [1, 2] and ev2.event is None


def test_parse_num_bytes_and_profile():
    assert parse_num_bytes('1G') == 1 << 30 and parse_num_bytes('64M') == 64 << 20
    assert parse_num_bytes('512KiB') == 512 << 10 and parse_num_bytes('1048576') == 1048576
    with pytest.raises(ValueError):
        parse_num_bytes('abc')
    p = KernelProfile(2000.0) + KernelProfile(1000.0)
    assert p.us == 3.0 and abs(p.gbps(3000) - 1.0) < 1e-9 and abs(p.tflops(3e6) - 1.0) < 1e-9


@pytest.mark.parametrize('ratio', [1.0, 2.0, 4.0])
@pytest.mark.parametrize('num_ranks,num_experts,num_topk', [(8, 64, 6), (8, 256, 8), (2, 16, 4), (16, 64, 4)])
def test_precise_gate_imbalance(ratio, num_ranks, num_experts, num_topk):
    torch.manual_seed(0)
    per_rank = num_experts // num_ranks
    upper = min(num_topk, num_ranks, int((num_ranks - 1) / ratio) + 1)
    if max(1, ceil_div(num_topk, per_rank)) > upper:
        pytest.skip('ratio not reachable for this shape')
    total = torch.zeros(num_ranks)
    for _ in range(num_ranks):
        scores = get_unbalanced_scores(4096, num_experts, num_ranks, num_topk, ratio, True, device=torch.device('cpu'))
        idx = scores.topk(num_topk, dim=-1).indices
        assert idx.unique(dim=1).shape == idx.shape
        total += torch.nn.functional.one_hot(idx // per_rank, num_ranks).any(dim=1).float().sum(0)
    practical = total[0] / total[1:].min().clamp(min=1)
    assert abs(practical - ratio) / ratio < 0.1
    if num_ranks > 2:
        assert total[1:].max() / total[1:].min().clamp(min=1) < 1.02


def test_random_gate_direction():
    torch.manual_seed(0)
    scores = get_unbalanced_scores(2048, 64, 8, 6, 2.0, False, device=torch.device('cpu'))
    hits = torch.nn.functional.one_hot(scores.topk(6, dim=-1).indices // 8, 8).any(dim=1).float().sum(0)
    assert 1.5 < (hits[0] / hits[1:].mean()).item() < 2.6


def test_per_block_fp8_cast_roundtrip():
    """128 x 128 block quantisation of expert weights: shapes, scale definition and reconstruction error."""
    from deep_ep.ops.grouped_gemm import per_block_cast_back, per_block_cast_to_fp8
    torch.manual_seed(0)
    w = torch.randn(3, 256, 384) * torch.tensor([0.01, 1.0, 30.0]).view(3, 1, 1)
    q, sf = per_block_cast_to_fp8(w)
    assert q.shape == w.shape and q.dtype == torch.float8_e4m3fn and sf.shape == (3, 2, 3) and sf.dtype == torch.float32
    blocks = w.reshape(3, 2, 128, 3, 128).abs().amax(dim=(2, 4))
    assert torch.allclose(sf, blocks / 448.0)
    back = per_block_cast_back(q, sf)
    # e4m3 keeps 3 mantissa bits: the error of an element is at most 1/16 of its block's maximum
    assert ((back - w).abs() <= blocks.repeat_interleave(128, 1).repeat_interleave(128, 2) / 16 + 1e-12).all()


def test_ue8m0_casts():
    """Power-of-two (UE8M0) scales: smallest power of two that keeps every value within the e4m3 range."""
    from deep_ep.ops.grouped_gemm import per_block_cast_to_fp8_ue8m0, per_token_cast_to_fp8_ue8m0, ue8m0_to_float
    torch.manual_seed(1)
    x = torch.randn(5, 384) * torch.tensor([1e-3, 0.1, 1.0, 50.0, 3000.0]).view(5, 1)
    q, sf = per_token_cast_to_fp8_ue8m0(x)
    assert q.dtype == torch.float8_e4m3fn and sf.dtype == torch.uint8 and sf.shape == (5, 3)
    scale = ue8m0_to_float(sf)
    amax = x.reshape(5, 3, 128).abs().amax(dim=2)
    assert (scale * 448 >= amax).all() and (scale * 224 < amax.clamp(min=1e-4)).all()      # tight within a factor of two
    assert torch.equal(torch.log2(scale), torch.log2(scale).round())
    back = q.float() * scale.repeat_interleave(128, dim=1)
    assert ((back - x).abs() <= amax.repeat_interleave(128, dim=1) / 8 + 1e-12).all()
    w = torch.randn(2, 256, 128)
    wq, wsf = per_block_cast_to_fp8_ue8m0(w)
    assert wq.shape == w.shape and wsf.shape == (2, 2, 1) and wsf.dtype == torch.uint8


def test_numa_binding_is_a_noop_without_a_gpu():
    import os
    from deep_ep.utils.envs import bind_to_device_numa_node
    before = os.sched_getaffinity(0)
    if not torch.cuda.is_available():
        assert bind_to_device_numa_node(0) is None
        assert os.sched_getaffinity(0) == before


def test_descriptor_exchange_between_processes_of_a_node():
    """The file-descriptor hand-over that the virtual-memory-management route of the symmetric allocation relies on."""
    import deep_ep
    assert deep_ep._C.fd_exchange_selftest()


def test_nvtx_range_decorator_is_transparent(monkeypatch):
    """Off: the function itself comes back. On: the call still returns its value and propagates exceptions (on a machine
    without CUDA the wrapper calls straight through)."""
    from deep_ep.utils.semantic import nvtx_range

    def f(a, b=2):
        return a + b
    monkeypatch.delenv('EP_NVTX', raising=False)
    assert nvtx_range('x')(f) is f
    monkeypatch.setenv('EP_NVTX', '1')
    wrapped = nvtx_range('x')(f)
    assert wrapped is not f and wrapped(1, b=3) == 4 and wrapped.__name__ == 'f'

    def boom():
        raise ValueError('boom')
    with pytest.raises(ValueError):
        nvtx_range('y')(boom)()


def test_build_time_environment_defaults_and_version(tmp_path, monkeypatch):
    """`setup.py` records the source revision and the build-time values of the JIT switches; importing the package turns
    them into defaults that the caller's environment overrides."""
    import importlib.util
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location('deep_ep_setup_probe', os.path.join(root, 'setup.py'))
    code = open(os.path.join(root, 'setup.py')).read().split('sources = [')[0]      # the helpers, without running setup()
    namespace = {'__file__': os.path.join(root, 'setup.py')}
    monkeypatch.setenv('EP_JIT_CACHE_DIR', '/baked/in/cache')
    monkeypatch.delenv('EP_JIT_DEBUG', raising=False)
    exec(compile(code, spec.origin, 'exec'), namespace)
    namespace['write_build_info'](str(tmp_path))
    info = {}
    exec(open(tmp_path / '_build_info.py').read(), info)
    assert info['persistent_envs'] == {'EP_JIT_CACHE_DIR': '/baked/in/cache'}
    assert info['version'].startswith('1.0.0+') and len(info['version']) > len('1.0.0+')
    # the installed defaults never override what the caller has set
    probe = ('import os, sys; sys.path.insert(0, %r); os.environ["EP_JIT_CACHE_DIR"] = "/mine"; import deep_ep; '
             'print(os.environ["EP_JIT_CACHE_DIR"], deep_ep.__version__)' % root)
    out = subprocess.check_output([sys.executable, '-c', probe]).decode().split()
    assert out[0] == '/mine' and out[1].startswith('1.0.0')


def test_parallel_mesh_layout_partitions_the_world():
    """For every factorisation of the world, each axis partitions the ranks into equal groups, a rank's three groups meet
    in that rank alone, EP groups are runs of neighbouring ranks, and coordinates and ranks convert both ways."""
    from hypothesis import given, settings, strategies as st
    from deep_ep.parallel import ParallelMesh

    @settings(max_examples=60, deadline=None)
    @given(st.integers(1, 4), st.integers(1, 4), st.integers(1, 4), st.data())
    def check(pp, dp, ep, data):
        world = pp * dp * ep
        rank = data.draw(st.integers(0, world - 1))
        mesh = ParallelMesh(ep_size=ep, pp_size=pp, dp_size=dp, world_size=world, rank=rank)
        mine = {}
        for axis, size in (('pp', pp), ('dp', dp), ('ep', ep)):
            groups = mesh.groups_of(axis)
            assert sorted(r for g in groups for r in g) == list(range(world)) and all(len(g) == size for g in groups)
            mine[axis] = set(mesh.axes[axis].ranks)
            assert rank in mine[axis]
        assert mine['pp'] & mine['dp'] & mine['ep'] == {rank}
        ep_ranks = sorted(mine['ep'])
        assert ep_ranks == list(range(ep_ranks[0], ep_ranks[0] + ep))            # neighbours: one NVSwitch domain
        assert mesh.rank_of(**mesh.coords) == rank and mesh.coords_of(rank) == mesh.coords
        assert mesh.coords_of(mesh.pp_next())['pp'] == (mesh.coords['pp'] + 1) % pp

    check()


def test_type_stubs_match_the_built_extension():
    """`deep_ep/_C.pyi` is what the stub generator makes of the built extension: a binding that is added or changed
    without regenerating the stubs fails here. The stubs must also be valid Python."""
    import ast
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location('generate_pyi', os.path.join(root, 'csrc', 'generate_pyi.py'))
    generator = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(generator)
    committed = open(os.path.join(root, 'deep_ep', '_C.pyi')).read()
    assert generator.generate() == committed, 'run `python csrc/generate_pyi.py`'
    declared = {node.name for node in ast.parse(committed).body if isinstance(node, (ast.FunctionDef, ast.ClassDef))}
    assert {'EPBuffer', 'PPBuffer', 'BucketBuffer', 'EngramBuffer', 'Context', 'barrier', 'calculate_ep_buffer_size'} <= declared


def test_ep_buffer_size_follows_the_wire_format():
    """`_C.calculate_ep_buffer_size` against a restatement of the wire format: a dispatch message is
    [payload][scale factors ^16][top-k indices i32][top-k weights f32][source index i32] ^16, one landing slot per source
    rank and token; a combine message is [bf16 payload][weights f32] ^16, one slot per master position (at most
    min(top-k, ranks)) and token; the buffer is the larger of the two areas, 2 MiB aligned. Every slot of the area passes
    the bounds predicate of the checked build and the first byte behind it does not."""
    from hypothesis import given, settings, strategies as st
    import deep_ep
    _C = deep_ep._C

    def up(x, a):
        return (x + a - 1) // a * a

    @settings(max_examples=80, deadline=None)
    @given(st.sampled_from([1, 2, 4, 8]), st.integers(1, 4096), st.sampled_from([128, 512, 2048, 7168]),
           st.integers(1, 8), st.booleans())
    def check(num_ranks, num_tokens, hidden, num_topk, fp8):
        payload = hidden if fp8 else 2 * hidden
        scale_bytes = (hidden + 31) // 32 * 2 if fp8 else 0            # room for the densest scale format (1 x 32, 2 bytes)
        dispatch_message = up(payload + up(scale_bytes, 16) + 8 * num_topk + 4, 16)
        combine_message = up(2 * hidden + 4 * num_topk, 16)
        dispatch_area = num_ranks * num_tokens * dispatch_message
        combine_area = min(num_topk, num_ranks) * num_tokens * combine_message
        expect = up(max(dispatch_area, combine_area), _C.get_num_allocation_alignment())
        assert _C.calculate_ep_buffer_size(num_ranks, num_tokens, hidden, num_topk, fp8) == expect
        last = (num_ranks * num_tokens - 1) * dispatch_message
        assert _C.landing_range_ok(last, dispatch_message, dispatch_area)
        assert not _C.landing_range_ok(last + dispatch_message, dispatch_message, dispatch_area)
        assert not _C.landing_range_ok(last + 8, dispatch_message, dispatch_area + 64)      # a bulk store starts on 16 bytes

    check()
    # top-k 0 reserves room for the largest top-k a buffer may be used with
    assert _C.calculate_ep_buffer_size(8, 4096, 7168, 0, True) >= _C.calculate_ep_buffer_size(8, 4096, 7168, 8, True)
