"""Run-time compiled kernels: the cubin cache and the specialised FP8 quantiser."""
import os

import pytest
import torch


@pytest.mark.gpu
@pytest.mark.parametrize('hidden', [128, 1024, 7168])
def test_jit_quant_matches_torch_bitwise(hidden, tmp_path):
    os.environ['EP_JIT_CACHE_DIR'] = str(tmp_path)
    from deep_ep.ops.quant import per_token_cast_to_fp8
    from deep_ep.utils.math import per_token_cast_to_fp8 as ref_cast
    torch.manual_seed(0)
    x = torch.randn(333, hidden, device='cuda', dtype=torch.bfloat16) * 5
    x[7] = 0
    q, sf = per_token_cast_to_fp8(x)
    rq, rsf = ref_cast(x)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8))
    assert torch.equal(sf, rsf)
    assert any(f.endswith('kernel.cubin') for _, _, files in os.walk(tmp_path) for f in files)


def test_jit_cache_key_and_errors(tmp_path):
    """Compiles without a GPU: nvcc cross-compiles for sm_100a; identical sources hit the cache, broken ones raise."""
    import deep_ep
    os.environ['EP_JIT_CACHE_DIR'] = str(tmp_path)
    src = 'extern "C" __global__ void k(int* p) { if (p) p[0] = 1; }\n'
    a = deep_ep._C.jit_compile('unit', src)
    stamp = os.path.getmtime(a)
    b = deep_ep._C.jit_compile('unit', src)
    assert a == b and os.path.getmtime(b) == stamp
    c = deep_ep._C.jit_compile('unit', src + '// changed\n')
    assert c != a
    with pytest.raises(deep_ep.EPException):
        deep_ep._C.jit_compile('broken', 'this is not CUDA')


def test_jit_cache_searches_every_root_and_writes_the_first(tmp_path):
    """`EP_JIT_CACHE_DIR=a:b`: a hit in any root is used, a miss is compiled into the first root."""
    import deep_ep
    first, second = tmp_path / 'first', tmp_path / 'second'
    src = 'extern "C" __global__ void k2(int* p) { if (p) p[0] = 2; }\n'
    saved = os.environ.get('EP_JIT_CACHE_DIR')
    try:
        os.environ['EP_JIT_CACHE_DIR'] = str(second)
        in_second = deep_ep._C.jit_compile('roots', src)
        assert in_second.startswith(str(second))
        os.environ['EP_JIT_CACHE_DIR'] = f'{first}:{second}'
        assert deep_ep._C.jit_cache_roots() == [str(first), str(second)]
        assert deep_ep._C.jit_compile('roots', src) == in_second                 # found behind the first root
        fresh = deep_ep._C.jit_compile('roots', src + '// other\n')
        assert fresh.startswith(str(first))                                       # misses go to the first root
        assert deep_ep._C.jit_launch_timeout_secs() == 300
    finally:
        if saved is None:
            os.environ.pop('EP_JIT_CACHE_DIR', None)
        else:
            os.environ['EP_JIT_CACHE_DIR'] = saved


def test_jit_paths_with_spaces_and_shell_characters(tmp_path):
    """The compiler is started as a process with an argument vector, not through a shell: a cache directory whose name
    has spaces, quotes and a `;` compiles, and nothing from the name is executed."""
    import deep_ep
    root = tmp_path / "cache dir; touch 'owned' $(echo x)"
    saved = os.environ.get('EP_JIT_CACHE_DIR')
    try:
        os.environ['EP_JIT_CACHE_DIR'] = str(root)
        cubin = deep_ep._C.jit_compile('spaces', 'extern "C" __global__ void k3(int* p) { if (p) p[0] = 3; }\n')
        assert cubin.startswith(str(root)) and os.path.getsize(cubin) > 0
        assert not (tmp_path / 'owned').exists() and not os.path.exists('owned')
    finally:
        if saved is None:
            os.environ.pop('EP_JIT_CACHE_DIR', None)
        else:
            os.environ['EP_JIT_CACHE_DIR'] = saved


def test_jit_concurrent_compilation_of_one_entry(tmp_path):
    """Ranks of a job compile the same kernel at the same moment into one cache: every process gets the same complete
    cubin (source and result are published with renames), and no temporary file stays behind."""
    import subprocess
    import sys
    program = (
        "import os, sys, deep_ep\n"
        "src = 'extern \"C\" __global__ void k4(float* p) { if (p) p[threadIdx.x] *= 2.f; }\\n'\n"
        "path = deep_ep._C.jit_compile('racing', src)\n"
        "print(path, os.path.getsize(path))\n")
    env = dict(os.environ, EP_JIT_CACHE_DIR=str(tmp_path))
    children = [subprocess.Popen([sys.executable, '-c', program], env=env, stdout=subprocess.PIPE, text=True) for _ in range(4)]
    answers = [child.communicate(timeout=600)[0].split() for child in children]
    assert all(child.returncode == 0 for child in children)
    assert len({tuple(answer) for answer in answers}) == 1 and int(answers[0][1]) > 0
    leftovers = [f for _, _, files in os.walk(tmp_path) for f in files if '.tmp.' in f]
    assert not leftovers


@pytest.mark.parametrize('kernel', ['dispatch', 'expand', 'combine', 'reduce'])
def test_specialised_ep_kernels_cross_compile(kernel, tmp_path):
    """Every shape-specialised EP kernel compiles for sm_100a (no GPU needed) from the three-line translation unit
    that the run-time specialiser generates."""
    import deep_ep
    os.environ['EP_JIT_CACHE_DIR'] = str(tmp_path)
    source = deep_ep._C.jit_specialized_source(kernel, 8, 6, 7168, 256)
    assert '<8, 6, 7168' in source and 'ep_specialized' in source
    cubin = deep_ep._C.jit_compile(f'ep_{kernel}_test', source)
    assert os.path.getsize(cubin) > 0


def _specialised_worker(rank, world_size, cache_dir):
    import torch.distributed as dist
    import deep_ep
    from ep_check import check_dispatch_combine
    os.environ['EP_JIT_CACHE_DIR'] = cache_dir
    dev = torch.device('cuda')
    torch.manual_seed(40 + rank)
    tokens, hidden, topk, experts = 200, 1024, 6, 16 * world_size
    with torch.inference_mode():
        buffer = deep_ep.EPBuffer(dist.group.WORLD, num_max_tokens_per_rank=tokens, hidden=hidden, num_topk=topk,
                                  explicitly_destroy=True, num_gpu_timeout_secs=10, num_cpu_timeout_secs=30)
        x = torch.randn(tokens, hidden, device=dev, dtype=torch.bfloat16)
        idx = torch.rand(tokens, experts, device=dev).topk(topk, dim=-1).indices
        w = torch.rand(tokens, topk, device=dev)
        results = []
        for specialised in (False, True):
            deep_ep._C.set_jit_specialization(specialised)
            assert deep_ep._C.get_jit_specialization() == specialised
            (rx, rsf), _, rw, handle, _ = buffer.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=experts, expert_alignment=128,
                                                         do_expand=True, do_zero_padding=True, fused_fp8_quant=True)
            y = torch.randn(rx.size(0), hidden, device=dev, dtype=torch.bfloat16, generator=torch.Generator(device=dev).manual_seed(5))
            combined, cw, _ = buffer.combine(y, handle, topk_weights=rw)
            torch.cuda.synchronize()
            buffer.runtime.check_status()
            slots = handle.recv_src_metadata[:, :-2]
            flat = slots[slots >= 0].long()
            results.append((rx.view(torch.uint8)[flat].clone(), rsf[flat].clone(), rw[flat].clone(), handle.recv_src_metadata.clone(),
                            combined.clone(), cw.clone()))
        for generic, special in zip(*results):
            assert torch.equal(generic, special), 'a shape-specialised EP kernel changes the result'
        # the specialised kernels were really built and loaded: four cubins in the cache
        cubins = [f for _, _, files in os.walk(cache_dir) for f in files if f == 'kernel.cubin']
        assert len(cubins) >= 4, cubins
        # and the full correctness sweep passes with them
        check_dispatch_combine(buffer, tokens, hidden, topk, experts, do_cpu_sync=True, defer=True, quick=True)
        deep_ep._C.set_jit_specialization(False)
        buffer.destroy()


@pytest.mark.gpu
def test_specialised_ep_kernels_match_generic_bitwise(master_port, tmp_path):
    from dist_utils import run_distributed
    world = min(torch.cuda.device_count(), 2)
    run_distributed(_specialised_worker, world, master_port, 'nccl', (str(tmp_path),))


def test_bounds_checked_build_compiles_and_its_predicate(tmp_path, monkeypatch):
    """`EP_DEBUG=1` makes the run-time compiler build the kernels with their bounds checks (a different cubin from the
    plain build), and the predicate those checks apply accepts exactly the aligned ranges inside the landing area."""
    import deep_ep
    monkeypatch.setenv('EP_JIT_CACHE_DIR', str(tmp_path))
    source = deep_ep._C.jit_specialized_source('dispatch', 2, 4, 1024, 16)
    plain = deep_ep._C.jit_compile('ep_dispatch_dbg_test', source)
    monkeypatch.setenv('EP_DEBUG', '1')
    checked = deep_ep._C.jit_compile('ep_dispatch_dbg_test', source)
    assert plain != checked and os.path.getsize(checked) > os.path.getsize(plain)
    ok = deep_ep._C.landing_range_ok
    assert ok(0, 7456, 7456 * 4) and ok(7456 * 3, 7456, 7456 * 4)
    assert not ok(7456 * 3 + 16, 7456, 7456 * 4)          # runs past the end
    assert not ok(-16, 32, 1024) and not ok(8, 32, 1024) and not ok(0, 24, 1024) and not ok(0, 0, 1024)
