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
