"""The allocation-free routing-layout entry point, called the way a non-PyTorch caller would: through the
exported C symbol with raw device pointers. Its results must equal the regular entry point's, call after call,
because every call reuses the one scratch array that lives inside the library."""
import ctypes

import pytest
import torch


def _library():
    import deep_ep
    lib = ctypes.CDLL(deep_ep._C.__file__)
    fn = lib.deep_ep_dispatch_layout_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.deep_ep_noalloc_last_error.restype = ctypes.c_char_p
    lib.deep_ep_noalloc_wait_status.restype = ctypes.c_int
    lib.deep_ep_noalloc_wait_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    return lib, fn


@pytest.mark.gpu
def test_no_alloc_layout_matches_regular_entry_point_twice():
    from deep_ep.ops.layout import get_dispatch_layout
    lib, fn = _library()
    torch.cuda.set_device(0)
    torch.manual_seed(21)
    stream = torch.cuda.current_stream()
    # two calls in a row with different shapes: the second must not see anything of the first
    for num_tokens, num_topk, num_experts, num_ranks in [(5000, 6, 256, 8), (777, 8, 64, 4)]:
        idx = torch.rand(num_tokens, num_experts, device='cuda').topk(num_topk, dim=-1).indices
        idx = idx.masked_fill(torch.rand(idx.shape, device='cuda') < 0.1, -1).contiguous()
        slots = torch.full((num_tokens, num_topk), -7, dtype=torch.int32, device='cuda')
        per_rank = torch.full((num_ranks,), -7, dtype=torch.int32, device='cuda')
        per_expert = torch.full((num_experts,), -7, dtype=torch.int32, device='cuda')
        rc = fn(idx.data_ptr(), num_tokens, num_topk, num_experts, num_ranks, slots.data_ptr(), per_rank.data_ptr(),
                per_expert.data_ptr(), stream.cuda_stream)
        assert rc == 0, lib.deep_ep_noalloc_last_error().decode()
        # the kernel's own verdict: it ran to completion (a wait that gave up would leave a non-zero status word)
        device_status = ctypes.c_int(-1)
        assert lib.deep_ep_noalloc_wait_status(stream.cuda_stream, ctypes.byref(device_status)) == 0
        assert device_status.value == 0, lib.deep_ep_noalloc_last_error().decode()
        ref_slots, ref_rank, ref_expert = get_dispatch_layout(idx, num_experts, num_ranks)
        torch.cuda.synchronize()
        assert torch.equal(slots, ref_slots)
        assert torch.equal(per_rank, ref_rank)
        assert torch.equal(per_expert, ref_expert)


@pytest.mark.gpu
def test_no_alloc_layout_rejects_oversized_requests():
    lib, fn = _library()
    torch.cuda.set_device(0)
    buf = torch.zeros(64, dtype=torch.int64, device='cuda')
    out = torch.zeros(4096, dtype=torch.int32, device='cuda')
    args = (out.data_ptr(), out.data_ptr(), out.data_ptr(), None)
    assert fn(buf.data_ptr(), (1 << 20) + 1, 4, 16, 2, *args) == 1          # too many tokens
    assert b'num_tokens' in lib.deep_ep_noalloc_last_error()
    assert fn(buf.data_ptr(), 8, 4, 4096, 2, *args) == 1                    # too many experts
    assert fn(buf.data_ptr(), 8, 4, 128, 128, *args) == 1                   # too many ranks
    assert fn(buf.data_ptr(), 8, 64, 16, 2, *args) == 1                     # too many top-k positions
    assert fn(None, 8, 4, 16, 2, *args) == 1                                # null input
    assert fn(buf.data_ptr(), 0, 4, 16, 2, *args) == 1                      # an empty batch is rejected, outputs untouched
    assert int(out.abs().sum()) == 0
