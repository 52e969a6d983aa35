"""GPU: the allocation-free weight quantiser against the regular one, through the C ABI.

``nvfp4_quantize_weight_static`` exists for callers that may not allocate device memory at
the moment of the call (a stream being captured, a serving loop that cannot take the
device-wide stall of a cudaMalloc, a process whose memory is fully handed to its own pool).
Its scratch is a fixed array inside the library, shared by every call on the device and
keeping the previous call's contents, so the check is made twice in a row with different
inputs: the second call must not see anything of the first.  The file sorts last on purpose:
if it fails, a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from nvfp4_gemm import _C

pytestmark = pytest.mark.gpu


def _quantise(fn, w):
    e, n, k = w.shape
    b = torch.full((e * n, k // 2), 0x55, dtype=torch.int8, device=w.device)
    sfb = torch.full((e * k // 64, n), -1, dtype=torch.int32, device=w.device)
    gw = torch.full((e,), float("nan"), dtype=torch.float32, device=w.device)
    rc = fn(w.data_ptr(), 0 if w.dtype == torch.bfloat16 else 1, e, n, k, b.data_ptr(), sfb.data_ptr(), gw.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _C.lib().nvfp4_last_error().decode()
    torch.cuda.synchronize()
    return b, sfb, gw


def test_static_scratch_quantiser_matches_regular_entry_point():
    assert torch.cuda.is_available()
    lib = _C.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(7)
    # first call: 5 experts with large values; second call: 3 experts with small ones -- stale
    # maxima from the first call would change every scale of the second
    cases = [(torch.randn(5, 192, 256, generator=g) * 3.0).to(torch.bfloat16),
             (torch.randn(3, 128, 128, generator=g) * 0.01)]
    import oracle
    for w in cases:
        w = w.to(dev)
        want = _quantise(lib.nvfp4_quantize_weight, w)
        got = _quantise(lib.nvfp4_quantize_weight_static, w)
        for x, y in zip(got, want):
            assert torch.equal(x, y)               # bit for bit, as for every other weight test
        for x, y in zip(got, oracle.quantize_weight(w.cpu())):
            assert torch.equal(x.cpu(), y)         # and against the CPU oracle directly, not only against the sibling entry


def test_static_scratch_quantiser_leaves_device_memory_as_it_found_it():
    """The point of the entry: no device allocation at call time.  With the outputs allocated beforehand (and one call
    made, so that the library has looked up its array's address), the free device memory the driver reports is the same
    before and after a call, and no allocation goes through torch's allocator either."""
    lib = _C.lib()
    dev = torch.device("cuda:0")
    w = (torch.randn(4, 256, 512, generator=torch.Generator().manual_seed(8)) * 0.5).to(torch.bfloat16).to(dev)
    e, n, k = w.shape
    b = torch.empty(e * n, k // 2, dtype=torch.int8, device=dev)
    sfb = torch.empty(e * k // 64, n, dtype=torch.int32, device=dev)
    gw = torch.empty(e, dtype=torch.float32, device=dev)
    args = (w.data_ptr(), 0, e, n, k, b.data_ptr(), sfb.data_ptr(), gw.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert lib.nvfp4_quantize_weight_static(*args) == 0
    torch.cuda.synchronize()
    for attempt in range(3):                       # the figure is device-wide: allow for a neighbour's allocation in between
        free_before, _ = torch.cuda.mem_get_info(dev)
        torch_before = torch.cuda.memory_allocated(dev)
        assert lib.nvfp4_quantize_weight_static(*args) == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        if free_after == free_before:
            break
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_allocated(dev) == torch_before


def test_static_scratch_quantiser_rejects_too_many_experts():
    lib = _C.lib()
    rc = lib.nvfp4_quantize_weight_static(None, 0, 1025, 128, 64, None, None, None, None)
    assert rc == 1 and b"exceeds" in lib.nvfp4_last_error()
