"""The allocation-free expert-offsets entry point, called through its exported C symbol.

Who needs it: callers that must not allocate device memory when they ask for routing offsets (every byte already
belongs to a framework's caching allocator, a serving process forbids cudaMalloc after start-up, or the hidden device
synchronisation of cudaMalloc is unacceptable on the path).  The variant keeps its counters in an array inside the
library image, so its results must equal those of HcclMoeExpertOffsets, call after call, although all calls share
that array.  This file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "hccl_b200" / "lib" / "libhccl_b200.so"


def _symbols():
    lib = ctypes.CDLL(str(LIB))
    args = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]
    for name in ("HcclMoeExpertOffsets", "HcclMoeExpertOffsetsNoAlloc"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = args
    return lib.HcclMoeExpertOffsets, lib.HcclMoeExpertOffsetsNoAlloc


def _call(fn, idx, n_experts, out):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(ctypes.c_void_p(idx.data_ptr()), idx.numel(), n_experts, ctypes.c_void_p(out.data_ptr()), stream)


def test_no_alloc_matches_allocating_entry_point_on_consecutive_calls():
    torch.cuda.set_device(0)
    reference, no_alloc = _symbols()
    # first call on the device (does the one-time address lookup), outside any stream capture
    for call, (tokens, topk, experts) in enumerate([(8192, 8, 256), (8192, 8, 256), (333, 3, 4096), (50000, 4, 17)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        idx = torch.randint(-2, experts, (tokens, topk), device="cuda", generator=g, dtype=torch.int32)
        want = torch.full((experts + 1,), -1, dtype=torch.int32, device="cuda")
        got = torch.full((experts + 1,), -1, dtype=torch.int32, device="cuda")
        assert _call(reference, idx, experts, want) == 0
        assert _call(no_alloc, idx, experts, got) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: offsets differ"      # integer results: exact
        # and both agree with plain PyTorch
        ref = torch.zeros(experts + 1, dtype=torch.int64, device="cuda")
        ref[1:] = torch.bincount(idx[idx >= 0].long(), minlength=experts).cumsum(0)
        assert torch.equal(got.long(), ref)


def test_no_alloc_rejects_more_experts_than_its_array_holds():
    torch.cuda.set_device(0)
    _, no_alloc = _symbols()
    idx = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.zeros(5000, dtype=torch.int32, device="cuda")
    assert _call(no_alloc, idx, 4097, out) == 1       # HCCL_E_PARA, nothing launched
    assert _call(no_alloc, idx, 0, out) == 1
    assert _call(no_alloc, idx, 4096, out) == 0       # the maximum itself is fine
    torch.cuda.synchronize()
    assert int(out[4096]) == 16 and int(out[1]) == 16
