"""The allocation-free GEMV entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need a GEMV (a host application that hands a
plug-in a fixed set of buffers, code running under a hard memory cap, hot paths where cudaMalloc's device
synchronisation is not acceptable).  For them `b2_wq_gemv_noalloc` keeps the split-k scratch inside the library.  This
file checks it against the regular entry point on two calls in a row, and that oversized problems are refused.  It is
named to be collected last, so a run that stops at the first failure has already run every other test."""
import ctypes as C

import pytest
import torch

from agens_engine_b200 import _lib
from agens_engine_b200.ops import linear as L
from agens_engine_b200.utils import quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    lib = _lib.cuda_lib()
    fn = lib.b2_wq_gemv_noalloc
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_long, C.c_int, C.c_void_p,
                   C.c_long, C.c_void_p, C.c_void_p, C.c_char_p]
    fn.restype = C.c_int
    return fn


def test_no_alloc_entry_matches_regular_entry_twice():
    fn = _entry()
    torch.manual_seed(0)
    ws = L.GemvWorkspace(DEV)
    err = C.create_string_buffer(160)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (n, k, bits, m, ks) in enumerate([(256, 2048, 4, 3, 4), (512, 1024, 3, 8, 2)]):
        ql = quant.quantize(torch.randn(n, k) * 0.02, bits, 128)
        lin = L.WqLinear.from_quant(ql, DEV, ks=ks)
        lin.rb = 2
        x = torch.randn(m, k).to(torch.bfloat16).to(DEV)
        ref = L.gemv(lin, x, ws)                      # regular entry point, caller-provided scratch
        y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
        before = torch.cuda.memory_allocated()
        # the driver's own count of free device memory (sees cudaMalloc by anyone in the process, not only PyTorch's
        # allocator); checked on the second call, after the first one loaded the kernel image and resolved the symbol
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(lin.wq.data_ptr(), n, k, bits, 128, ks, x.data_ptr(), x.stride(0), m, y.data_ptr(), y.stride(0),
                status.data_ptr(), stream, err)
        torch.cuda.synchronize()
        assert rc == 0, err.value
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was taken during the call"
        assert int(status.item()) == 0
        assert torch.allclose(y.float(), ref.float(), rtol=2e-2, atol=1e-3), call
        assert torch.equal(y, ref), call               # same kernel, same schedule: identical bits


def test_no_alloc_entry_rejects_what_does_not_fit():
    fn = _entry()
    err = C.create_string_buffer(160)
    x = torch.zeros(32, 5120, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(32, 151936, dtype=torch.bfloat16, device=DEV)
    wq = torch.zeros(16, dtype=torch.uint8, device=DEV)
    rc = fn(wq.data_ptr(), 151936, 5120, 4, 128, 2, x.data_ptr(), 5120, 32, y.data_ptr(), 151936, None,
            torch.cuda.current_stream().cuda_stream, err)
    assert rc == 1 and b"built-in array holds" in err.value
    rc = fn(wq.data_ptr(), 100, 5120, 4, 128, 2, x.data_ptr(), 5120, 1, y.data_ptr(), 151936, None,
            torch.cuda.current_stream().cuda_stream, err)
    assert rc == 1 and b"bad argument" in err.value
