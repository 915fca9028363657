"""The allocation-free bias-gradient entry point, called through its exported C symbol.

Some users of the kernel library may not allocate device memory when they call it (they run
inside someone else's memory pool, or after all free memory was handed to an arena), so
``llmb_dbias_noalloc`` keeps its scratch inside the library.  The test loads the shared object
with ctypes, calls the symbol twice in a row (the second call meets the first call's leftovers in
the shared scratch) and compares with the regular entry point that takes caller scratch.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math

import pytest
import torch

from llm_mojo_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _symbol():
    L = ctypes.CDLL(_lib.lib_path())
    fn = L.llmb_dbias_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    ref = L.llmb_dbias
    ref.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                    ctypes.c_int, ctypes.c_void_p]
    ref.restype = ctypes.c_int
    nbytes = L.llmb_dbias_scratch_bytes
    nbytes.argtypes = [ctypes.c_int, ctypes.c_int]
    nbytes.restype = ctypes.c_longlong
    return fn, ref, nbytes


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    fn, ref, nbytes = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    code = 1 if dtype == torch.bfloat16 else 0
    g = torch.Generator().manual_seed(5)
    # two different shapes back to back: the second call reuses scratch the first one dirtied
    for rows, OC in ((4096 + 17, 3072), (777, 768)):
        dout = torch.randn(rows, OC, generator=g).to(dtype).cuda()
        want = torch.zeros(OC, device="cuda")
        scratch = torch.empty(int(nbytes(rows, OC)), dtype=torch.uint8, device="cuda")
        assert ref(want.data_ptr(), dout.data_ptr(), scratch.data_ptr(), scratch.numel(), rows, OC, code, stream) == 0
        got = torch.zeros(OC, device="cuda")
        fp32 = dout.float().sum(0)
        tol = 1e-3 * math.sqrt(rows)
        for call in (1, 2):              # dbias accumulates: after n calls it holds n times the column sums
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            assert fn(got.data_ptr(), dout.data_ptr(), rows, OC, code, stream) == 0
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before      # nothing went through torch's allocator
            if call == 2:                # the driver's own count of free bytes also sees a raw cudaMalloc; the first call
                assert torch.cuda.mem_get_info()[0] >= free_before      # on a device may still load the kernels' module
            assert torch.allclose(got, call * want, atol=tol, rtol=1e-3)
            assert torch.allclose(got, call * fp32, atol=2 * tol, rtol=1e-3)


def test_noalloc_rejects_misaligned_rows():
    fn, _, _ = _symbol()
    dout = torch.zeros(64 * 768 + 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(768, device="cuda")
    assert fn(out.data_ptr(), dout.data_ptr() + 2, 64, 768, 1, torch.cuda.current_stream().cuda_stream) == 2


def test_noalloc_rejects_sizes_beyond_its_scratch():
    fn, _, _ = _symbol()
    rows, OC = 128 * 512, 16384           # 128 slabs x 16384 columns > 2^20 floats
    dout = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")     # never touched: the call must refuse first
    out = torch.zeros(OC, device="cuda")
    assert fn(out.data_ptr(), dout.data_ptr(), rows, OC, 1, torch.cuda.current_stream().cuda_stream) == 2
    torch.cuda.synchronize()
    assert torch.all(out == 0)
