"""The allocation-free C entry point of the quantised GEMV, called through its exported symbol.

Some users of this library cannot allocate device memory on the serving path (their host owns all of
it, or their plug-in contract forbids allocator calls), so `llaminar_gemv_noalloc` keeps its split-K
scratch in a fixed device array.  This test calls it twice in a row via ctypes with raw device pointers
and checks both results against the regular entry point, which uses torch-allocated scratch.
Collected last on purpose: a failure here cannot hide the other tests under `pytest -x`.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from llaminar_b200.ops import build
    build.load()                                  # builds if needed and loads libtorch dependencies first
    lib = ctypes.CDLL(build.so_path())
    fn = lib.llaminar_gemv_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p]
    lib.llaminar_gemv_noalloc_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("qt_name,m", [("Q4_K", 1), ("Q6_K", 3), ("Q8_0", 4)])
def test_noalloc_gemv_matches_regular_entry_point_twice(qt_name, m):
    from llaminar_b200 import ops
    from llaminar_b200.gguf import GGMLType, quantize
    lib = _lib()
    qt = GGMLType[qt_name]
    n, k = 1000, 2048                             # n is not a multiple of 128: exercises the padded tile
    g = torch.Generator(device="cuda").manual_seed(7)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.05
    pw = ops.pack_matrix(quantize(w, qt), qt, n, k)
    stream = torch.cuda.current_stream()
    for call in range(2):
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        ref = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ops.gemv(pw, x, ref, scratch=ops.scratch_for("cuda"))
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.llaminar_gemv_noalloc(pw.data.data_ptr(), pw.fmt, n, k, x.data_ptr(), m, out.data_ptr(), stream.cuda_stream)
        assert rc == 0, lib.llaminar_gemv_noalloc_error().decode()
        torch.cuda.synchronize()
        rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
        assert rel < 2e-2, (call, rel)
        assert torch.isfinite(out.float()).all()


def test_noalloc_gemv_rejects_oversize():
    lib = _lib()
    dummy = torch.zeros(16, device="cuda")
    p = dummy.data_ptr()
    assert lib.llaminar_gemv_noalloc(p, 0, 65536 + 128, 256, p, 1, p, None) != 0
    assert b"exceeds" in lib.llaminar_gemv_noalloc_error()
    assert lib.llaminar_gemv_noalloc(p, 0, 128, 256, p, 5, p, None) != 0
    assert lib.llaminar_gemv_noalloc(p, 0, 128, 100, p, 1, p, None) != 0
