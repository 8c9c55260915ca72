"""The allocation-free INT4 GEMV entry point, called through its exported C symbol.

Some users of the library may not allocate device memory where they need a projection
(a callback inside another runtime that forbids cudaMalloc, a process with a memory
budget fixed at start-up, a latency path that cannot afford the device synchronisation
an allocation implies).  For them `b2_gemv_int4_noalloc` carries its own split-K scratch
inside the library image.  Here it is checked against the regular entry point, which
gets its scratch from the caller, on two consecutive calls: the second call reuses the
built-in block with whatever the first one left in it.

Collected last on purpose (file name), and self-contained so that it also passes alone
in a fresh process.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, pk, x, out, stream):
    fn = lib.b2_gemv_int4_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_int, C.c_int, C.c_void_p]
    return fn(pk.qfrag.data_ptr(), pk.szfrag.data_ptr(), x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0),
              x.shape[0], pk.K, pk.N, 32 << pk.gshift, pk.off32 * 32, stream)


def test_noalloc_gemv_matches_regular_entry_point_twice():
    from mi50grad_b200.ops import kernels as K
    from mi50grad_b200.ops import lib as L
    from mi50grad_b200.ops.packing import pack_int4
    from mi50grad_b200.utils.quant import random_int4_linear
    lib = L.lib()
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(2024)
    Kd, N = 6144, 5120                       # row-parallel shape: split over 6 CTAs along K, so scratch is used
    lin = random_int4_linear(Kd, N, 128, gen)
    pk = pack_int4(lin, dev)
    assert pk.k_splits > 1
    req = lib.b2_gemv_int4_noalloc_required
    req.restype = C.c_size_t
    assert 4096 < req(3, Kd, N) <= (4 << 20)
    stream = torch.cuda.current_stream().cuda_stream
    dense = lin.dense()
    for call, rows in enumerate((3, 1)):
        x = torch.randn(rows, Kd, generator=gen).half().to(dev)
        ref = torch.zeros(rows, N, dtype=torch.float16, device=dev)
        K.gemv(pk, x, out=ref)                                   # existing entry point, caller-provided scratch
        out = torch.full((rows, N), float("nan"), dtype=torch.float16, device=dev)
        rc = _call_noalloc(lib, pk, x, out, stream)
        assert rc == 0, lib.b2_gemv_int4_noalloc_strerror(rc)
        torch.cuda.synchronize()
        rel = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert rel < 2e-3, f"call {call}: {rel}"
        gold = x.float().cpu() @ dense.t()
        assert float((out.float().cpu() - gold).abs().max() / gold.abs().max()) < 2e-3


def test_noalloc_gemv_rejects_oversized_and_bad_arguments():
    from mi50grad_b200.ops import lib as L
    lib = L.lib()
    fn = lib.b2_gemv_int4_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_int, C.c_int, C.c_void_p]
    err = lib.b2_gemv_int4_noalloc_strerror
    err.restype = C.c_char_p
    dummy = torch.zeros(64, dtype=torch.float16, device="cuda")
    p = dummy.data_ptr()
    # 8 rows x 400k outputs split along K: partial sums exceed the built-in block -> refused, nothing launched
    rc = fn(p, p, p, 1 << 20, p, 1 << 20, 8, 1024, 400_000, 128, 0, None)
    assert rc == -2 and b"scratch" in err(rc)
    assert fn(None, p, p, 64, p, 64, 1, 64, 64, 128, 0, None) == -1
    assert fn(p, p, p, 64, p, 64, 9, 64, 64, 128, 0, None) == -1
    assert fn(p, p, p, 64, p, 64, 1, 64, 64, 100, 0, None) == -1
    # alignment rules: an odd row stride, or pointers off their natural alignment, are refused before any launch
    assert fn(p, p, p, 65, p, 64, 2, 64, 64, 128, 0, None) == -1
    assert fn(p, p, p + 2, 64, p, 64, 1, 64, 64, 128, 0, None) == -1
    assert fn(p + 8, p, p, 64, p, 64, 1, 64, 64, 128, 0, None) == -1
    assert fn(p, p + 4, p, 64, p, 64, 1, 64, 64, 128, 0, None) == -1
    assert b"misaligned" in err(-1)
    torch.cuda.synchronize()
