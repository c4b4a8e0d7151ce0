"""The allocation-free C entry point against the regular RMSNorm backward.

Some users of the library cannot let it allocate device memory: they have given the whole device to another
runtime's arena, or they call from a C program that has no PyTorch allocator, or they sit in a loop where an
allocation stall or an out-of-memory failure half-way through is unacceptable. For them the library exports
``pt_rmsnorm_bwd_noalloc`` whose only scratch memory is a fixed array inside the library image. This test
calls that symbol the way such a user would -- through the shared object's C ABI with raw device pointers --
twice in a row (the array is shared between calls and keeps old contents), and checks both results against
the regular entry point. It also checks that an over-sized problem is refused with the documented code.

The file name sorts last on purpose: if it fails under ``pytest -x`` every other test has already run.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from picotron_b200 import build
    lib = ctypes.CDLL(build.ext_path())
    fn = lib.pt_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.pt_noalloc_strerror.restype = ctypes.c_char_p
    lib.pt_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _bf(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g).to(torch.bfloat16)


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from picotron_b200.ops import _ext
    C = _ext.load()
    lib = _lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    # second call: smaller, stale data left behind; third: the widest row the entry point accepts; fourth: no residual
    # gradient (dres == NULL)
    cases = [(300, 2048, True), (77, 1024, True), (300, 4096, True), (130, 2048, False)]
    for call, (T, H, with_dres) in enumerate(cases):
        x, dy = _bf(T, H, seed=10 + call), _bf(T, H, seed=20 + call)
        dres = _bf(T, H, seed=30 + call) if with_dres else None
        w = (1 + 0.1 * _bf(H, seed=40 + call).float()).to(torch.bfloat16)
        _, rstd = C.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = C.rmsnorm_bwd(dy, x, w, rstd, dres)
        dx = torch.empty_like(x)
        dw = torch.full((H,), float("nan"), device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.pt_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                        dres.data_ptr() if with_dres else None, dx.data_ptr(), dw.data_ptr(), T, H, stream)
        assert rc == 0, lib.pt_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            # the driver's own count of free device memory (a cudaMalloc inside the C entry point would not show in the
            # PyTorch allocator's statistics); checked from the second call on, when the symbol look-up and the lazy
            # loading of the kernels are behind us
            assert torch.cuda.mem_get_info()[0] >= free_before
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=3e-2)
        torch.testing.assert_close(dw, dw_ref, rtol=1e-3, atol=1e-2 * math.sqrt(T))


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    x = _bf(4, 8192, seed=1)
    rstd = torch.ones(4, device="cuda")
    dw = torch.zeros(8192, device="cuda")
    rc = lib.pt_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), rstd.data_ptr(), None, x.data_ptr(),
                                    dw.data_ptr(), 4, 8192, torch.cuda.current_stream().cuda_stream)
    assert rc == -21
    assert b"too large" in lib.pt_noalloc_strerror(rc)
    torch.cuda.synchronize()
