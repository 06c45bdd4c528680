"""The allocation-free mat-vec entry point (csrc/cuda/volta_noalloc.h), called the way a host without an
allocator would call it: straight through the exported C symbol, with caller-owned inputs and outputs and
no workspace argument. It must agree with the ordinary entry point (which takes scratch buffers from the
caller) on two calls in a row, since the built-in scratch keeps its contents between calls.
Collected last on purpose: a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sym():
    from volta_engine_b200 import _lib
    fn = _lib.kernels().ve_nvfp4_gemv_mma_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_long,
                   ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def test_static_scratch_matvec_matches_regular_entry_twice():
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.quant import nvfp4 as qn
    from util import assert_close
    dev = "cuda"
    fn = _sym()
    g = torch.Generator(device=dev).manual_seed(5)
    N, Kd, KS = 2048, 4096, 4
    w = torch.randn(N, Kd, generator=g, device=dev) * 0.02
    p, s, gs = qn.quantize_nvfp4(w, search=False)
    wg, sg = qn.prepack_gv(p, s)
    stream = torch.cuda.current_stream().cuda_stream
    for call_no, M in enumerate((3, 11)):
        x = (torch.randn(M, Kd, generator=g, device=dev)).to(torch.bfloat16)
        res = (torch.randn(M, N, generator=g, device=dev)).to(torch.bfloat16)
        want = K.nvfp4_gemv_mma(wg, sg, gs, x, N, Kd, residual=res, ks=KS)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = fn(wg.data_ptr(), sg.data_ptr(), gs, x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0),
                res.data_ptr(), res.stride(0), M, N, Kd, KS, stream)
        assert rc == 0, f"call {call_no}: CUDA error {rc}"
        torch.cuda.synchronize()
        assert_close(out, want, name=f"static scratch call {call_no}")
        assert torch.equal(out, want)  # same kernel, same split order: identical bits
    # oversize requests are refused without launching
    assert fn(wg.data_ptr(), sg.data_ptr(), gs, x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), None, 0,
              1, 65536, 64, 8, stream) != 0
    torch.cuda.synchronize()


def test_static_scratch_limits_and_reuse():
    """The corners of the built-in scratch: no split (no counter clearing), a call that fills the scratch exactly
    (KS * N == 32768, the last slot), and a small call right after a large one (partials of the large call are still in
    the shared array). Each must agree bit for bit with the entry point that takes caller-owned scratch."""
    from volta_engine_b200.ops import kernels as K
    from volta_engine_b200.quant import nvfp4 as qn
    dev = "cuda"
    fn = _sym()
    g = torch.Generator(device=dev).manual_seed(9)
    stream = torch.cuda.current_stream().cuda_stream
    for N, Kd, KS, M in ((1024, 512, 1, 2), (8192, 1024, 4, 5), (256, 1024, 4, 1), (8192, 1024, 4, 16), (512, 2048, 2, 3)):
        w = torch.randn(N, Kd, generator=g, device=dev) * 0.02
        p, s_, gs = qn.quantize_nvfp4(w, search=False)
        wg, sg = qn.prepack_gv(p, s_)
        x = torch.randn(M, Kd, generator=g, device=dev).to(torch.bfloat16)
        want = K.nvfp4_gemv_mma(wg, sg, gs, x, N, Kd, ks=KS)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = fn(wg.data_ptr(), sg.data_ptr(), gs, x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), None, 0,
                M, N, Kd, KS, stream)
        assert rc == 0, (N, Kd, KS, M, rc)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (N, Kd, KS, M)
    # one past the limit is refused
    assert fn(wg.data_ptr(), sg.data_ptr(), gs, x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), None, 0,
              1, 8192 + 16, 1024, 4, stream) != 0
