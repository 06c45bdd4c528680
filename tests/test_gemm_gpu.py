"""tcgen05 GEMMs (bf16, W4A16, W4A4) against fp32 matmul of the same (de)quantised operands."""
import pytest
import torch

from volta_engine_b200.ops import kernels as K
from volta_engine_b200.quant import nvfp4 as qn
from util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, std=1.0, seed=0, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * std).to(dtype)


@pytest.mark.parametrize("T,N,Kd", [(16, 256, 512), (100, 384, 1024), (300, 1024, 5120), (2048, 512, 2048)])
def test_gemm_bf16(T, N, Kd):
    W, x = rnd(N, Kd, std=0.05, seed=1), rnd(T, Kd, seed=2)
    want = x.float() @ W.float().t()
    got = K.gemm_bf16(W, x)
    assert K.check_status(DEV) == 0
    assert_close(got, want, name="gemm bf16")
    res = rnd(T, N, seed=3)
    got = K.gemm_bf16(W, x, residual=res, alpha=0.5)
    assert_close(got, 0.5 * want + res.float(), name="gemm bf16 alpha+residual")
    got32 = K.gemm_bf16(W, x, out_f32=True)
    assert_close(got32, want, rel=1e-3, name="gemm bf16 f32 out")


@pytest.mark.parametrize("T,N,Kd", [(17, 256, 512), (200, 384, 1024), (600, 1024, 5120)])
def test_gemm_w4a16(T, N, Kd):
    w = rnd(N, Kd, std=0.02, seed=4, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w, search=False)
    wd = qn.dequantize_nvfp4(p, s, g)
    x = rnd(T, Kd, seed=5)
    got = K.gemm_w4a16(p, qn.scales_blocked_k128(s), g, x)
    assert K.check_status(DEV) == 0
    assert_close(got, x.float() @ wd.t(), name="gemm w4a16")


@pytest.mark.parametrize("T,N,Kd", [(129, 256, 128), (300, 512, 640), (1000, 1024, 5120), (2048, 768, 2176)])
def test_gemm_w4a16_wide_tiles(T, N, Kd):
    """The 256 x 256-tile prefill kernel (two weight sub-tiles per activation tile): ragged token counts, K that is an odd
    multiple of 128 (the last 128-wide scale block is half used per stage), residual input, and agreement with the
    128-feature-tile kernel on the same operands."""
    w = rnd(N, Kd, std=0.02, seed=14, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w, search=False)
    wd = qn.dequantize_nvfp4(p, s, g)
    x = rnd(T, Kd, seed=15)
    sf = qn.scales_blocked_k128(s)
    want = x.float() @ wd.t()
    got = K.gemm_w4a16(p, sf, g, x)
    assert K.check_status(DEV) == 0
    assert_close(got, want, name="gemm w4a16 wide")
    res = rnd(T, N, seed=16)
    assert_close(K.gemm_w4a16(p, sf, g, x, residual=res), want + res.float(), name="gemm w4a16 wide + residual")
    K.GEMM_WIDE = False
    try:
        narrow = K.gemm_w4a16(p, sf, g, x)
    finally:
        K.GEMM_WIDE = True
    assert_close(got, narrow.float(), rel=1e-2, name="wide vs 128-feature tiles")


@pytest.mark.parametrize("T,N,Kd", [(16, 256, 512), (130, 384, 1024), (600, 1024, 5120)])
def test_gemm_w4a4(T, N, Kd):
    w = rnd(N, Kd, std=0.02, seed=6, dtype=torch.float32)
    p, s, g = qn.quantize_nvfp4(w, search=False)
    wd = qn.dequantize_nvfp4(p, s, g)
    x = rnd(T, Kd, seed=7)
    xp, xs = K.nvfp4_quant_rows(x, blocked=True)
    rp, rs = K.nvfp4_quant_rows(x, blocked=False)
    xd = qn.dequantize_nvfp4(rp, rs, 1.0)
    got = K.gemm_w4a4(p, qn.scales_atoms_512(s), g, xp, xs, T)
    assert K.check_status(DEV) == 0
    assert_close(got, xd @ wd.t(), name="gemm w4a4")
