"""Block-wise FP8 linear forward (act_quant + block-scaled FP8 GEMM on tcgen05) against a restatement of
the reference's Triton kernels' arithmetic (llmc/compression/quantization/kernel.py:7-53, :153-242) in
torch ops.  The Triton kernels themselves cannot run where the fixtures are made, so this parity is
not pinned to reference output."""
import pytest
import torch

from oracle import quant_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
def test_act_quant_matches_the_restated_kernel(dtype):
    from lightcompress_b200.fp8_linear import act_quant
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(3, 70, 512, generator=g) * 2).to(dtype)
    x[0, 0, :128] = 0                       # an all-zero group: scale 0, NaN codes, like the reference
    x[1, 2, 5] = 300.0
    y, s = act_quant(x.cuda())
    ry, rs = quant_ref.fp8_act_quant(x)
    assert y.dtype == torch.float8_e4m3fn and s.shape == (3, 70, 4) and s.dtype == torch.float32
    assert torch.equal(s.cpu(), rs)
    a, b = y.cpu().view(torch.uint8), ry.view(torch.uint8)
    nan = (a & 0x7f) == 0x7f
    assert torch.equal(nan, (b & 0x7f) == 0x7f) and bool(nan[0, 0, :128].all())
    assert torch.equal(a[~nan], b[~nan])


@pytest.mark.parametrize('M,N,K', [(128, 128, 128), (300, 256, 512), (1000, 1408, 2048), (64, 200, 384),
                                   (2048, 4096, 4096)])
def test_fp8_block_gemm_matches_the_restated_kernel(M, N, K):
    from lightcompress_b200.fp8_linear import act_quant, fp8_gemm
    from lightcompress_b200.quant import weight_cast_to_fp8
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    w[:, ::61] *= 20
    w = w.cuda()
    if N % 128 == 0 or K % 128 == 0:
        wq, ws = weight_cast_to_fp8(w, 128)
    a, a_s = act_quant(x)
    c = fp8_gemm(a, a_s, wq, ws, out_dtype=torch.float32)
    ref = quant_ref.fp8_block_gemm(a, a_s, wq, ws)
    err = float((c - ref).abs().max() / ref.abs().max())
    print(f'M={M} N={N} K={K}: max |C - ref| = {err:.2e} of max |C|')
    # products of e4m3 values are exact; what differs is the tensor core's accumulation of a k block
    assert err < 2e-3
    cb = fp8_gemm(a, a_s, wq, ws)
    assert cb.dtype == torch.bfloat16
    assert torch.allclose(cb.float(), ref, rtol=1e-2, atol=1e-2 * float(ref.abs().max()))
    # against the unquantised product: the FP8 linear approximates x @ w^T
    full = x.float() @ w.float().t()
    rel = float((c - full).norm() / full.norm())
    assert rel < 0.08, rel


def test_block_wise_fp8_forward_func():
    from lightcompress_b200.fp8_linear import block_wise_fp8_forward_func
    from lightcompress_b200.quant import weight_cast_to_bf16, weight_cast_to_fp8
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4, 96, 1024, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(768, 1024, generator=g) * 0.03).to(torch.bfloat16).cuda()
    bias = torch.randn(768, generator=g).to(torch.bfloat16).cuda()
    wq, ws = weight_cast_to_fp8(w, 128)
    y = block_wise_fp8_forward_func(x, wq, ws, 128, bias)
    assert y.shape == (4, 96, 768) and y.dtype == torch.bfloat16
    ref = torch.nn.functional.linear(x.float(), weight_cast_to_bf16(wq, ws, 128).float(), bias.float())
    assert float((y.float() - ref).norm() / ref.norm()) < 0.05
