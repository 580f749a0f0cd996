"""Block-wise FP8 linear forward (act_quant + block-scaled FP8 GEMM on tcgen05) against a restatement of
the reference's Triton kernels' arithmetic (llmc/compression/quantization/kernel.py:7-53, :153-242) in
torch ops, and against those Triton kernels themselves, run on the same GPU from the copy of the
reference's package that travels with the tests (the last test: that is the pin)."""
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
    # the kernel divides like the reference's Triton kernel (approximate full-range division), the restatement
    # exactly: a quotient within an ulp of the midpoint of two e4m3 values may get the neighbouring code
    diff = a[~nan] != b[~nan]
    assert float(diff.float().mean()) < 1e-4
    assert int((a[~nan][diff].int() - b[~nan][diff].int()).abs().max().item() if diff.any() else 0) <= 1


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


def _reference_triton_kernels():
    """The reference's own Triton kernels (llmc/compression/quantization/kernel.py), loaded by file path from
    the copy of its package that travels with the tests; None where that copy or Triton is missing."""
    import importlib.util
    import os
    from oracle import ref_driver as rd
    root = rd.find_reference()
    if root is None:
        return None
    path = os.path.join(root, 'llmc', 'compression', 'quantization', 'kernel.py')
    try:
        import triton  # noqa: F401
        spec = importlib.util.spec_from_file_location('llmc_ref_triton_kernels', path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    except Exception:
        return None


def test_block_fp8_kernels_against_the_reference_triton_kernels_on_this_gpu():
    """Pins the block-wise FP8 path to the reference itself: its Triton kernels act_quant, weight_cast_to_fp8,
    weight_cast_to_bf16 and fp8_gemm (kernel.py:7-242) run on this GPU on the same inputs.  Codes and scales
    bit for bit; the GEMM to 1e-5 of max |C| (the two accumulate the 128-wide k blocks in different orders)."""
    ref = _reference_triton_kernels()
    if ref is None:
        pytest.skip('no reference copy or no Triton')
    from lightcompress_b200.fp8_linear import act_quant, fp8_gemm
    from lightcompress_b200.quant import weight_cast_to_bf16, weight_cast_to_fp8
    g = torch.Generator().manual_seed(77)
    M, N, K = 256, 384, 512
    x = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    w[:, ::61] *= 20
    w = w.cuda()
    try:
        ry, rs = ref.act_quant(x)
        rw, rws = ref.weight_cast_to_fp8(w)
        rback = ref.weight_cast_to_bf16(rw, rws)
        rc = ref.fp8_gemm(ry, rs, rw, rws)
        torch.cuda.synchronize()
    except Exception as e:                                  # Triton without a backend for this GPU
        pytest.skip(f'the reference Triton kernels do not compile here: {type(e).__name__}')
    from lightcompress_b200 import fp8_linear
    y, s = act_quant(x)
    assert torch.equal(s, rs)
    assert torch.equal(y.view(torch.uint8), ry.view(torch.uint8))
    wq, ws = fp8_linear.weight_cast_to_fp8(w)
    assert torch.equal(ws.reshape(rws.shape), rws)
    assert torch.equal(wq.view(torch.uint8), rw.view(torch.uint8))
    back = fp8_linear.weight_cast_to_bf16(wq, ws)
    assert torch.equal(back, rback.to(torch.bfloat16).reshape(back.shape))      # the Triton kernel writes fp32
    c = fp8_gemm(y, s, wq, ws, out_dtype=torch.float32)
    err = float((c.float() - rc.float()).abs().max() / rc.float().abs().max())
    print(f'fp8_gemm vs the reference Triton kernel: max |diff| / max |C| = {err:.2e}')
    assert err < 1e-5
    # the torch helper's arithmetic (quant.py:36-45), which the fixtures pin, differs from the Triton kernel's
    # in the last bit of some scales (exact quotient against a multiplication by fl(1/448))
    wq2, ws2 = weight_cast_to_fp8(w)
    ulp = (ws2.reshape(rws.shape).view(torch.int32).long() - rws.view(torch.int32).long()).abs().max().item()
    print(f'torch-helper scales vs Triton scales: max distance {ulp} ulp, '
          f'{float((wq2.view(torch.uint8) != rw.view(torch.uint8)).float().mean()):.4%} of the codes differ')
    assert ulp <= 1
