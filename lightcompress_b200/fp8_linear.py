"""Host mirror of the reference's block-wise FP8 linear forward.

Same names and arguments as the Triton entry points the reference imports when Triton is usable
(llmc/compression/quantization/kernel.py: act_quant :31-53, fp8_gemm :217-242) and as
block_wise_fp8_forward_func (module_utils.py:41-46); each is one kernel through the C ABI.
"""
import torch

from . import _lib as L


def act_quant(x, block_size=128):
    """(e4m3 tensor of x's shape, fp32 scales (*x.shape[:-1], x.shape[-1] // 128))."""
    if block_size != 128:
        raise NotImplementedError('the block-wise FP8 kernels use groups of 128')
    L.require_cuda(x)
    assert x.is_contiguous(), 'Input tensor must be contiguous'
    assert x.size(-1) % block_size == 0, \
        f'Last dimension size must be divisible by block_size (block_size={block_size})'
    y = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((*x.shape[:-1], x.size(-1) // block_size), dtype=torch.float32, device=x.device)
    L.call('lc_fp8_e4m3_act_quant', L.ptr(x), L.lc_dtype(x), x.numel(), block_size, L.ptr(y), L.ptr(s),
           L.stream_of(x))
    return y, s


def weight_cast_to_fp8(x, block_size=128):
    """kernel.py:73-83 (the Triton version the reference binds on GPUs with FP8 support,
    base_blockwise_quantization.py:22-27): (e4m3 weight, fp32 scale per 128 x 128 block) with that kernel's
    arithmetic -- scale = max|x| * fl(1/448), no floor.  `lightcompress_b200.quant.weight_cast_to_fp8` is the
    torch helper's arithmetic (quant.py:36-45: exactly rounded quotient, floor 1e-5)."""
    if block_size != 128:
        raise NotImplementedError('the block-wise FP8 kernels use 128 x 128 blocks')
    L.require_cuda(x)
    assert x.is_contiguous() and x.dim() == 2
    m, n = x.shape
    y = torch.empty((m, n), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((-(-m // 128), -(-n // 128)), dtype=torch.float32, device=x.device)
    L.call('lc_fp8_e4m3_block_quant_triton', L.ptr(x), L.lc_dtype(x), m, n, 128, None, L.ptr(y), L.ptr(s),
           L.stream_of(x))
    return y, s


def weight_cast_to_bf16(x, s, block_size=128):
    """kernel.py:115-131: e4m3 weight times its block scale (the Triton kernel writes the default dtype; its
    callers cast to bf16, which is what this returns)."""
    from .quant import weight_cast_to_bf16 as cast
    return cast(x, s, block_size)


def fp8_gemm(a, a_s, b, b_s, out_dtype=torch.bfloat16):
    """a: (..., K) e4m3 with scales a_s (..., K / 128); b: (N, K) e4m3 with scales b_s (ceil(N / 128), K / 128).
    Returns (..., N) in out_dtype (the reference allocates torch.get_default_dtype() and its caller casts
    to bf16).  The device status word is checked here (one synchronisation)."""
    L.require_cuda(a, a_s, b, b_s)
    assert a.is_contiguous() and b.is_contiguous(), 'Input tensors must be contiguous'
    assert a_s.is_contiguous() and b_s.is_contiguous(), 'Scaling factor tensors must be contiguous'
    K = a.size(-1)
    M = a.numel() // K
    N = b.size(0)
    c = torch.empty((*a.shape[:-1], N), dtype=out_dtype, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    L.call('lc_fp8_block_gemm', L.ptr(a), L.ptr(a_s), L.ptr(b), L.ptr(b_s), M, N, K, L.ptr(c),
           L.LC_BF16 if out_dtype == torch.bfloat16 else L.LC_F32, L.ptr(status), L.stream_of(a))
    code = int(status.item())
    if code:
        raise L.LcError('lc_fp8_block_gemm', code, L.status_string(code))
    return c


def block_wise_fp8_forward_func(x, w, w_scale, block_size, bias):
    x, scale = act_quant(x, block_size)
    y = fp8_gemm(x, scale, w, w_scale).to(torch.bfloat16)
    if bias is not None:
        y += bias
    return y
