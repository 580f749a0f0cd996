"""Packing of 4-bit codes into the two export layouts the reference writes
(llmc/compression/quantization/module_utils.py: VllmRealQuantLinear.pack :931-955,
AutoawqRealQuantLinear.gemm_pack :1099-1158)."""
import torch

from . import _lib as L


def pack_compressed_tensors_int4(weight, wquantizer):
    """Symmetric int4 real quant + compressed-tensors packing in one pass over the weight:
    returns (packed int32 (rows, cols/8), scales (rows, n_groups))."""
    if not wquantizer.sym or wquantizer.bit != 4:
        raise NotImplementedError('compressed-tensors int4 packing is for symmetric 4-bit weights')
    fake, packed, s, z = wquantizer.quant_all_dynamic(weight, packed=True)
    if packed.shape[1] % 4:
        raise ValueError('in_features must be a multiple of 8')
    return packed.view(torch.int32), s


def pack_autoawq_gemm(codes_u8, zeros_u8):
    """AutoAWQ GEMM layout: codes (out, in) uint8 -> qweight (in, out/8) int32; zeros (out, n_groups)
    uint8 -> qzeros (n_groups, out/8) int32."""
    L.require_cuda(codes_u8, zeros_u8)
    outs = []
    for t in (codes_u8, zeros_u8):
        t = t.contiguous()
        R, C = t.shape
        o = torch.empty((C, R // 8), dtype=torch.int32, device=t.device)
        L.call('lc_pack_int4_awq', L.ptr(t), R, C, L.ptr(o), L.stream_of(t))
        outs.append(o)
    return outs[0], outs[1]
