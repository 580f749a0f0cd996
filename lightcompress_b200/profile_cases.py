"""Small, self-terminating workloads of each kernel family, sized for profiler captures
(inputs larger than the 126 MB L2, a few hundred MB on the device, a handful of launches).

    python -m lightcompress_b200.profile_cases hessian|hessian_wide|rtn|fp8|gptq|factor|block_ops|fp8_linear|mse|awq_clip|act_static|quik|w48 [--launches N]
"""
import argparse

import torch

from . import FloatQuantizer, GPTQ, IntegerQuantizer
from . import _lib as L


def hessian(n):
    C, T = 4096, 16384
    g = torch.Generator().manual_seed(1)
    X = torch.randn(T, C, generator=g).to(torch.bfloat16).cuda()
    H = torch.zeros(C, C, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    for _ in range(n):
        L.call('lc_hessian_accum', L.ptr(X), T, C, L.ptr(H), 1.0, 1.0, 0, L.ptr(status), L.stream_of(X))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for T1 in (2048,):
        for _ in range(n):
            L.call('lc_hessian_accum', L.ptr(X), T1, C, L.ptr(H), 1.0, 1.0, 0, L.ptr(status), L.stream_of(X))
    torch.cuda.synchronize()


def hessian_wide(n):
    """The down_proj width: C = 11008, 16384 tokens per launch."""
    C, T = 11008, 16384
    g = torch.Generator().manual_seed(5)
    X = torch.randn(T, C, generator=g).to(torch.bfloat16).cuda()
    H = torch.zeros(C, C, device='cuda')
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    for _ in range(n):
        L.call('lc_hessian_accum', L.ptr(X), T, C, L.ptr(H), 1.0, 1.0, 0, L.ptr(status), L.stream_of(X))
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def factor(n):
    """Blocked triangular inverse (and the tensor-core GEMM under it) on a 4096 x 4096 Hessian."""
    C = 4096
    g = torch.Generator().manual_seed(6)
    X = torch.randn(2 * C, C, generator=g).cuda()
    H = X.t() @ X
    solver = GPTQ(IntegerQuantizer(4, False, 'per_group', group_size=128), {'actorder': True})
    for _ in range(n):
        solver.factorize(H, 0.5)
    solver.check_status()
    torch.cuda.synchronize()


def block_ops(n):
    """RMS norm, rotary embedding and SiLU-gate on one 2048-token sequence of Llama-2-7B width."""
    from . import block_ops as B
    g = torch.Generator().manual_seed(7)
    x = torch.randn(8, 2048, 4096, generator=g).to(torch.bfloat16).cuda()
    w = torch.ones(4096, dtype=torch.bfloat16, device='cuda')
    q = x.view(8, 2048, 32, 128).transpose(1, 2)
    cs = torch.randn(8, 2048, 128, generator=g).to(torch.bfloat16).cuda()
    gate = torch.randn(8 * 2048, 11008, generator=g).to(torch.bfloat16).cuda()
    for _ in range(n):
        B._rms_raw(x, w, 1e-5)
        B.rope_apply_one(q, cs, cs)
        B.silu_mul(gate, gate)
    torch.cuda.synchronize()


def fp8_linear(n):
    """Block-wise FP8 linear forward: act_quant + block-scaled FP8 GEMM, M = 8192, N = 11008, K = 4096."""
    from .fp8_linear import act_quant, fp8_gemm
    from .quant import weight_cast_to_fp8
    g = torch.Generator().manual_seed(8)
    x = torch.randn(8192, 4096, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(11008, 4096, generator=g) * 0.05).to(torch.bfloat16).cuda()
    wq, ws = weight_cast_to_fp8(w)
    for _ in range(n):
        a, a_s = act_quant(x)
        fp8_gemm(a, a_s, wq, ws)
    torch.cuda.synchronize()


def mse(n):
    """MSE range search, W4 asymmetric g128 on an 8192 x 4096 fp32 weight."""
    g = torch.Generator().manual_seed(9)
    w = (torch.randn(8192, 4096, generator=g) * 0.02).cuda()
    qz = IntegerQuantizer(4, False, 'per_group', group_size=128, calib_algo='mse')
    grouped = qz.reshape_tensor(w)
    for _ in range(n):
        qz.get_tensor_range(grouped)
    torch.cuda.synchronize()


def awq_clip(n):
    """AWQ clip search of one 4096 x 4096 bf16 linear on 512 sampled tokens (W4 asymmetric g128)."""
    from .awq import Awq
    g = torch.Generator().manual_seed(10)
    w = (torch.randn(4096, 4096, generator=g) * 0.02).to(torch.bfloat16).cuda()
    x = torch.randn(16, 512, 4096, generator=g).to(torch.bfloat16).cuda()
    awq = Awq(IntegerQuantizer(4, False, 'per_group', group_size=128), {}, calib_seq_len=512)
    for _ in range(n):
        awq.auto_clip_layer(w, x, apply=False)
    torch.cuda.synchronize()


def rtn(n):
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(8192, 4096, generator=g) * 0.02).cuda()
    qz = IntegerQuantizer(4, False, 'per_group', group_size=128)
    for _ in range(n):
        qz.fake_quant_weight_dynamic(w)
    for _ in range(n):
        qz.quant_all_dynamic(w, packed=True)
    wb = w.to(torch.bfloat16)
    for _ in range(n):
        qz.fake_quant_weight_dynamic(wb)
    qa = IntegerQuantizer(8, True, 'per_token')
    x = torch.randn(16384, 4096, generator=g).to(torch.bfloat16).cuda()
    for _ in range(n):
        qa.fake_quant_act_dynamic(x)
    torch.cuda.synchronize()


def fp8(n):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(65536, 2048, generator=g).to(torch.bfloat16).cuda()
    q = FloatQuantizer('e4m3', True, 'per_token', use_qtorch=True)
    for _ in range(n):
        q.fake_quant_act_dynamic(x)
    torch.cuda.synchronize()


def gptq(n):
    R = C = 4096
    g = torch.Generator().manual_seed(4)
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16).cuda()
    X = torch.randn(8192, C, generator=g).to(torch.bfloat16).cuda()
    H = torch.zeros(C, C, device='cuda')
    L.call('lc_hessian_accum', L.ptr(X), X.shape[0], C, L.ptr(H), 1.0, 1.0, 0, None, L.stream_of(X))
    solver = GPTQ(IntegerQuantizer(4, False, 'per_group', group_size=128), {'actorder': True})
    for _ in range(n):
        solver.solve(W, H, 2.0 / 4)
    torch.cuda.synchronize()


def act_static(n):
    """Per-tensor ranges of 8 calibration tensors of 64 MB (bf16) in one launch."""
    qz = IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_minmax')
    g = torch.Generator(device='cuda').manual_seed(8)
    acts = [torch.randn(4, 2048, 4096, generator=g, device='cuda').to(torch.bfloat16) for _ in range(8)]
    for _ in range(n):
        qz._tensor_ranges(acts)
    torch.cuda.synchronize()


def quik(n):
    """QUIK: per-channel max |x| of 65536 x 4096 bf16 and the masked per-token fake quant of 32768 x 4096."""
    from .quik import QUIK
    g = torch.Generator(device='cuda').manual_seed(9)
    x = torch.randn(65536, 4096, generator=g, device='cuda').to(torch.bfloat16)
    aq = IntegerQuantizer(8, True, 'per_token')
    q = QUIK(IntegerQuantizer(4, True, 'per_channel'), aq, {'fp_relative': False, 'fp_features': 256, 'fp_threshold': 0.0})
    order = torch.randperm(4096, generator=g, device='cuda')
    args = {'int_indices': order[:-256], 'fp_indices': order[-256:]}
    for _ in range(n):
        q.get_tensor_scale('l', x)
        aq.fake_quant_act_dynamic(x[:32768], args)
    torch.cuda.synchronize()


def w48(n):
    """Weight48IntegerQuantizer on a 16384 x 8192 bf16 weight (the levels of rtn_w_a_wint4aint8.yml)."""
    from . import Weight48IntegerQuantizer
    bit4 = {'symmetric': False, 'granularity': 'per_group', 'group_size': 128, 'scales_bit': 8,
            'scales_symmetric': True, 'zeros_bit': 8, 'zeros_symmetric': True}
    bit8 = {'symmetric': True, 'granularity': 'per_channel', 'int_range': [-120, 120]}
    qz = Weight48IntegerQuantizer(48, bit4, bit8)
    g = torch.Generator(device='cuda').manual_seed(10)
    w = torch.randn(16384, 8192, generator=g, device='cuda').to(torch.bfloat16)
    for _ in range(n):
        qz.fake_quant_weight_dynamic(w)
    torch.cuda.synchronize()


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('case', choices=['hessian', 'hessian_wide', 'rtn', 'fp8', 'gptq', 'factor', 'block_ops', 'fp8_linear', 'mse', 'awq_clip', 'act_static', 'quik', 'w48'])
    ap.add_argument('--launches', type=int, default=3)
    a = ap.parse_args()
    {'hessian': hessian, 'hessian_wide': hessian_wide, 'rtn': rtn, 'fp8': fp8, 'gptq': gptq, 'factor': factor,
     'block_ops': block_ops, 'fp8_linear': fp8_linear, 'mse': mse, 'awq_clip': awq_clip, 'act_static': act_static,
     'quik': quik, 'w48': w48}[a.case](a.launches)
    print('done', a.case)
