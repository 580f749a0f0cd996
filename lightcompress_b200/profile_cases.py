"""Small, self-terminating workloads of each kernel family, sized for profiler captures
(inputs larger than the 126 MB L2, a few hundred MB on the device, a handful of launches).

    python -m lightcompress_b200.profile_cases hessian|rtn|fp8|gptq [--launches N]
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


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('case', choices=['hessian', 'rtn', 'fp8', 'gptq'])
    ap.add_argument('--launches', type=int, default=3)
    a = ap.parse_args()
    {'hessian': hessian, 'rtn': rtn, 'fp8': fp8, 'gptq': gptq}[a.case](a.launches)
    print('done', a.case)
