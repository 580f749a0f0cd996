"""SpQR on the GPU against the reference's own outputs (tests/golden/spqr_layer.pt) and the pinned oracle.

The outlier decisions compare a leave-one-out error difference with a threshold; the kernel evaluates
those errors with reciprocals instead of divisions and sums them in its own order, so a decision can
differ where the difference sits within rounding of the threshold.  Bars: outlier masks differ in fewer
than 0.05 % of positions, codes in fewer than 0.1 %, deployed weights likewise; where no decision differs
the statistics are bit-identical."""
import math

import pytest
import torch

from oracle import spqr_ref

pytestmark = pytest.mark.gpu


def _solver(c, **special):
    from lightcompress_b200 import IntegerQuantizer, SpQR
    wq = IntegerQuantizer(c['bit'], False, 'per_group', group_size=c['group'], round_zp=False)
    sp = dict(actorder=c['actorder'], percdamp=c['percdamp'], blocksize=128, relative_threshold=c['rel_threshold'],
              simplified_outliers=c['simplified'])
    sp.update(special)
    return SpQR(wq, sp, c['W'].dtype), wq


def _codes(weight, scales, zeros, perm, bit, group):
    wp = weight[:, perm].reshape(-1, group)
    return torch.clamp(torch.round(wp / scales.clamp_min(1e-9) + zeros), 0, 2 ** bit - 1).reshape(weight.shape)


def test_layer_matches_reference_golden(golden):
    for key, c in golden('spqr_layer.pt').items():
        solver, wq = _solver(c)
        layer = torch.nn.Linear(c['W'].shape[1], c['W'].shape[0], bias=False, dtype=c['W'].dtype).cuda()
        layer.weight.data = c['W'].cuda()
        solver.layer_init(layer, 'l')
        for i in range(c['X'].shape[0]):
            solver.add_batch(layer, 'l', c['X'][i:i + 1].cuda())
        solver.layer_transform(layer, 'l')
        solver.check_status()
        fq = solver.w_qdq(layer, wq)
        perm = layer.buf_perm.cpu() if c['actorder'] else torch.arange(c['W'].shape[1])
        assert torch.equal(perm, c['buf_perm']), key
        mask = layer.buf_mask.to_dense().cpu() != 0
        mask_diff = float((mask != c['mask']).float().mean())
        ours = _codes(layer.weight.data.cpu(), layer.buf_scales.cpu(), layer.buf_zeros.cpu(), perm, c['bit'], c['group'])
        ref = _codes(c['weight'], c['buf_scales'], c['buf_zeros'], c['buf_perm'], c['bit'], c['group'])
        code_diff = float((ours != ref).float().mean())
        fq_diff = float((fq.cpu() != c['w_qdq']).float().mean())
        s_same = float((layer.buf_scales.cpu() == c['buf_scales']).float().mean())
        print(f'spqr {key}: outliers {int(mask.sum())} (reference {int(c["mask"].sum())}), mask differs {mask_diff:.4%}, '
              f'codes {code_diff:.4%}, deployed weights {fq_diff:.4%}, scales bit-equal {s_same:.4%}')
        assert layer.buf_scales.shape == c['buf_scales'].shape and layer.buf_zeros.shape == c['buf_zeros'].shape
        assert layer.weight.dtype == torch.float32 and fq.dtype == c['w_qdq'].dtype
        assert mask_diff < 5e-4 and code_diff < 1e-3 and fq_diff < 1e-3, key
        rel = float((layer.weight.data.cpu() - c['weight']).norm() / c['weight'].norm())
        assert rel < 1e-3, (key, rel)


@pytest.mark.parametrize('R,C,T,thr', [(256, 1024, 2048, 0.2), (384, 2304, 4096, 0.2), (256, 1024, 2048, math.inf)])
def test_layer_matches_oracle_on_the_same_gpu(R, C, T, thr):
    """Wider layers (the tensor-core trailing update from 2304 columns), oracle = the pinned restatement
    evaluated with torch on this GPU, column order and threshold pinned to the oracle's."""
    from lightcompress_b200 import GPTQ
    g = torch.Generator().manual_seed(R + C)
    W = torch.randn(R, C, generator=g) * 0.02
    W[torch.rand(R, C, generator=g) < 0.01] *= 8
    W = W.to(torch.bfloat16).cuda()
    X = torch.randn(T, C, generator=g)
    X[:, torch.randperm(C, generator=g)[:C // 100]] *= 20
    X = X.to(torch.bfloat16).cuda()
    H = (X.float().t() @ X.float()) * (2.0 / 4)
    res = spqr_ref.quantize_layer(W, H, percdamp=1.0, relative_threshold=thr)
    c = dict(bit=4, group=16, actorder=True, percdamp=1.0, rel_threshold=thr, simplified=False, W=W)
    solver, wq = _solver(c)
    solver.h_upper = False
    fac = solver.factorize(H, 1.0, perm=res['buf_perm'])
    thr_dev = torch.full((1,), float(res['threshold']), dtype=torch.float32, device='cuda')
    out = solver.solve(W, H, 1.0, factor=fac, threshold=thr_dev)
    solver.check_status()
    own_thr = float(solver.outlier_threshold(W.float()[:, res['buf_perm']], fac['U']))
    assert abs(own_thr - float(res['threshold'])) <= 1e-3 * abs(float(res['threshold'])) or thr == math.inf
    mask_diff = float((out['mask'].bool() != res['mask']).float().mean())
    ours = _codes(out['weight'], out['buf_scales'], out['buf_zeros'], res['buf_perm'], 4, 16)
    ref = _codes(res['weight'], res['buf_scales'], res['buf_zeros'], res['buf_perm'], 4, 16)
    code_diff = float((ours != ref).float().mean())
    print(f'spqr {R}x{C}: outliers {int(out["mask"].sum())} (oracle {int(res["mask"].sum())}), mask differs '
          f'{mask_diff:.4%}, codes {code_diff:.4%}')
    assert mask_diff < 5e-4 and code_diff < 1e-3
    layer = torch.nn.Linear(C, R, bias=False, dtype=torch.bfloat16).cuda()
    solver._install(layer, out)
    fq = solver.w_qdq(layer, wq)
    want = spqr_ref.w_qdq({k: out[k] if k != 'mask' else out['mask'].bool() for k in
                           ('weight', 'mask', 'buf_scales', 'buf_zeros', 'buf_perm', 'buf_invperm')}, torch.bfloat16)
    assert torch.equal(fq, want)


def test_dead_input_channels_follow_the_reference_order_of_operations():
    """spqr.py:143-149: the damp is a fraction of mean |diag| taken with the dead columns at 0, and a dead
    column's diagonal becomes exactly 1 afterwards (GPTQ sets it before dampening)."""
    g = torch.Generator().manual_seed(71)
    R, C, T = 128, 512, 2048
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16).cuda()
    X = torch.randn(T, C, generator=g).to(torch.bfloat16)
    dead = torch.tensor([7, 300, 510])
    X[:, dead] = 0
    X = X.cuda()
    H = (X.float().t() @ X.float()) * (2.0 / 4)
    res = spqr_ref.quantize_layer(W, H, percdamp=1.0, relative_threshold=0.2)
    c = dict(bit=4, group=16, actorder=True, percdamp=1.0, rel_threshold=0.2, simplified=False, W=W)
    solver, wq = _solver(c)
    solver.h_upper = False
    fac = solver.factorize(H, 1.0, perm=res['buf_perm'])
    rel = float((fac['U'] - res['U']).abs().max() / res['U'].abs().max())
    assert rel < 1e-4, rel
    thr_dev = torch.full((1,), float(res['threshold']), dtype=torch.float32, device='cuda')
    out = solver.solve(W, H, 1.0, factor=fac, threshold=thr_dev)
    solver.check_status()
    assert bool((out['weight'][:, dead.cuda()] == 0).all())
    ours = _codes(out['weight'], out['buf_scales'], out['buf_zeros'], res['buf_perm'], 4, 16)
    ref = _codes(res['weight'], res['buf_scales'], res['buf_zeros'], res['buf_perm'], 4, 16)
    code_diff = float((ours != ref).float().mean())
    print(f'spqr dead channels: codes {code_diff:.4%}, U relative difference {rel:.2e}')
    assert code_diff < 1e-3
