"""The three-term tf32 tensor-core GEMM and the native factorisation built on it, against fp64 /
cuSOLVER results of the same matrices (the reference's chain is torch.linalg.cholesky ->
cholesky_inverse -> cholesky(upper), llmc/compression/quantization/gptq.py:172-174)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lo(x):
    return x - (x.view(torch.int32) & -8192).view(torch.float32)


@pytest.mark.parametrize('M,N,K,beta,sign,flags', [
    (128, 256, 128, 0, 1.0, 0), (384, 1000, 512, 1, -1.0, 0), (1024, 1024, 1024, 1, -1.0, 1),
    (640, 640, 640, 0, 1.0, 2), (640, 512, 640, 0, -1.0, 4), (300, 516, 48, 1, 1.0, 0)])
def test_tf32x3_gemm_matches_fp64(M, N, K, beta, sign, flags):
    from lightcompress_b200 import _lib as L
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(K, M, generator=g).cuda()
    B = torch.randn(K, N, generator=g).cuda()
    if flags & 2:
        B = torch.tril(B)          # B[k][n] = 0 for k < n
    if flags & 4:
        A = torch.triu(A)          # A[k][m] = 0 for k > m
    C0 = torch.randn(M, N, generator=g).cuda()
    C = C0.clone()
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    A_lo, B_lo = _lo(A), _lo(B)
    L.call('lc_tf32x3_gemm_tn', L.ptr(C), N, L.ptr(A), L.ptr(A_lo), M, L.ptr(B), L.ptr(B_lo), N, M, N, K,
           beta, sign, flags, L.ptr(status), L.stream_of(C))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = beta * C0.double() + sign * (A.double().t() @ B.double())
    err = (C.double() - ref).abs()
    if flags & 1:   # only tiles that reach the diagonal are computed; the upper triangle is the contract
        mask = torch.triu(torch.ones(M, N, dtype=torch.bool, device='cuda'))
        err = err[mask]
    # The tensor core adds each MMA's products into the fp32 accumulator with truncation, 3 * K / 8 times
    # per output, so the error grows with K (measured about 1e-5 of the largest output at K = 1024;
    # single-pass tf32 would be about 1e-3).
    rel = float(err.max() / ref.abs().max())
    print(f'M={M} N={N} K={K} flags={flags}: max error {float(err.max()):.2e} = {rel:.2e} of max |C|')
    assert rel < 4e-5, rel


@pytest.mark.parametrize('native', ['native', 'native_full'])
@pytest.mark.parametrize('n', [128, 384, 1152, 4096])
def test_native_factorisation_matches_cusolver(n, native):
    from lightcompress_b200 import GPTQ, IntegerQuantizer
    g = torch.Generator().manual_seed(n)
    X = torch.randn(3 * n, n, generator=g)
    X[:, torch.randperm(n, generator=g)[:max(1, n // 100)]] *= 20
    H = (X.t() @ X).cuda()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    facs = {}
    for mode in (native, 'direct'):
        solver = GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'factorization': mode})
        facs[mode] = solver.factorize(H, 2.0 / 3)
        solver.check_status()
    facs['native'] = facs[native]
    torch.cuda.synchronize()
    U1, U2 = facs['native']['U'], facs['direct']['U']
    assert torch.equal(facs['native']['perm'], facs['direct']['perm'])
    assert torch.equal(U1, torch.triu(U1))
    rel = float((U1 - U2).abs().max() / U2.abs().max())
    # U^T U Hp = I, in fp64, for both
    perm = facs['native']['perm']
    Hp = (H.double() * (2.0 / 3))[perm][:, perm]
    Hp += torch.eye(n, device='cuda', dtype=torch.float64) * 0.01 * Hp.diagonal().mean()
    r1 = float(((U1.double().t() @ U1.double()) @ Hp - torch.eye(n, device='cuda', dtype=torch.float64)).abs().max())
    r2 = float(((U2.double().t() @ U2.double()) @ Hp - torch.eye(n, device='cuda', dtype=torch.float64)).abs().max())
    print(f'n={n} {native}: native vs cuSOLVER max rel diff {rel:.2e}; residual |U^T U H - I| native {r1:.2e} cuSOLVER {r2:.2e}')
    assert rel < 1e-4
    assert r1 < max(4 * r2, 1e-3)
    if facs['native']['U_lo'] is not None:
        assert torch.equal(facs['native']['U_lo'], _lo(U1))


def test_blocked_cholesky_matches_cusolver():
    """The 1024-row blocked Cholesky used for wide matrices (forced here at n = 2304: two full blocks and a
    ragged one) against cuSOLVER's potrf of the same matrix, through the whole factorisation."""
    from lightcompress_b200 import GPTQ, IntegerQuantizer
    n = 2304
    g = torch.Generator().manual_seed(n)
    X = torch.randn(3 * n, n, generator=g)
    X[:, torch.randperm(n, generator=g)[:23]] *= 20
    H = (X.t() @ X).cuda()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    facs = []
    for min_n in (1024, 1 << 30):
        solver = GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'blocked_cholesky_min': min_n})
        facs.append(solver.factorize(H, 2.0 / 3))
        solver.check_status()
    U1, U2 = facs[0]['U'], facs[1]['U']
    rel = float((U1 - U2).abs().max() / U2.abs().max())
    perm = facs[0]['perm']
    Hp = (H.double() * (2.0 / 3))[perm][:, perm]
    Hp += torch.eye(n, device='cuda', dtype=torch.float64) * 0.01 * Hp.diagonal().mean()
    eye = torch.eye(n, device='cuda', dtype=torch.float64)
    r1 = float(((U1.double().t() @ U1.double()) @ Hp - eye).abs().max())
    r2 = float(((U2.double().t() @ U2.double()) @ Hp - eye).abs().max())
    print(f'blocked Cholesky vs potrf: max rel diff of U {rel:.2e}; residual {r1:.2e} vs {r2:.2e}')
    assert torch.equal(U1, torch.triu(U1))
    assert rel < 1e-4 and r1 < max(6 * r2, 1e-3)


def test_native_factorisation_reports_not_positive_definite():
    from lightcompress_b200 import GPTQ, IntegerQuantizer
    n = 256
    H = -torch.eye(n).cuda()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    solver = GPTQ(wq, {'actorder': False, 'percdamp': 0.0, 'factorization': 'native_full'})
    solver.factorize(H, 1.0)
    with pytest.raises(torch.linalg.LinAlgError):
        solver.check_status()
    solver = GPTQ(wq, {'actorder': False, 'percdamp': 0.0, 'factorization': 'native'})
    solver.factorize(H, 1.0)           # asynchronous: potrf's info word is read at check_status()
    with pytest.raises(torch.linalg.LinAlgError):
        solver.check_status()


@pytest.mark.parametrize('R,C', [(512, 2048)])
def test_solver_codes_native_vs_cusolver_factor(R, C):
    """weight_transform on the native factor against the cuSOLVER factor: < 0.1 % of the codes differ."""
    from lightcompress_b200 import GPTQ, IntegerQuantizer
    g = torch.Generator().manual_seed(77)
    W = (torch.randn(R, C, generator=g) * 0.02).to(torch.bfloat16).cuda()
    X = torch.randn(3 * C, C, generator=g)
    X[:, torch.randperm(C, generator=g)[:C // 100]] *= 20
    H = (X.t() @ X).cuda()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    res = {}
    for mode in ('native', 'direct'):
        solver = GPTQ(wq, {'actorder': True, 'percdamp': 0.01, 'factorization': mode})
        res[mode] = solver.solve(W, H, 2.0 / 3)
        solver.check_status()
    mism = float((res['native']['codes_perm'] != res['direct']['codes_perm']).float().mean())
    print(f'R={R} C={C}: codes on the native factor vs the cuSOLVER factor: mismatch {mism:.5%}')
    assert mism < 1e-3
