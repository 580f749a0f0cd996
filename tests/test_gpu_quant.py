"""GPU parity of the fused quant / dequant kernels, called through the C ABI, against the
committed reference outputs (tests/golden) and against the CPU oracle on seeded inputs.
Integer and byte results are compared bit for bit."""
import pytest
import torch

from oracle import quant_ref

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


def _same(a, b, what=''):
    a = a.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape, (what, a.dtype, b.dtype, a.shape, b.shape)
    if a.is_floating_point() and a.dtype != torch.float8_e4m3fn:
        # compare bit patterns, but let +0 == -0 and NaN == NaN like torch.equal would not
        ia = a.contiguous().view(torch.int32 if a.dtype == torch.float32 else torch.int16)
        ib = b.contiguous().view(ia.dtype)
        bad = (ia != ib) & ~((a == 0) & (b == 0)) & ~(a.isnan() & b.isnan())
        assert not bad.any(), f'{what}: {int(bad.sum())} of {a.numel()} elements differ'
    else:
        assert torch.equal(_bits(a), _bits(b)), what


def test_rtn_matches_reference_golden(golden):
    from lightcompress_b200 import IntegerQuantizer
    for key, c in golden('rtn_int.pt').items():
        kw = {'group_size': c['group_size']} if c['group_size'] else {}
        qz = IntegerQuantizer(c['bit'], c['sym'], c['granularity'], **kw)
        w = c['w'].cuda()
        if 'codes' in c:
            _same(qz.fake_quant_weight_dynamic(w), c['fake'], key + ' fake')
            codes, s, z = qz.real_quant_weight_dynamic(w)
            _same(codes, c['codes'], key + ' codes')
            _same(s, c['scales'], key + ' scales')
            if c['sym']:
                assert z is None
            else:
                _same(z, c['zeros'], key + ' zeros')
            # static path reproduces the dynamic one when fed the same parameters
            t, s2, z2, qmax, qmin = qz.get_tensor_qparams(w)
            _same(s2.reshape(s.shape), c['scales'], key + ' qparams')
            fq = qz.fake_quant_weight_static(w, {'scales': s2, 'zeros': z2, 'qmax': qmax, 'qmin': qmin})
            _same(fq, c['fake'], key + ' static')
        else:
            _same(qz.fake_quant_act_dynamic(w), c['fake'], key + ' act')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize('shape,gran,gs', [((4096, 4096), 'per_group', 128), ((512, 11008), 'per_group', 128),
                                           ((300, 4096), 'per_channel', None), ((64, 11008), 'per_channel', None),
                                           ((7, 33, 1408), 'per_token', None), ((5, 1000), 'per_token', None),
                                           ((16, 96), 'per_group', 32), ((3, 130), 'per_channel', None)])
def test_rtn_matches_oracle(dtype, shape, gran, gs):
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(1000 + len(shape) + shape[-1])
    w = (torch.randn(*shape, generator=g) * 0.02).to(dtype)
    for sym, bit in ((False, 4), (True, 4), (False, 8), (True, 8)):
        kw = {'group_size': gs} if gs else {}
        qz = IntegerQuantizer(bit, sym, gran, **kw)
        wc = w.cuda()
        _same(qz.fake_quant_weight_dynamic(wc), quant_ref.int_fake_quant_dynamic(w, bit, sym, gran, gs), 'fake')
        if w.dim() == 2:
            q, s, z = quant_ref.int_real_quant_dynamic(w, bit, sym, gran, gs)
            codes, s2, z2 = qz.real_quant_weight_dynamic(wc)
            _same(codes, q, 'codes')
            _same(s2, s, 'scales')
            if not sym:
                _same(z2, z, 'zeros')
            if bit == 4 and shape[-1] % 2 == 0:
                fake, packed, s3, z3 = qz.quant_all_dynamic(wc, packed=True)
                off = 8 if sym else 0
                _same(packed, quant_ref.pack_int4_rows((q + off).to(torch.uint8)), 'packed')
                _same(s3, s, 'scales(all)')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_rtn_rounding_boundaries_are_exact(dtype):
    """Elements placed within a few ulps of every rounding boundary of w / s (half-integers, and
    for bf16 the bf16 rounding midpoints): the reciprocal-based division must agree with the IEEE
    division of the reference on each of them."""
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(1234)
    rows = 4096
    s0 = (torch.rand(rows, 1, generator=g) * 0.05 + 1e-3)
    k = torch.randint(0, 15, (rows, 128), generator=g).float()
    w = (k + 0.5) * s0
    # walk a few ulps around each boundary
    steps = torch.randint(-3, 4, (rows, 128), generator=g, dtype=torch.int32)
    wi = w.view(torch.int32) + steps
    w = wi.view(torch.float32).clone()
    w[:, 0] = 0.0
    w[:, 1] = 15.0 * s0[:, 0]          # pins min = 0, max = 15 s0 so that the scale is ~s0
    w = w.to(dtype)
    if dtype == torch.bfloat16:
        # also sit on bf16 midpoints of the quotient: w = s * (m + half-ulp), a few fp32 ulps around
        s_b = w[:, 1:2].float() / 15
        m = torch.randint(64, 128, (rows, 64), generator=g).float() / 8   # bf16-representable quotients
        mid = (m + 1.0 / 32) * s_b                                          # half a bf16 ulp above (ulp = 1/16)
        w[:, 64:] = mid.to(dtype)
    for sym, bit in ((False, 4), (False, 8), (True, 4)):
        qz = IntegerQuantizer(bit, sym, 'per_group', group_size=128)
        q, sc, z = quant_ref.int_real_quant_dynamic(w, bit, sym, 'per_group', 128)
        codes, s2, z2 = qz.real_quant_weight_dynamic(w.cuda())
        _same(codes, q, 'codes')
        _same(s2, sc, 'scales')
        _same(qz.fake_quant_weight_dynamic(w.cuda()), quant_ref.int_fake_quant_dynamic(w, bit, sym, 'per_group', 128),
              'fake')
    # non-finite and huge inputs take the exact path
    w2 = (torch.randn(64, 256, generator=g)).to(dtype)
    w2[0, 3] = float('inf')
    w2[1, 7] = float('nan')
    w2[2, :128] = 3e37 if dtype == torch.float32 else 3e37
    w2[3, :] = 0
    qz = IntegerQuantizer(4, False, 'per_group', group_size=128)
    _same(qz.fake_quant_weight_dynamic(w2.cuda()), quant_ref.int_fake_quant_dynamic(w2, 4, False, 'per_group', 128),
          'non-finite')


def test_rtn_full_size_roundtrip_property():
    """Config-1 size: quantising the dequantised output again is a fixed point for the codes."""
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(1001)
    w = (torch.randn(4096, 4096, generator=g) * 0.02).cuda()
    qz = IntegerQuantizer(4, False, 'per_group', group_size=128)
    fake, codes, s, z = qz.quant_all_dynamic(w)
    assert int(codes.min()) >= 0 and int(codes.max()) <= 15
    deq = ((codes.float().reshape(-1, 128) - z.reshape(-1, 1).float()) * s.reshape(-1, 1)).reshape(w.shape)
    assert torch.equal(deq, fake)
    assert float((fake - w).abs().max()) <= float(s.max()) * 0.5 + 1e-7


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('sym', [False, True])
@pytest.mark.parametrize('gran,gs,shape', [('per_group', 128, (256, 1024)), ('per_channel', None, (192, 512)),
                                           ('per_channel', None, (64, 2048))])
def test_mse_range_matches_oracle_on_the_gpu(dtype, sym, gran, gs, shape):
    """lc_rtn_mse_range against the oracle's chain of torch ops run on the same GPU: the same powf, the
    same association of the group sums, so ranges and fake-quantised weights are equal bit for bit."""
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    w = torch.randn(*shape, generator=g) * 0.02
    w += torch.randn(*shape, generator=g) * 0.2 * (torch.rand(*shape, generator=g) > 0.98)   # outliers worth clipping
    w[0] = 0.0
    w = w.to(dtype).cuda()
    kw = {'group_size': gs} if gs else {}
    qz = IntegerQuantizer(4, sym, gran, calib_algo='mse', **kw)
    grouped = quant_ref.group_view(w, gran, gs)
    mn, mx = qz.get_tensor_range(qz.reshape_tensor(w))
    rmn, rmx = quant_ref.mse_range(grouped, 4, sym)
    frac = float(((mn != rmn) | (mx != rmx)).float().mean())
    shrunk = float((rmx != grouped.float().amax(-1, keepdim=True)).float().mean())
    print(f'{dtype} sym={sym} {gran}: {frac:.4%} of the ranges differ; {shrunk:.1%} of the groups were shrunk')
    assert shrunk > 0.2
    assert frac == 0.0
    fake = qz.fake_quant_weight_dynamic(w)
    assert fake.dtype == w.dtype
    assert torch.equal(fake, quant_ref.int_fake_quant_mse(w, 4, sym, gran, gs))
    t, s, z, qmax, qmin = qz.get_tensor_qparams(w)
    rs, rz, _, _ = quant_ref.int_qparams_from_range(rmn, rmx, 4, sym)
    assert torch.equal(s, rs) and (sym or torch.equal(z, rz)) and s.dtype == torch.float32


def test_mse_range_against_the_reference_golden(golden):
    """Against the reference's own CPU result: CPU and GPU differ in powf and in the order of the
    group sums, which can move a near-tie of the error curve to a neighbouring grid step."""
    from lightcompress_b200 import IntegerQuantizer
    n = bad = 0
    for key, c in golden('rtn_mse.pt').items():
        kw = {'group_size': c['group_size']} if c['group_size'] else {}
        if c['granularity'] == 'per_channel' and c['w'].shape[-1] % 128:
            continue
        qz = IntegerQuantizer(c['bit'], c['sym'], c['granularity'], calib_algo='mse', **kw)
        w = c['w'].cuda()
        mn, mx = qz.get_tensor_range(qz.reshape_tensor(w))
        diff = (mn.cpu() != c['min']) | (mx.cpu() != c['max'])
        n += diff.numel()
        bad += int(diff.sum())
        fake = qz.fake_quant_weight_dynamic(w).cpu()
        # where the range agrees the fake-quantised group agrees bit for bit
        g_fake = quant_ref.group_view(fake, c['granularity'], c['group_size'])
        g_ref = quant_ref.group_view(c['fake'], c['granularity'], c['group_size'])
        same = ~diff.view(-1)
        assert torch.equal(g_fake[same], g_ref[same]), key
    print(f'mse ranges vs the CPU reference: {bad} of {n} groups on another grid step')
    assert n > 0 and bad <= 0.02 * n


def test_fp8_matches_reference_golden_and_oracle(golden):
    from lightcompress_b200 import FloatQuantizer
    for key, c in golden('fp8_e4m3.pt').items():
        qw = FloatQuantizer('e4m3', True, 'per_channel', use_qtorch=True)
        qa = FloatQuantizer('e4m3', True, 'per_token', use_qtorch=True)
        _same(qw.fake_quant_weight_dynamic(c['w'].cuda()), c['fake'], key + ' fake')
        codes, s, z = qw.real_quant_weight_dynamic(c['w'].cuda())
        assert z is None
        _same(codes.view(torch.uint8), c['codes'], key + ' codes')
        _same(s, c['scales'], key + ' scales')
        _same(qa.fake_quant_act_dynamic(c['x'].cuda()), c['fake_act'], key + ' act')
    g = torch.Generator().manual_seed(5002)
    for dtype in (torch.bfloat16, torch.float32, torch.float16):
        for shape in ((1408, 2048), (2048, 1408), (37, 1001), (16, 11008)):
            w = (torch.randn(*shape, generator=g)).to(dtype)
            qw = FloatQuantizer('e4m3', True, 'per_channel', use_qtorch=True)
            _same(qw.fake_quant_weight_dynamic(w.cuda()), quant_ref.fp8_fake_quant_dynamic(w), 'fp8 fake')
            q, s = quant_ref.fp8_real_quant_dynamic(w)
            codes, s2, _ = qw.real_quant_weight_dynamic(w.cuda())
            _same(codes.view(torch.uint8), q.view(torch.uint8), 'fp8 codes')
            _same(s2, s, 'fp8 scales')


def test_fp8_block_wise_matches_reference_golden_and_oracle(golden):
    """128 x 128 block-wise e4m3 weights: codes, fp32 scales, dequantised bf16 and fake-quantised weights
    against the reference's CPU result (fixtures) and against the oracle on larger seeded tensors."""
    from lightcompress_b200 import FloatQuantizer
    from lightcompress_b200.quant import weight_cast_to_bf16, weight_cast_to_fp8
    for key, c in golden('fp8_block.pt').items():
        w = c['w'].cuda()
        codes, scales = weight_cast_to_fp8(w, 128)
        assert torch.equal(codes.cpu().view(torch.uint8), c['codes']), key
        _same(scales, c['scales'], key)
        _same(weight_cast_to_bf16(codes, scales, 128), c['back'], key)
        qz = FloatQuantizer('e4m3', True, 'per_block', block_size=128, use_qtorch=True)
        _same(qz.fake_quant_weight_dynamic(w), c['fake'], key)
    g = torch.Generator().manual_seed(88)
    for dtype, shape in ((torch.bfloat16, (1408, 2048)), (torch.float16, (1000, 1024)), (torch.float32, (512, 700)),
                         (torch.bfloat16, (384, 1001))):
        w = (torch.randn(*shape, generator=g) * 0.05).to(dtype)
        w[:, ::97] *= 40
        codes, scales = weight_cast_to_fp8(w.cuda(), 128)
        rc, rs = quant_ref.fp8_block_real_quant(w)
        assert torch.equal(codes.cpu().view(torch.uint8), rc.view(torch.uint8)), (dtype, shape)
        _same(scales, rs)
        _same(weight_cast_to_bf16(codes, scales), quant_ref.fp8_block_dequant(rc, rs))
        qz = FloatQuantizer('e4m3', True, 'per_block', block_size=128, use_qtorch=True)
        _same(qz.fake_quant_weight_dynamic(w.cuda()), quant_ref.fp8_block_fake_quant(w))
    with pytest.raises(RuntimeError):
        weight_cast_to_fp8(torch.zeros(130, 130, device='cuda'), 128)
    # per-token-group activations (1 x 128 groups): every group is a row of the per-row kernel
    x = torch.randn(4, 33, 512, generator=g).to(torch.bfloat16)
    qa = FloatQuantizer('e4m3', True, 'per_group', group_size=128, use_qtorch=True)
    ref = quant_ref.fp8_fake_quant_dynamic(x.reshape(-1, 128)).reshape(x.shape)
    _same(qa.fake_quant_act_dynamic(x.cuda()), ref)


def test_export_packing_layouts():
    """compressed-tensors int4 (LC_CODES_PACK4 viewed as int32) and the AutoAWQ GEMM layout against
    restatements of the reference's packers."""
    from lightcompress_b200 import IntegerQuantizer
    from lightcompress_b200.export import pack_autoawq_gemm, pack_compressed_tensors_int4
    g = torch.Generator().manual_seed(6001)
    w = (torch.randn(256, 512, generator=g) * 0.02).to(torch.bfloat16)
    qs = IntegerQuantizer(4, True, 'per_group', group_size=128)
    packed, s = pack_compressed_tensors_int4(w.cuda(), qs)
    q, s_ref, _ = quant_ref.int_real_quant_dynamic(w, 4, True, 'per_group', 128)
    assert torch.equal(packed.cpu(), quant_ref.pack_compressed_tensors(q))
    _same(s, s_ref, 'scales')
    # static scales on an fp32 weight: the export of a GPTQ layer solved with static_groups
    from lightcompress_b200.export import pack_compressed_tensors_int4_static
    w32 = (w.float() + 0.003 * torch.randn(256, 512, generator=g))
    packed2, s_back = pack_compressed_tensors_int4_static(w32.cuda(), s, qs)
    q2 = quant_ref.int_quant(w32.reshape(-1, 128), s_ref.reshape(-1, 1), torch.tensor(0.0), *reversed(
        quant_ref.int_range(4, True))).reshape(256, 512)
    assert torch.equal(packed2.cpu(), quant_ref.pack_compressed_tensors(q2))
    assert s_back.shape == (256, 4)
    qa = IntegerQuantizer(4, False, 'per_group', group_size=128)
    codes, s2, z2 = qa.real_quant_weight_dynamic(w.cuda())
    qweight, qzeros = pack_autoawq_gemm(codes.to(torch.uint8), z2.to(torch.uint8))
    assert torch.equal(qweight.cpu(), quant_ref.pack_autoawq(codes.cpu().t().contiguous()))
    assert torch.equal(qzeros.cpu(), quant_ref.pack_autoawq(z2.cpu().t().contiguous()))
