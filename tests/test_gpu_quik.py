"""QUIK on the GPU through the C ABI: activation statistic, column split and the masked mixed-precision
fake quant, bit-exact against the committed reference outputs and the CPU oracle."""
import pytest
import torch

from oracle import quant_ref

pytestmark = pytest.mark.gpu


def _quik(sym, wbit=4, abit=8, fp_features=24, threshold=0.0):
    from lightcompress_b200 import IntegerQuantizer
    from lightcompress_b200.quik import QUIK
    return QUIK(IntegerQuantizer(wbit, sym, 'per_channel'), IntegerQuantizer(abit, sym, 'per_token'),
                {'fp_relative': False, 'fp_features': fp_features, 'fp_threshold': threshold})


def test_quik_matches_reference_golden(golden):
    for key, c in golden('quik_mixed.pt').items():
        q = _quik(c['sym'], c['wbit'], c['abit'], c['fp_ids'].numel())
        hidden = c['w'].shape[1]
        lin = torch.nn.Linear(hidden, c['w'].shape[0], bias=False, dtype=c['w'].dtype).cuda()
        lin.weight.data = c['w'].cuda()
        root = torch.nn.ModuleDict({'fc': lin})
        hooks = q.register_hooks(root, prefix='model.layers.0')
        for a in c['acts']:
            lin(a.cuda())
        for h in hooks:
            h.remove()
        assert torch.equal(q.act_scales['model.layers.0.fc'].cpu(), c['stat']), key
        q.block_opt({'fc': lin}, 'model.layers.0')
        assert torch.equal(lin.buf_int_ids.cpu(), c['int_ids']) and torch.equal(lin.buf_fp_ids.cpu(), c['fp_ids']), key
        fw = q.w_qdq(lin, q.wquantizer)
        fa = q.a_qdq(c['acts'][0].cuda(), lin, q.aquantizer)
        assert fw.dtype == c['fake_w'].dtype and torch.equal(fw.cpu(), c['fake_w']), key
        assert fa.shape == c['fake_a'].shape and torch.equal(fa.cpu(), c['fake_a']), key


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('sym', [True, False])
def test_masked_fake_quant_vs_oracle(dtype, sym):
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(91)
    for rows, cols, n_fp in ((96, 4096, 256), (17, 11008, 256), (300, 264, 8)):
        t = torch.randn(rows, cols, generator=g) * 0.1
        t[:, ::53] *= 30
        t = t.to(dtype)
        order = torch.randperm(cols, generator=g)
        int_ids, fp_ids = order[:-n_fp], order[-n_fp:]
        for bit, gran in ((4, 'per_channel'), (8, 'per_token')):
            ref = quant_ref.int_fake_quant_mixed(t, bit, sym, gran, int_ids, fp_ids)
            qz = IntegerQuantizer(bit, sym, gran)
            out = qz.fake_quant_weight_dynamic(t.cuda(), {'int_indices': int_ids.cuda(), 'fp_indices': fp_ids.cuda()})
            assert torch.equal(out.cpu(), ref), (dtype, sym, rows, cols, bit)
    # columns in neither list come out zero, like the reference's zeros_like + scatters
    t = torch.randn(8, 64, generator=g).to(dtype)
    int_ids, fp_ids = torch.arange(0, 40), torch.arange(48, 64)
    ref = quant_ref.int_fake_quant_mixed(t, 8, sym, 'per_token', int_ids, fp_ids)
    out = IntegerQuantizer(8, sym, 'per_token').fake_quant_act_dynamic(
        t.cuda().reshape(2, 4, 64), {'int_indices': int_ids.cuda(), 'fp_indices': fp_ids.cuda()})
    assert torch.equal(out.cpu().reshape(8, 64), ref)
    with pytest.raises(NotImplementedError):
        IntegerQuantizer(4, sym, 'per_group', group_size=8).fake_quant_weight_dynamic(
            t.cuda(), {'int_indices': int_ids.cuda(), 'fp_indices': fp_ids.cuda()})


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_col_absmax_vs_oracle_and_bandwidth(dtype):
    q = _quik(True)
    g = torch.Generator(device='cuda').manual_seed(5)
    xs = [torch.randn(3, 1000 + 37 * i, 4096, generator=g, device='cuda').to(dtype) for i in range(4)]
    xs[2][1, 5, 77] = float('nan')
    stat = None
    for x in xs:
        q.get_tensor_scale('l', x)
        stat = quant_ref.quik_col_absmax(stat, x.cpu())
    got = q.act_scales['l'].cpu()
    same = (got == stat) | (torch.isnan(got) & torch.isnan(stat))
    assert bool(same.all()) and bool(torch.isnan(got[77]))
    big = torch.randn(65536, 4096, device='cuda').to(dtype)
    for _ in range(3):
        q.get_tensor_scale('b', big)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(5):
        q.get_tensor_scale('b', big)
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 5
    print(f'lc_quik_col_absmax 65536x4096 {dtype}: {ms:.3f} ms = {big.numel() * big.element_size() / ms / 1e6:.0f} GB/s')


def test_masked_fake_quant_bandwidth():
    from lightcompress_b200 import IntegerQuantizer
    x = torch.randn(32768, 4096, device='cuda', dtype=torch.bfloat16)
    order = torch.randperm(4096, device='cuda')
    args = {'int_indices': order[:-256], 'fp_indices': order[-256:]}
    qz = IntegerQuantizer(8, True, 'per_token')
    for _ in range(3):
        qz.fake_quant_act_dynamic(x, args)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(10):
        qz.fake_quant_act_dynamic(x, args)
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 10
    print(f'lc_rtn_int_fake_quant_masked 32768x4096 bf16: {ms:.3f} ms = {2 * x.numel() * 2 / ms / 1e6:.0f} GB/s')


def test_quik_without_outliers_stops_like_the_reference():
    q = _quik(True, fp_features=0)
    lin = torch.nn.Linear(64, 8, bias=False).cuda()
    with pytest.raises(TypeError):
        q.block_opt({'fc': lin}, 'model.layers.0')
