"""Weight48IntegerQuantizer (two-level 8 -> 4 bit fake quant) on the GPU through the C ABI: bit-exact
against the committed reference outputs and, on larger weights, against the CPU oracle."""
import pytest
import torch

from oracle import quant_ref

pytestmark = pytest.mark.gpu

BIT4 = {'symmetric': False, 'granularity': 'per_group', 'group_size': 128, 'scales_bit': 8,
        'scales_symmetric': True, 'zeros_bit': 8, 'zeros_symmetric': True}
BIT8 = {'symmetric': True, 'granularity': 'per_channel', 'int_range': [-120, 120]}


def _run(w, bit4, bit8):
    from lightcompress_b200 import Weight48IntegerQuantizer
    qz = Weight48IntegerQuantizer(48, dict(bit4), dict(bit8))
    out = qz.fake_quant_weight_dynamic(w.cuda())
    torch.cuda.synchronize()
    return out.cpu()


def test_w48_matches_reference_golden(golden):
    for key, c in golden('rtn_w48.pt').items():
        out = _run(c['w'], c['bit4'], c['bit8'])
        assert out.dtype == c['fake'].dtype and torch.equal(out, c['fake']), key


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('R,C', [(64, 4096), (33, 11008), (7, 128), (16, 16384)])
def test_w48_vs_oracle(dtype, R, C):
    g = torch.Generator().manual_seed(R * 131 + C)
    w = torch.randn(R, C, generator=g) * 0.03
    w[:, ::97] *= 8
    w[0] = 0
    w[1, :256] = float('nan') if R > 1 else 0
    w = w.to(dtype)
    for bit4 in (BIT4, {'symmetric': True, 'granularity': 'per_group', 'group_size': 128}):
        for bit8 in (BIT8, {'symmetric': False, 'granularity': 'per_channel'}):
            ref = quant_ref.w48_fake_quant(w, bit4, bit8)
            out = _run(w, bit4, bit8)
            same = (out == ref) | (torch.isnan(out) & torch.isnan(ref))
            assert bool(same.all()), (dtype, R, C, bit4['symmetric'], bit8['symmetric'], int((~same).sum()))


def test_w48_rejects_what_the_reference_rejects():
    from lightcompress_b200 import Weight48IntegerQuantizer
    qz = Weight48IntegerQuantizer(48, dict(BIT4), dict(BIT8))
    with pytest.raises(ValueError):
        qz.fake_quant_weight_dynamic(torch.zeros(4, 200, device='cuda', dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        Weight48IntegerQuantizer(4, dict(BIT4), dict(BIT8))


def test_w48_bandwidth():
    """16384 x 8192 bf16 (268 MB, larger than L2): read + write once."""
    from lightcompress_b200 import Weight48IntegerQuantizer
    qz = Weight48IntegerQuantizer(48, dict(BIT4), dict(BIT8))
    w = torch.randn(16384, 8192, device='cuda', dtype=torch.bfloat16)
    for _ in range(3):
        qz.fake_quant_weight_dynamic(w)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(10):
        qz.fake_quant_weight_dynamic(w)
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 10
    print(f'lc_rtn_w48_fake_quant 16384x8192 bf16: {ms:.3f} ms = {2 * w.numel() * 2 / ms / 1e6:.0f} GB/s')
