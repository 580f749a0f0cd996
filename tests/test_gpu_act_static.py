"""Static per-tensor activation quantisation on the GPU: batched range kernel, moving average and the
static fake quant, against the committed reference outputs, the CPU oracle and the stock torch ops
the reference would run on the same GPU.  Integer / min-max work: everything is compared bit for bit."""
import pytest
import torch

from oracle import quant_ref

pytestmark = pytest.mark.gpu


def _quantizer(c):
    from lightcompress_b200 import IntegerQuantizer
    return IntegerQuantizer(c['bit'], c['sym'], 'per_tensor', calib_algo=c['algo'])


def _same(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape, (a.dtype, b.dtype, a.shape, b.shape)
    assert torch.equal(a.cpu(), b.cpu())


def test_batch_qparams_and_static_fake_quant_match_reference(golden):
    for key, c in golden('act_static.pt').items():
        qz = _quantizer(c)
        sl, zl, qminl, qmaxl = qz.get_batch_tensors_qparams([a.cuda() for a in c['acts']])
        assert len(sl) == 1
        _same(sl[0], c['scales'])
        _same(zl[0], c['zeros'])
        # like register_act_qparams (base_blockwise_quantization.py:597-611) the buffers live on the GPU
        args = {'scales': sl[0].cuda(), 'zeros': zl[0].cuda(), 'qmax': qmaxl[0].cuda(), 'qmin': qminl[0].cuda()}
        x = c['x'].cuda()
        fq = qz.fake_quant_act_static(x, args)
        # the ops the reference runs on those CUDA buffers (quant.py:698-716)
        stock = ((torch.clamp(torch.round(x / args['scales']) + args['zeros'], args['qmin'], args['qmax'])
                  - args['zeros']) * args['scales']).to(x.dtype)
        _same(fq, stock)
        # A 0-dim fp32 CUDA buffer is cast to the activation dtype by the tensor ops; on the CPU, where the
        # fixture was made, it stays fp32.  The two agree when the scale is a value of the activation dtype.
        s_cast = sl[0].to(c['dtype'])
        if torch.equal(s_cast.float().cpu(), sl[0].float().cpu()):
            _same(fq, c['fake'])
        ref = quant_ref.int_fake_quant_static(c['x'], s_cast.cpu(), zl[0].cpu(), c['bit'], c['sym'], 'per_tensor')
        _same(fq, ref)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
def test_ranges_of_large_and_ragged_tensors(dtype):
    """More tensors than one launch takes (64), sizes that are not whole chunks, an unaligned view, NaN."""
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator(device='cuda').manual_seed(31)
    qz = IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_minmax')
    big = torch.randn(70, 300, 1031, generator=g, device='cuda').to(dtype)
    tensors = [big[i] for i in range(70)]
    tensors.append(torch.randn(5, generator=g, device='cuda').to(dtype))
    tensors.append(torch.randn(2 * 16384 + 1, generator=g, device='cuda').to(dtype)[1:])     # not 16-byte aligned
    withnan = torch.randn(40000, generator=g, device='cuda').to(dtype)
    withnan[12345] = float('nan')
    tensors.append(withnan)
    tensors.append(torch.full((3, 7), -2.5, device='cuda', dtype=dtype))
    mins, maxs, _ = qz._tensor_ranges(tensors)
    for i, t in enumerate(tensors):
        assert torch.equal(mins[i].to(dtype), torch.min(t)) or (torch.isnan(mins[i]) and torch.isnan(torch.min(t))), i
        assert torch.equal(maxs[i].to(dtype), torch.max(t)) or (torch.isnan(maxs[i]) and torch.isnan(torch.max(t))), i
    assert torch.isnan(mins[72]) and torch.isnan(maxs[72])
    mn, mx = qz.get_minmax_range(tensors[3])
    assert mn.dtype == dtype and mn.dim() == 0 and torch.equal(mn, torch.min(tensors[3])) and torch.equal(
        mx, torch.max(tensors[3]))


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('algo', ['static_minmax', 'static_moving_minmax'])
def test_static_ranges_equal_the_oracle_and_the_stock_ops(dtype, algo):
    from lightcompress_b200 import IntegerQuantizer
    g = torch.Generator().manual_seed(77)
    acts = [(torch.randn(2, 256, 512, generator=g) * (1 + 0.1 * i) - 0.05 * i).to(dtype) for i in range(33)]
    for sym in (True, False):
        qz = IntegerQuantizer(8, sym, 'per_tensor', calib_algo=algo)
        sl, zl, _, _ = qz.get_batch_tensors_qparams([a.cuda() for a in acts], alpha=0.01)
        (s, z, _, _), = quant_ref.batch_tensors_qparams(acts, 8, sym, algo, alpha=0.01)
        _same(sl[0], s)
        _same(zl[0], z)
        if algo == 'static_moving_minmax':
            # the reference's own chain of 0-dim CUDA ops
            m_min = m_max = None
            for a in acts:
                a = a.cuda()
                mn, mx = torch.min(a), torch.max(a)
                if m_min is None:
                    m_min, m_max = mn, mx
                else:
                    m_min = m_min + 0.01 * (mn - m_min)
                    m_max = m_max + 0.01 * (mx - m_max)
            mins, maxs = qz.get_static_moving_minmax_range([a.cuda() for a in acts], 0.01)
            _same(mins[0], m_min)
            _same(maxs[0], m_max)
    # a single batched tensor is split along its first dim (quant.py:116-119); tuples are stacked per input
    qz = IntegerQuantizer(8, True, 'per_tensor', calib_algo=algo)
    one = torch.stack(acts[:4]).cuda()
    a1 = qz.get_batch_tensors_qparams([one])[0][0]
    a2 = qz.get_batch_tensors_qparams([t.cuda() for t in acts[:4]])[0][0]
    _same(a1, a2)
    pairs = [(acts[i].cuda(), acts[i + 1].cuda()) for i in range(0, 6, 2)]
    sl2 = qz.get_batch_tensors_qparams(pairs)[0]
    assert len(sl2) == 2
    _same(sl2[0], qz.get_batch_tensors_qparams([p[0] for p in pairs])[0][0])
    _same(sl2[1], qz.get_batch_tensors_qparams([p[1] for p in pairs])[0][0])


def test_range_kernel_bandwidth():
    """One launch over 16 x 64 MB of bf16 activations (larger than L2), reported in GB/s."""
    from lightcompress_b200 import IntegerQuantizer
    qz = IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_minmax')
    acts = [torch.randn(4, 2048, 4096, device='cuda', dtype=torch.bfloat16) for _ in range(16)]
    for _ in range(3):
        qz._tensor_ranges(acts)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(5):
        qz._tensor_ranges(acts)
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 5
    nbytes = sum(a.numel() * 2 for a in acts)
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(5):
        for a in acts:
            torch.max(a)
            torch.min(a)
    ev[1].record()
    torch.cuda.synchronize()
    ms_t = ev[0].elapsed_time(ev[1]) / 5
    print(f'lc_act_range_per_tensor: {ms:.3f} ms for {nbytes / 1e9:.2f} GB = {nbytes / ms / 1e6:.0f} GB/s; '
          f'torch.max + torch.min per tensor: {ms_t:.3f} ms')
    assert ms < ms_t
