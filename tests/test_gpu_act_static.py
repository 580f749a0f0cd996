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


def test_histogram_kernel_equals_torch_histc_on_this_gpu():
    """lc_act_hist_per_tensor against torch.histc on the same GPU (what the reference calls there), bin
    for bin: ranges wider than the data, equal to it (x == max lands in the last bin), and narrower."""
    import ctypes
    from lightcompress_b200 import _lib as L
    g = torch.Generator().manual_seed(2400)
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        ts = [(torch.randn(n, generator=g) * sc).to(dtype).cuda() for n, sc in ((300001, 1.0), (4096, 3.0), (77, 0.5),
                                                                                (1 << 21, 1.7))]
        mins = torch.tensor([float(ts[0].min()), -20.0, float(ts[2].min()), -2.0], device='cuda')
        maxs = torch.tensor([float(ts[0].max()), 25.0, float(ts[2].max()), 2.5], device='cuda')
        n = len(ts)
        hist = torch.empty((n, 2048), device='cuda')
        ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
        numels = (ctypes.c_int64 * n)(*[t.numel() for t in ts])
        L.call('lc_act_hist_per_tensor', ptrs, numels, n, L.lc_dtype(ts[0]), L.ptr(mins), L.ptr(maxs), 2048,
               L.ptr(hist), L.stream_of(ts[0]))
        for i, t in enumerate(ts):
            want = torch.histc(t.float(), 2048, min=float(mins[i]), max=float(maxs[i]))
            assert torch.equal(hist[i], want), (dtype, i, int((hist[i] != want).sum()))


def test_static_hist_qparams_match_oracle_and_golden(golden):
    """calib_algo 'static_hist' end to end: the searched range, the scale and the fake-quantised activations
    against the oracle evaluated on the same GPU (torch.histc there), and against the reference's CPU
    fixture where CPU and CUDA histc bin alike."""
    from lightcompress_b200 import IntegerQuantizer
    for key, c in golden('act_hist.pt').items():
        acts = [a.cuda() for a in c['acts']]
        qz = IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_hist')
        mins, maxs = qz.get_static_hist_range([a.clone() for a in acts])
        rmin, rmax = quant_ref.static_hist_range([a.clone() for a in acts], 8)
        assert torch.equal(mins[0], rmin[0]) and torch.equal(maxs[0], rmax[0]), (key, mins, rmin, maxs, rmax)
        sl, zl, qminl, qmaxl = qz.get_batch_tensors_qparams([a.clone() for a in acts])
        (s, z, qmax, qmin), = quant_ref.batch_tensors_qparams([a.clone() for a in acts], 8, True, 'static_hist')
        assert torch.equal(sl[0].cpu(), s.cpu())
        fq = qz.fake_quant_act_static(c['x'].cuda(), {'scales': sl[0], 'zeros': zl[0], 'qmax': qmaxl[0], 'qmin': qminl[0]})
        same = bool(torch.equal(sl[0].cpu(), c['scales']))
        print(f'static_hist {key}: range [{float(mins[0]):.5f}, {float(maxs[0]):.5f}], scale equal to the CPU fixture: {same}')
        # the static fake quant against the stock tensor ops with the scale as a 0-dim CUDA buffer (how the
        # reference holds it at deploy time; its CUDA kernels cast such a scale to the activation dtype, its
        # CPU kernels do not, so the CPU fixture only applies to fp32 activations)
        s_dev = sl[0].cuda()
        xq = c['x'].cuda()
        stock = torch.clamp(torch.round(xq / s_dev), qminl[0].cuda(), qmaxl[0].cuda()) * s_dev
        assert torch.equal(fq, stock.to(fq.dtype))
        if same and c['dtype'] == torch.float32:
            assert torch.equal(fq.cpu(), c['fake'])
