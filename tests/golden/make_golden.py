"""Generates the golden fixtures in this directory by running the reference itself on CPU.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/LightCompress

The reference is imported unmodified; three process-local shims make its CUDA-only lines
run on CPU (`Tensor.cuda` -> identity, `torch.cuda.synchronize` -> no-op, a stub `accelerate`
/ `easydict` when those packages are absent) and a single-rank gloo group satisfies the
`dist.all_reduce` calls in `GPTQ.add_batch`.  The FP8 fixtures additionally substitute the
un-vendored `qtorch.quant.float_quantize` by a float8_e4m3fn round trip; they are marked
`pinned: False` for that reason.

Inputs are small and stored next to the outputs, so the tests never need the reference.
"""
import contextlib
import copy
import os
import sys
import types

import torch


def _import_reference(ref_root):
    os.environ.update(WORLD_SIZE='1', RANK='0', LOCAL_RANK='0',
                      MASTER_ADDR='127.0.0.1', MASTER_PORT='29613')
    import torch.distributed as dist
    import transformers  # noqa: F401  (must precede the accelerate stub)
    if 'accelerate' not in sys.modules:
        try:
            import accelerate  # noqa: F401
        except Exception:
            acc = types.ModuleType('accelerate')
            acc.init_empty_weights = contextlib.nullcontext
            sys.modules['accelerate'] = acc
    try:
        import easydict  # noqa: F401
    except ImportError:
        ed = types.ModuleType('easydict')

        class EasyDict(dict):
            __getattr__ = dict.__getitem__
            __setattr__ = dict.__setitem__
        ed.EasyDict = EasyDict
        sys.modules['easydict'] = ed
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.empty_cache = lambda *a, **k: None
    sys.path.insert(0, ref_root)
    if not dist.is_initialized():
        dist.init_process_group('gloo', rank=0, world_size=1)
    import llmc.compression.quantization.quant as rq
    import llmc.compression.quantization.gptq as rg
    return rq, rg


def _rtn_inputs(gen, dtype, rows, cols):
    w = (torch.randn(rows, cols, generator=gen) * 0.02)
    # edge rows: constant group (1e-5 floor), exact zeros, tiny magnitudes, wide range,
    # values on exact .5 multiples of a power-of-two step (round-half-even ties)
    w[0, :128] = 0.0137
    w[1, :] = 0.0
    w[2, :128] = torch.randn(128, generator=gen) * 1e-7
    w[3, :128] = torch.randn(128, generator=gen) * 50.0
    step = 2.0 ** -6
    w[4, :128] = (torch.arange(128) - 64).float() * step * 0.5
    w[4, 0], w[4, 127] = -7.5 * step * 1.0, 7.5 * step
    w[5, :128] = torch.linspace(0, 15, 128) * 0.25
    return w.to(dtype)


def make_rtn(rq, out_dir):
    gen = torch.Generator().manual_seed(1001)
    cases = {}
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for sym in (False, True):
            for bit in (4, 8):
                for gran, gs in (('per_group', 128), ('per_group', 64), ('per_channel', None)):
                    w = _rtn_inputs(gen, dtype, 12, 384)
                    kw = {'group_size': gs} if gs else {}
                    qz = rq.IntegerQuantizer(bit, sym, gran, **kw)
                    fq = qz.fake_quant_weight_dynamic(w.clone())
                    codes, scales, zeros = qz.real_quant_weight_dynamic(w.clone())
                    key = f'{str(dtype)[6:]}_{"sym" if sym else "asym"}_b{bit}_{gran}_{gs}'
                    cases[key] = dict(w=w, bit=bit, sym=sym, granularity=gran, group_size=gs,
                                      fake=fq, codes=codes, scales=scales, zeros=zeros)
    # per-token activations (B, T, C)
    for dtype in (torch.float32, torch.bfloat16):
        for sym in (False, True):
            x = torch.randn(2, 5, 320, generator=gen).to(dtype)
            x[0, 0, 7] = 37.0
            qz = rq.IntegerQuantizer(8, sym, 'per_token')
            fq = qz.fake_quant_act_dynamic(x.clone())
            key = f'act_{str(dtype)[6:]}_{"sym" if sym else "asym"}_b8_per_token'
            cases[key] = dict(w=x, bit=8, sym=sym, granularity='per_token', group_size=None, fake=fq)
    torch.save(cases, os.path.join(out_dir, 'rtn_int.pt'))
    print('rtn_int.pt', len(cases), 'cases')


def make_rtn_mse(rq, out_dir):
    """calib_algo 'mse': the searched ranges (get_tensor_range) and the fake-quantised weight."""
    gen = torch.Generator().manual_seed(1002)
    cases = {}
    for dtype in (torch.float32, torch.bfloat16):
        for sym in (False, True):
            for gran, gs in (('per_group', 128), ('per_channel', None)):
                w = _rtn_inputs(gen, dtype, 12, 256 if gs is None else 384)
                w[6, :128] += torch.randn(128, generator=gen) * 0.3 * (torch.rand(128, generator=gen) > 0.97)
                kw = {'group_size': gs} if gs else {}
                qz = rq.IntegerQuantizer(4, sym, gran, calib_algo='mse', **kw)
                mn, mx = qz.get_tensor_range(qz.reshape_tensor(w.clone()))
                fq = qz.fake_quant_weight_dynamic(w.clone())
                key = f'{str(dtype)[6:]}_{"sym" if sym else "asym"}_{gran}_{gs}'
                cases[key] = dict(w=w, bit=4, sym=sym, granularity=gran, group_size=gs, min=mn.clone(),
                                  max=mx.clone(), fake=fq)
    torch.save(cases, os.path.join(out_dir, 'rtn_mse.pt'))
    print('rtn_mse.pt', len(cases), 'cases')


def make_act_static(rq, out_dir):
    """Static per-tensor activation quantisation: get_batch_tensors_qparams with calib_algo
    'static_minmax' / 'static_moving_minmax' and fake_quant_act_static with the resulting buffers."""
    gen = torch.Generator().manual_seed(2003)
    cases = {}
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for algo in ('static_minmax', 'static_moving_minmax'):
            for sym in (True, False):
                acts = [(torch.randn(2, 12, 128, generator=gen) * (1 + 0.3 * i) + 0.1 * i).to(dtype) for i in range(6)]
                qz = rq.IntegerQuantizer(8, sym, 'per_tensor', calib_algo=algo)
                sl, zl, qminl, qmaxl = qz.get_batch_tensors_qparams([a.clone() for a in acts])
                assert len(sl) == 1
                x = (torch.randn(2, 9, 128, generator=gen) * 1.5).to(dtype)
                args = {'scales': sl[0], 'zeros': zl[0], 'qmax': qmaxl[0], 'qmin': qminl[0]}
                fq = qz.fake_quant_act_static(x.clone(), args)
                name = f"{str(dtype).split('.')[-1]}_{algo}_{'sym' if sym else 'asym'}"
                cases[name] = dict(acts=acts, dtype=dtype, algo=algo, sym=sym, bit=8, scales=sl[0], zeros=zl[0],
                                   x=x, fake=fq)
    torch.save(cases, os.path.join(out_dir, 'act_static.pt'))
    print('act_static.pt', len(cases), 'cases')


def make_act_hist(rq, out_dir):
    """calib_algo 'static_hist' (symmetric per_tensor int8): get_batch_tensors_qparams over a batch whose
    running range widens twice (so that histograms are re-binned), then fake_quant_act_static."""
    gen = torch.Generator().manual_seed(2008)
    cases = {}
    for dtype in (torch.bfloat16, torch.float32):
        scales = (1.0, 0.6, 1.4, 1.0, 2.2, 0.9)
        acts = [(torch.randn(2, 40, 128, generator=gen) * sc).to(dtype) for sc in scales]
        acts[1][0, 0, 0] = 0.25            # a tensor whose range lies inside the running one
        qz = rq.IntegerQuantizer(8, True, 'per_tensor', calib_algo='static_hist')
        mins, maxs = qz.get_static_hist_range([a.clone() for a in acts])
        sl, zl, qminl, qmaxl = qz.get_batch_tensors_qparams([a.clone() for a in acts])
        x = (torch.randn(2, 9, 128, generator=gen) * 1.5).to(dtype)
        fq = qz.fake_quant_act_static(x.clone(), {'scales': sl[0], 'zeros': zl[0], 'qmax': qmaxl[0], 'qmin': qminl[0]})
        cases[str(dtype).split('.')[-1]] = dict(acts=acts, dtype=dtype, min=mins[0], max=maxs[0], scales=sl[0],
                                                 x=x, fake=fq)
    torch.save(cases, os.path.join(out_dir, 'act_hist.pt'))
    print('act_hist.pt', len(cases), 'cases')


W48_BIT4 = {'symmetric': False, 'granularity': 'per_group', 'group_size': 128, 'scales_bit': 8,
            'scales_symmetric': True, 'zeros_bit': 8, 'zeros_symmetric': True}
W48_BIT8 = {'symmetric': True, 'granularity': 'per_channel', 'int_range': [-120, 120]}


def make_w48(rq, out_dir):
    """Weight48IntegerQuantizer.fake_quant_weight_dynamic with the levels of the reference's own
    rtn_w_a_wint4aint8.yml, plus a symmetric 4-bit level without scale / zero-point limits."""
    gen = torch.Generator().manual_seed(2004)
    cases = {}
    plain4 = {'symmetric': True, 'granularity': 'per_group', 'group_size': 128}
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for name, bit4 in (('yml', W48_BIT4), ('sym4', plain4)):
            for R, C in ((24, 384), (5, 1024)):
                w = (torch.randn(R, C, generator=gen) * 0.05)
                w[0, :128] = 0.0                   # a constant group: the 1e-5 floor of the 4-bit scale
                w[1, 7] = 3.0                      # an outlier that saturates the row's 8-bit range
                w = w.to(dtype)
                qz = rq.Weight48IntegerQuantizer(48, copy.deepcopy(bit4), copy.deepcopy(W48_BIT8))
                fq = qz.fake_quant_weight_dynamic(w.clone())
                cases[f"{str(dtype).split('.')[-1]}_{name}_{R}x{C}"] = dict(w=w, bit4=bit4, bit8=W48_BIT8, fake=fq)
    torch.save(cases, os.path.join(out_dir, 'rtn_w48.pt'))
    print('rtn_w48.pt', len(cases), 'cases')


def make_quik(rq, out_dir):
    """The mixed-precision fake quant QUIK's w_qdq / a_qdq run (IntegerQuantizer with int_indices /
    fp_indices), with the column split quik.py:119-120 derives from the activation statistic."""
    gen = torch.Generator().manual_seed(2005)
    cases = {}
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for sym in (True, False):
            hidden, n_fp = 256, 24
            acts = [torch.randn(2, 20, hidden, generator=gen) for _ in range(3)]
            for a in acts:
                a[:, :, ::11] *= 12
            acts = [a.to(dtype) for a in acts]
            stat = None
            for a in acts:
                m = torch.max(a.view(-1, hidden).abs().detach(), dim=0)[0].float().cpu()      # quik.py:35-42
                stat = m if stat is None else torch.max(stat, m)
            order = torch.sort(stat)[1]
            int_ids, fp_ids = order[:-n_fp].clone(), order[-n_fp:].clone()
            args = {'int_indices': int_ids, 'fp_indices': fp_ids, 'current_bit': torch.tensor(8)}
            w = (torch.randn(40, hidden, generator=gen) * 0.05).to(dtype)
            wq = rq.IntegerQuantizer(4, sym, 'per_channel')
            aq = rq.IntegerQuantizer(8, sym, 'per_token')
            fw = wq.fake_quant_weight_dynamic(w.clone(), dict(args))
            fa = aq.fake_quant_act_dynamic(acts[0].clone(), dict(args))
            name = f"{str(dtype).split('.')[-1]}_{'sym' if sym else 'asym'}"
            cases[name] = dict(acts=acts, stat=stat, int_ids=int_ids, fp_ids=fp_ids, w=w, sym=sym, wbit=4, abit=8,
                               fake_w=fw, fake_a=fa)
    torch.save(cases, os.path.join(out_dir, 'quik_mixed.pt'))
    print('quik_mixed.pt', len(cases), 'cases')


def make_fp8(rq, out_dir):
    rq.float_quantize = lambda x, e, m, rounding: x.to(torch.float8_e4m3fn).float()
    gen = torch.Generator().manual_seed(5001)
    cases = {}
    for dtype in (torch.bfloat16, torch.float32, torch.float16):
        w = (torch.randn(10, 352, generator=gen) * 0.02).to(dtype)
        w[1, :] = 0
        w[2, :] = (torch.randn(352, generator=gen) * 1e-6).to(dtype)
        qz = rq.FloatQuantizer('e4m3', True, 'per_channel', use_qtorch=True)
        fq = qz.fake_quant_weight_dynamic(w.clone())
        codes, scales, _ = qz.real_quant_weight_dynamic(w.clone())
        x = torch.randn(3, 4, 352, generator=gen).to(dtype)
        qa = rq.FloatQuantizer('e4m3', True, 'per_token', use_qtorch=True)
        fa = qa.fake_quant_act_dynamic(x.clone())
        cases[str(dtype)[6:]] = dict(w=w, fake=fq, codes=codes.view(torch.uint8), scales=scales,
                                     x=x, fake_act=fa, pinned=False)
    torch.save(cases, os.path.join(out_dir, 'fp8_e4m3.pt'))
    print('fp8_e4m3.pt', len(cases), 'cases')
    # block-wise weights (one fp32 scale per 128 x 128 block): quant.py's own weight_cast_to_fp8 /
    # weight_cast_to_bf16 (the torch versions the reference uses when its Triton kernels are unavailable)
    blk = {}
    for name, shape, dtype in (('bf16_128x256', (128, 256), torch.bfloat16), ('bf16_140x128', (140, 128), torch.bfloat16),
                               ('bf16_128x132', (128, 132), torch.bfloat16), ('f32_130x128', (130, 128), torch.float32)):
        w = (torch.randn(*shape, generator=gen) * 0.02).to(dtype)
        w[:64, :64] = 0
        w[100:, 100:] *= 30
        codes, scales = rq.weight_cast_to_fp8(w.clone(), 128)
        back = rq.weight_cast_to_bf16(codes, scales, 128)
        qz = rq.FloatQuantizer('e4m3', True, 'per_block', block_size=128, use_qtorch=True)
        fq = qz.fake_quant_weight_dynamic(w.clone())
        blk[name] = dict(w=w, codes=codes.view(torch.uint8), scales=scales, back=back, fake=fq, pinned=False)
    torch.save(blk, os.path.join(out_dir, 'fp8_block.pt'))
    print('fp8_block.pt', len(blk), 'cases')


def _ref_gptq_layer(rq, rg, W, X, bit, sym, actorder, percdamp=0.01, n_out=0, static_groups=False,
                    per_channel=False):
    """Drives the reference GPTQ class on one nn.Linear, bypassing its model plumbing.  n_out > 0: owq."""
    g = object.__new__(rg.GPTQ)
    g.dev = torch.device('cpu')
    g.wquantizer = (rq.IntegerQuantizer(bit, sym, 'per_channel') if per_channel
                    else rq.IntegerQuantizer(bit, sym, 'per_group', group_size=128))
    g.true_sequential, g.static_groups, g.actorder = True, static_groups, actorder
    g.percdamp, g.blocksize, g.owq, g.chunk_num = percdamp, 128, n_out > 0, 1
    g.need_perm = (actorder and not static_groups and not per_channel) or n_out > 0
    if n_out:
        g.n_out_dict = {'l': n_out}
    g.layers_cache = {'l': {}}
    g.model_dtype = W.dtype
    layer = torch.nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype)
    layer.weight.data = W.clone()
    # collect_block_qparams leaves RTN buffers on the layer (base_blockwise_quantization.py:362-376)
    _, s, z, qmax, qmin = g.wquantizer.get_tensor_qparams(layer.weight.data)
    layer.register_buffer('buf_scales', s)
    layer.register_buffer('buf_zeros', z)
    layer.register_buffer('buf_qmax', qmax)
    layer.register_buffer('buf_qmin', qmin)
    g.layer_init(layer, 'l')
    for i in range(X.shape[0]):
        g.add_batch(layer, 'l', X[i:i + 1], None)
    H = g.layers_cache['l']['H'].clone()
    g.layer_transform(layer, 'l')
    fq = g.w_qdq(layer, g.wquantizer)
    perm = layer.buf_perm if g.need_perm else torch.arange(W.shape[1])
    codes = g.wquantizer.quant(layer.weight.data[:, perm].reshape(-1, W.shape[1] if per_channel else 128),
                               layer.buf_scales,
                               layer.buf_zeros if not sym else torch.tensor(0.0),
                               layer.buf_qmax, layer.buf_qmin).reshape(W.shape)
    return dict(W=W, X=X, H=H, bit=bit, sym=sym, actorder=actorder, percdamp=percdamp,
                weight=layer.weight.data.clone(), buf_scales=layer.buf_scales.clone(),
                buf_zeros=None if sym else layer.buf_zeros.clone(),
                buf_perm=perm.clone(), codes_perm=codes.to(torch.int16), w_qdq=fq.clone(), n_out=n_out)


def make_gptq(rq, rg, out_dir):
    gen = torch.Generator().manual_seed(2001)
    cases = {}
    for name, R, C, ns, T, sym, act in (('asym_act', 48, 384, 6, 160, False, True),
                                        ('sym_act', 32, 256, 4, 128, True, True),
                                        ('asym_noact', 32, 256, 4, 128, False, False)):
        W = (torch.randn(R, C, generator=gen) * 0.02).to(torch.bfloat16)
        X = torch.randn(ns, T, C, generator=gen)
        out_ch = torch.randperm(C, generator=gen)[:max(1, C // 100)]
        X[:, :, out_ch] *= 20
        X = X.to(torch.bfloat16)
        cases[name] = _ref_gptq_layer(rq, rg, W, X, 4, sym, act)
    torch.save(cases, os.path.join(out_dir, 'gptq_layer.pt'))
    print('gptq_layer.pt', len(cases), 'cases')


def make_gptq_static(rq, rg, out_dir):
    """GPTQ with static_groups (the setting of the reference's vllm / sglang / autoawq export configs)."""
    gen = torch.Generator().manual_seed(2006)
    cases = {}
    for name, R, C, ns, T, sym, act in (('sym_act', 48, 384, 6, 160, True, True),
                                        ('asym_act', 32, 256, 4, 128, False, True),
                                        ('asym_noact', 32, 256, 4, 128, False, False)):
        W = (torch.randn(R, C, generator=gen) * 0.02).to(torch.bfloat16)
        X = torch.randn(ns, T, C, generator=gen)
        out_ch = torch.randperm(C, generator=gen)[:max(1, C // 100)]
        X[:, :, out_ch] *= 20
        X = X.to(torch.bfloat16)
        cases[name] = _ref_gptq_layer(rq, rg, W, X, 4, sym, act, static_groups=True)
    torch.save(cases, os.path.join(out_dir, 'gptq_static.pt'))
    print('gptq_static.pt', len(cases), 'cases')


def make_gptq_per_channel(rq, rg, out_dir):
    """GPTQ on per_channel 8-bit weights (the reference's w8a8 configs, step_2_gptq.yml)."""
    gen = torch.Generator().manual_seed(2007)
    cases = {}
    for name, R, C, ns, T, bit, sym in (('w8_sym', 48, 384, 6, 160, 8, True), ('w4_asym', 32, 256, 4, 128, 4, False)):
        W = (torch.randn(R, C, generator=gen) * 0.02).to(torch.bfloat16)
        X = torch.randn(ns, T, C, generator=gen)
        out_ch = torch.randperm(C, generator=gen)[:max(1, C // 100)]
        X[:, :, out_ch] *= 20
        X = X.to(torch.bfloat16)
        cases[name] = _ref_gptq_layer(rq, rg, W, X, bit, sym, True, static_groups=True, per_channel=True)
    torch.save(cases, os.path.join(out_dir, 'gptq_per_channel.pt'))
    print('gptq_per_channel.pt', len(cases), 'cases')


def make_gptq_owq(rq, rg, out_dir):
    """GPTQ with owq (gptq.py:44-50, :66-83): the n_out columns with the largest Hessian diagonal stay fp."""
    gen = torch.Generator().manual_seed(2002)
    cases = {}
    for name, R, C, ns, T, sym, n_out in (('asym_out6', 48, 384, 6, 160, False, 6),
                                          ('sym_out2', 32, 256, 4, 128, True, 2)):
        W = (torch.randn(R, C, generator=gen) * 0.02).to(torch.bfloat16)
        X = torch.randn(ns, T, C, generator=gen)
        out_ch = torch.randperm(C, generator=gen)[:max(1, C // 50)]
        X[:, :, out_ch] *= 20
        X = X.to(torch.bfloat16)
        cases[name] = _ref_gptq_layer(rq, rg, W, X, 4, sym, False, n_out=n_out)
    torch.save(cases, os.path.join(out_dir, 'gptq_owq.pt'))
    print('gptq_owq.pt', len(cases), 'cases')


def _ref_spqr_layer(rq, rs, W, X, bit, group, percdamp, rel_threshold, simplified, actorder=True):
    """Drives the reference SpQR class (spqr.py) on one nn.Linear, bypassing its model plumbing."""
    g = object.__new__(rs.SpQR)
    g.dev = torch.device('cpu')
    g.wquantizer = rq.IntegerQuantizer(bit, False, 'per_group', group_size=group, round_zp=False)
    sub = dict(bit=3, symmetric=False, granularity='per_group', group_size=16, round_zp=False)
    g.scale_quantizer = rq.IntegerQuantizer(**sub)
    g.zero_quantizer = rq.IntegerQuantizer(**sub)
    g.Q = rq.IntegerQuantizer(bit, False, 'per_channel', round_zp=False)
    g.true_sequential, g.actorder, g.percdamp, g.blocksize = True, actorder, percdamp, 128
    g.relative_threshold, g.simplified_outliers = rel_threshold, simplified
    if actorder:
        g.need_perm = True
    g.layers_cache = {'l': {}}
    g.model_dtype = W.dtype
    layer = torch.nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype)
    layer.weight.data = W.clone()
    g.layer_init(layer, 'l')
    for i in range(X.shape[0]):
        g.add_batch(layer, 'l', X[i:i + 1], X[i:i + 1])
    H = g.layers_cache['l']['H'].clone()
    g.layer_transform(layer, 'l')
    fq = g.w_qdq(layer, g.wquantizer)
    perm = layer.buf_perm if actorder else torch.arange(W.shape[1])
    return dict(W=W, X=X, H=H, bit=bit, group=group, percdamp=percdamp, rel_threshold=rel_threshold,
                simplified=simplified, actorder=actorder, weight=layer.weight.data.clone(),
                buf_scales=layer.buf_scales.clone(), buf_zeros=layer.buf_zeros.clone(), buf_perm=perm.clone(),
                mask=layer.buf_mask.to_dense().bool(), w_qdq=fq.clone())


def make_spqr(rq, out_dir):
    """SpQR (spqr.py:184-285) with the settings of the reference's spqr_w_only.yml (4 bit, groups of 16,
    3-bit second-level statistics, relative_threshold 0.2, percdamp 1) and its two other outlier modes."""
    import math
    import llmc.compression.quantization.spqr as rs
    gen = torch.Generator().manual_seed(2011)
    cases = {}
    for name, R, C, ns, T, thr, simp, act in (('loo_act', 48, 384, 6, 160, 0.2, False, True),
                                              ('simplified_act', 32, 256, 4, 128, 0.2, True, True),
                                              ('no_outliers_act', 32, 256, 4, 128, math.inf, False, True),
                                              ('loo_noact', 32, 256, 4, 128, 0.1, False, False)):
        W = (torch.randn(R, C, generator=gen) * 0.02)
        W[torch.rand(R, C, generator=gen) < 0.01] *= 8           # weight outliers for the detector to find
        W = W.to(torch.bfloat16)
        X = torch.randn(ns, T, C, generator=gen)
        out_ch = torch.randperm(C, generator=gen)[:max(1, C // 100)]
        X[:, :, out_ch] *= 20
        X = X.to(torch.bfloat16)
        cases[name] = _ref_spqr_layer(rq, rs, W, X, 4, 16, 1.0, thr, simp, act)
        print(name, 'outliers', int(cases[name]['mask'].sum()), 'of', R * C)
    torch.save(cases, os.path.join(out_dir, 'spqr_layer.pt'))
    print('spqr_layer.pt', len(cases), 'cases')


def make_gptq_block(ref_root, out_dir):
    """The reference's own GPTQ through its own driver -- model adapter, first-block catcher,
    ALGO_REGISTRY['GPTQ'](...), run_block_loop() (blockwise_optimization.py:31-42 ->
    base_blockwise_quantization.py:403-549) -- on a random-init two-layer Llama, settings of
    gptq_w_only.yml.  Stored: the blocks' initial state, the first block's inputs, what every linear is
    left with, and the tensors handed to the block after the last one."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(out_dir)))
    from oracle import ref_driver as rd
    ref = rd.import_reference(ref_root, on_cpu=True)
    shape = dict(hidden=128, inter=256, heads=2, layers=2, vocab=64, max_pos=256)
    n, T = 6, 48
    cfg = rd.tiny_llama_config(**shape)
    model = rd.synth_llama_adapter(ref, cfg, seed=21)
    state0 = [{k: v.clone() for k, v in b.state_dict().items()} for b in model.get_blocks()]
    calib = rd.calib_ids(n, T, cfg.vocab_size, seed=22)
    model.collect_first_block_input(calib, None)
    first = model.get_first_block_input()
    x0 = [t.clone() for t in first['data']]
    kw0 = {k: ((tuple(t.clone() for t in v) if isinstance(v, tuple) else v.clone() if torch.is_tensor(v) else v))
           for k, v in first['kwargs'][0].items() if k != 'use_cache'}
    algo = ref.ALGO_REGISTRY['GPTQ'](model, rd.gptq_quant_config(), first, None,
                                     rd.AttrDict(model=dict(type='Llama'), calib=dict(bs=1, seq_len=T, n_samples=n),
                                                 quant=rd.gptq_quant_config()))
    algo.run_block_loop()
    out = dict(shape=shape, T=T, state0=state0, x0=x0, kwargs=kw0, linears=rd.linear_state(model),
               next_inputs=[t.clone() for t in algo.input['data']],
               module_classes=sorted({type(m).__name__ for b in model.get_blocks() for m in b.modules()}))
    torch.save(out, os.path.join(out_dir, 'gptq_block_loop.pt'))
    print('gptq_block_loop.pt', len(out['linears']), 'blocks')


class _TorchProxy:
    """Stands in for the `torch` name inside the reference's awq module: drops device='cuda'."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def tensor(*a, device=None, **k):
        return torch.tensor(*a, **k)

    @staticmethod
    def zeros_like(*a, device=None, **k):
        return torch.zeros_like(*a, **k)


def tiny_llama_block(hidden=256, inter=512, heads=4, T=64, seed=0):
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=1, vocab_size=128, max_position_embeddings=4 * T)
    cfg._attn_implementation = 'sdpa'
    block = LlamaDecoderLayer(cfg, 0).to(torch.bfloat16)
    g = torch.Generator().manual_seed(seed)
    for p in block.parameters():
        p.data = ((torch.randn(p.shape, generator=g) * 0.02) if p.dim() == 2
                  else (1 + 0.1 * torch.randn(p.shape, generator=g))).to(torch.bfloat16)
    rot = LlamaRotaryEmbedding(cfg)
    pos = torch.arange(T)[None]
    cos, sin = rot(torch.zeros(1, T, hidden, dtype=torch.bfloat16), pos)
    return block, {'position_embeddings': (cos, sin), 'attention_mask': None, 'position_ids': pos}


def make_awq(rq, out_dir):
    """Drives the reference Awq class (search_scale_subset / apply_scale / AutoClipper) on one tiny
    Llama block, bypassing its model plumbing."""
    import llmc.compression.quantization.awq as rawq
    import llmc.compression.quantization.auto_clip as rclip
    rawq.torch = _TorchProxy()
    torch.nn.Module.cuda = lambda self, *a, **k: self
    # The reference recognises norm layers through transformers' ALL_LAYERNORM_LAYERS
    # (module_utils.py:9, :1180).  The transformers releases it is written for (>= 4.45,
    # requirements/runtime.txt) register LlamaRMSNorm there; the 5.x release installed here no
    # longer does, which would make the reference skip the two norm-fed subsets.  Restore the entry.
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    from transformers.pytorch_utils import ALL_LAYERNORM_LAYERS
    if LlamaRMSNorm not in ALL_LAYERNORM_LAYERS:
        ALL_LAYERNORM_LAYERS.append(LlamaRMSNorm)
    cases = {}
    for name, sym, clip_sym in (('asym', False, False), ('sym_clipsym', True, True)):
        block, kwargs = tiny_llama_block(seed=11)
        g = torch.Generator().manual_seed(3001)
        x = torch.randn(4, 64, 256, generator=g)
        x[:, :, torch.randperm(256, generator=g)[:3]] *= 20
        x = x.to(torch.bfloat16)
        state0 = {k: v.clone() for k, v in block.state_dict().items()}

        a = object.__new__(rawq.Awq)
        a.wquantizer = rq.IntegerQuantizer(4, sym, 'per_group', group_size=128)
        a.aquantizer, a.w_only, a.padding_mask = None, True, None
        a.trans, a.trans_version, a.save_scale, a.awq_bs, a.save_mem = True, 'v2', False, None, True
        a.weight_clip, a.clip_version, a.act_static, a.true_sequential = True, 'v1', False, False
        a.has_gqa, a.do_gqa_trans, a.block_idx, a.n_samples = False, False, 0, 4

        class Cfg(dict):
            __getattr__ = dict.__getitem__
        a.config = Cfg(model=Cfg(type='Llama'), calib=Cfg(seq_len=64))

        class Model:
            # llmc/models/__init__.py imports every adapter (and packages that are not installed),
            # so the four Llama subsets (llmc/models/llama.py:52-91) are written out here
            block_name_prefix = 'model.layers'

            @staticmethod
            def get_subsets_in_block(b):
                sa, mlp = b.self_attn, b.mlp
                return [
                    {'layers': {'self_attn.q_proj': sa.q_proj, 'self_attn.k_proj': sa.k_proj,
                                'self_attn.v_proj': sa.v_proj},
                     'prev_op': [b.input_layernorm], 'input': ['self_attn.q_proj'], 'inspect': sa, 'has_kwargs': True},
                    {'layers': {'self_attn.o_proj': sa.o_proj}, 'prev_op': [sa.v_proj],
                     'input': ['self_attn.o_proj'], 'inspect': sa.o_proj, 'has_kwargs': False},
                    {'layers': {'mlp.gate_proj': mlp.gate_proj, 'mlp.up_proj': mlp.up_proj},
                     'prev_op': [b.post_attention_layernorm], 'input': ['mlp.gate_proj'], 'inspect': mlp,
                     'has_kwargs': False, 'is_mlp': True},
                    {'layers': {'mlp.down_proj': mlp.down_proj}, 'prev_op': [mlp.up_proj],
                     'input': ['mlp.down_proj'], 'inspect': mlp.down_proj, 'has_kwargs': False, 'is_mlp': True},
                ]
        a.model = Model()
        a.auto_clipper = rclip.AutoClipper(w_only=True, wquantizer=a.wquantizer, aquantizer=None, clip_version='v1',
                                           clip_sym=clip_sym, save_clip=False, padding_mask=None)
        # cache the linears' inputs the way BlockwiseOpt.cache_input_hook does
        feats, hooks = {}, []
        for n, m in block.named_modules():
            if isinstance(m, torch.nn.Linear):
                def hook(mod, inp, out, n=n):
                    feats.setdefault(n, []).append(inp[0].data.clone())
                hooks.append(m.register_forward_hook(hook))
        with torch.no_grad():
            block(x, **kwargs)
        for h in hooks:
            h.remove()
        a.block_transform(block, feats, [dict(kwargs, past_key_values=None, use_cache=False)])
        cases[name] = dict(x=x, sym=sym, clip_sym=clip_sym, state0=state0,
                           state1={k: v.clone() for k, v in block.state_dict().items()})
    torch.save(cases, os.path.join(out_dir, 'awq_block.pt'))
    print('awq_block.pt', len(cases), 'cases')


def make_export_configs(ref_root, out_dir):
    """config.json entries written by the reference's export helpers (llmc/utils/export_vllm.py,
    export_autoawq.py), loaded by file path (they only need json)."""
    import importlib.util
    import json
    import tempfile

    def load(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, 'llmc', 'utils', name + '.py'))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    ev, ea = load('export_vllm'), load('export_autoawq')

    class AD(dict):
        __getattr__ = dict.__getitem__

        def __init__(self, d):
            super().__init__({k: (AD(v) if isinstance(v, dict) else v) for k, v in d.items()})

    class Model:
        def skip_layer_name(self):
            return ['lm_head']
    w8 = dict(bit=8, symmetric=True, granularity='per_channel')
    fp8 = dict(quant_type='float-quant', bit='e4m3', symmetric=True)
    cases = {
        'w4a16_g128_pack': dict(weight=dict(bit=4, symmetric=True, granularity='per_group', group_size=128,
                                            need_pack=True)),
        'w8a8_int': dict(weight=w8, act=dict(bit=8, symmetric=True, granularity='per_token')),
        'w4a16_channel': dict(weight=dict(bit=4, symmetric=False, granularity='per_channel')),
        'fp8_block': dict(weight=dict(fp8, granularity='per_block', block_size=128),
                          act=dict(fp8, granularity='per_group', group_size=128)),
        'fp8_static': dict(weight=dict(fp8, granularity='per_tensor'),
                           act=dict(fp8, granularity='per_tensor', static=True)),
        'w8a8_static': dict(weight=w8, act=dict(bit=8, symmetric=True, granularity='per_tensor', static=True)),
    }
    out = {}

    def fresh_dir():
        d = tempfile.mkdtemp()
        with open(os.path.join(d, 'config.json'), 'w') as f:
            json.dump({'model_type': 'llama', 'quantization_config': {'old': 1}}, f)
        return d
    for k, c in cases.items():
        d = fresh_dir()
        ev.update_vllm_quant_config(Model(), AD({'quant': c}), d)
        with open(os.path.join(d, 'config.json')) as f:
            out['vllm_' + k] = {'in': c, 'config_json': json.load(f)}
    c = dict(weight=dict(bit=4, symmetric=False, granularity='per_group', group_size=128, pack_version='gemm_pack'))
    d = fresh_dir()
    ea.update_autoawq_quant_config(AD({'quant': c}), d)
    with open(os.path.join(d, 'config.json')) as f:
        out['autoawq'] = {'in': c, 'config_json': json.load(f)}
    with open(os.path.join(out_dir, 'export_configs.json'), 'w') as f:
        json.dump(out, f, indent=1)
    print('export_configs.json', len(out), 'cases')


if __name__ == '__main__':
    ref_root = sys.argv[1]
    out_dir = os.path.dirname(os.path.abspath(__file__))
    rq, rg = _import_reference(ref_root)
    torch.set_num_threads(1)
    only = set(sys.argv[2:])            # optional: names of the fixtures to (re)make; default all
    steps = {'rtn': lambda: make_rtn(rq, out_dir), 'rtn_mse': lambda: make_rtn_mse(rq, out_dir),
             'gptq': lambda: make_gptq(rq, rg, out_dir), 'gptq_owq': lambda: make_gptq_owq(rq, rg, out_dir),
             'gptq_per_channel': lambda: make_gptq_per_channel(rq, rg, out_dir),
             'gptq_static': lambda: make_gptq_static(rq, rg, out_dir),
             'quik': lambda: make_quik(rq, out_dir), 'w48': lambda: make_w48(rq, out_dir), 'act_static': lambda: make_act_static(rq, out_dir), 'act_hist': lambda: make_act_hist(rq, out_dir), 'fp8': lambda: make_fp8(rq, out_dir), 'awq': lambda: make_awq(rq, out_dir),
             'export': lambda: make_export_configs(ref_root, out_dir),
             'gptq_block': lambda: make_gptq_block(ref_root, out_dir), 'spqr': lambda: make_spqr(rq, out_dir)}
    for name, step in steps.items():
        if not only or name in only:
            step()
