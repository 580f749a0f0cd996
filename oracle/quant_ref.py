"""Oracle restatement of the reference quantizer arithmetic (test infrastructure).

Follows llmc/compression/quantization/quant.py:
  reshape_tensor :611-641, get_minmax_range :134-145, get_mse_range :147-205, get_qparams :544-558,
  IntegerQuantizer.quant/dequant/quant_dequant :698-716,
  fake_quant_weight_dynamic :832-868, real_quant_weight_dynamic :915-952,
  fake_quant_act_dynamic :753-782, FloatQuantizer :963-1002, :1042-1080.

Everything is evaluated with torch CPU ops *in the dtype of the input tensor*,
because that is what the reference does: for a bf16 weight every intermediate
(min, max, scale, zero, w/s ...) is rounded to bf16 after each op.
"""
import torch


def int_range(bit, sym):
    """qmin/qmax as 0-dim tensors with the reference's dtypes (quant.py:664-676)."""
    if sym:
        return torch.tensor(-(2 ** (bit - 1))), torch.tensor(2 ** (bit - 1) - 1)
    return torch.tensor(0.0), torch.tensor(2 ** bit - 1)


def group_view(t, granularity, group_size=None):
    """quant.py:611-641 without padding: per_group -> (-1, g); otherwise identity."""
    if granularity == 'per_group':
        if t.shape[-1] >= group_size:
            if t.shape[-1] % group_size:
                raise ValueError(
                    f'Dimension {t.shape[-1]} not divisible by group size {group_size}')
            return t.reshape(-1, group_size)
        return t
    if granularity in ('per_channel', 'per_token', 'per_tensor'):
        return t
    raise NotImplementedError(granularity)


def int_qparams(g, bit, sym):
    """min/max -> (scales, zeros, qmax, qmin); quant.py:134-145 and :544-558."""
    qmin, qmax = int_range(bit, sym)
    qmin, qmax = qmin.to(g.device), qmax.to(g.device)      # quant.py:546-547
    mx = g.amax(dim=-1, keepdim=True)
    mn = g.amin(dim=-1, keepdim=True)
    if sym:
        a = torch.max(mx.abs(), mn.abs()).clamp(min=1e-5)
        return a / qmax, torch.tensor(0.0), qmax, qmin
    s = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
    z = (qmin - torch.round(mn / s)).clamp(qmin, qmax)
    return s, z, qmax, qmin


def int_quant(g, s, z, qmax, qmin):
    """quant.py:698-700 (round_zp=True, torch.round = half to even)."""
    return torch.clamp(torch.round(g / s) + z, qmin.to(g.device), qmax.to(g.device))


def int_dequant(q, s, z):
    """quant.py:709-711."""
    return (q - z) * s


def int_fake_quant_dynamic(w, bit, sym, granularity, group_size=None):
    """fake_quant_weight_dynamic / fake_quant_act_dynamic (quant.py:832-868, :753-782)."""
    g = group_view(w, granularity, group_size)
    s, z, qmax, qmin = int_qparams(g, bit, sym)
    out = int_dequant(int_quant(g, s, z, qmax, qmin), s, z)
    return out.reshape(w.shape).to(w.dtype)


def int_fake_quant_static(w, s, z, bit, sym, granularity, group_size=None):
    """fake_quant_weight_static (quant.py:784-830) without the optional args."""
    qmin, qmax = int_range(bit, sym)
    g = group_view(w, granularity, group_size)
    out = int_dequant(int_quant(g, s, z, qmax, qmin), s, z)
    return out.reshape(w.shape).to(w.dtype)


def int_qparams_from_range(mn, mx, bit, sym):
    """get_qparams on a given (min, max) (quant.py:544-558, round_zp=True)."""
    qmin, qmax = int_range(bit, sym)
    qmin, qmax = qmin.to(mn.device), qmax.to(mn.device)
    if sym:
        a = torch.max(mx.abs(), mn.abs()).clamp(min=1e-5)
        return a / qmax, torch.tensor(0.0), qmax, qmin
    s = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
    z = (qmin - torch.round(mn / s)).clamp(qmin, qmax)
    return s, z, qmax, qmin


def int_fake_quant_mixed(t, bit, sym, granularity, int_indices, fp_indices):
    """fake_quant_weight_dynamic / fake_quant_act_dynamic with int_indices / fp_indices (quant.py:753-782,
    :832-868): the last dim's integer columns are gathered and quantised, then both parts are scattered
    into a zeroed tensor."""
    q = t[..., int_indices]
    fp = t[..., fp_indices]
    q = int_fake_quant_dynamic(q, bit, sym, granularity)
    out = torch.zeros_like(t)
    out[..., int_indices] = q
    out[..., fp_indices] = fp
    return out


def quik_col_absmax(running, tensor):
    """QUIK get_tensor_scale (quik.py:35-42): running per-channel max |x| in fp32 on the host."""
    hidden = tensor.shape[-1]
    m = torch.max(tensor.view(-1, hidden).abs().detach(), dim=0)[0].float().cpu()
    return m if running is None else torch.max(running, m)


def quik_select(layer_scales, outlier_num):
    """QUIK.block_opt (quik.py:119-120): the outlier_num channels with the largest statistic stay fp."""
    order = torch.sort(layer_scales)[1]
    return order[:-outlier_num], order[-outlier_num:]


def w48_level(cfg, bit):
    """Weight48IntegerQuantizer.__init__ (quant.py:1232-1287) for one of its two levels: code range
    and the clamps of scale and zero point.  (The reference derives the zero-point clamp from
    scales_bit, quant.py:1272-1281; restated as is.)"""
    c = dict(cfg)
    if 'int_range' in c:
        qmin, qmax = c['int_range']
    elif c['symmetric']:
        qmin, qmax = -(2 ** (bit - 1)), 2 ** (bit - 1) - 1
    else:
        qmin, qmax = 0, 2 ** bit - 1
    out = {'symmetric': c['symmetric'], 'qmin': torch.tensor(qmin), 'qmax': torch.tensor(qmax),
           'granularity': c.get('granularity'), 'group_size': c.get('group_size')}
    if 'scales_bit' in c:
        if c['scales_symmetric']:
            out['scales_qmin'], out['scales_qmax'] = -(2 ** (c['scales_bit'] - 1)), 2 ** (c['scales_bit'] - 1) - 1
        else:
            out['scales_qmin'], out['scales_qmax'] = 0, 2 ** c['scales_bit'] - 1
    else:
        out['scales_qmin'], out['scales_qmax'] = -torch.inf, torch.inf
    if 'zeros_bit' in c:
        if c['zeros_symmetric']:
            out['zeros_qmin'], out['zeros_qmax'] = -(2 ** (c['scales_bit'] - 1)), 2 ** (c['scales_bit'] - 1) - 1
        else:
            out['zeros_qmin'], out['zeros_qmax'] = 0, 2 ** c['scales_bit'] - 1
    else:
        out['zeros_qmin'], out['zeros_qmax'] = out['qmin'], out['qmax']
    return out


def _w48_qparams(t, lv):
    """get_minmax_range over the last dim + Weight48IntegerQuantizer.get_qparams (quant.py:1304-1323)."""
    mx = t.amax(dim=-1, keepdim=True)
    mn = t.amin(dim=-1, keepdim=True)
    qmin, qmax = lv['qmin'].to(t.device), lv['qmax'].to(t.device)
    if lv['symmetric']:
        scales = torch.max(mx.abs(), mn.abs()).clamp(min=1e-5) / qmax
        zeros = torch.tensor(0.0)
    else:
        scales = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
        zeros = qmin - torch.round(mn / scales)
    scales = scales.clamp(lv['scales_qmin'], lv['scales_qmax'])
    zeros = zeros.clamp(lv['zeros_qmin'], lv['zeros_qmax'])
    return scales, zeros, qmax, qmin


def w48_fake_quant(w, bit4, bit8):
    """Weight48IntegerQuantizer.fake_quant_weight_dynamic (quant.py:1338-1367): 16 -> 8 bits per the
    bit8 level, 8 -> 4 bits per the bit4 level on the codes, and back."""
    l8, l4 = w48_level(bit8, 8), w48_level(bit4, 4)

    def view(t, lv):
        if lv['granularity'] == 'per_group':
            if t.shape[-1] % lv['group_size']:
                raise ValueError(f"Dimension {t.shape[-1]} not divisible by group size {lv['group_size']}")
            return t.reshape(-1, lv['group_size'])
        return t
    t8 = view(w, l8)
    s8, z8, qmax8, qmin8 = _w48_qparams(t8, l8)
    c8 = torch.clamp(torch.round(t8 / s8) + z8, qmin8, qmax8)
    shape8, dtype8 = c8.shape, c8.dtype
    t4 = view(c8, l4)
    s4, z4, qmax4, qmin4 = _w48_qparams(t4, l4)
    c4 = torch.clamp(torch.round(t4 / s4) + z4, qmin4, qmax4)
    d8 = ((c4 - z4) * s4).reshape(shape8).to(dtype8)
    return ((d8 - z8) * s8).reshape(w.shape).to(w.dtype)


def reshape_batch_tensors(act_tensors):
    """quant.py:105-122: a list of tensors is one input; a single tensor is split along its batch
    dim; tuples (several inputs per call) are stacked per input."""
    assert len(act_tensors) > 0
    if isinstance(act_tensors[0], tuple):
        return [torch.stack(list(ts)) for ts in zip(*act_tensors)]
    if len(act_tensors) == 1:
        return [[act_tensors[0][i] for i in range(act_tensors[0].size(0))]]
    return [act_tensors]


def static_minmax_range(act_tensors):
    """get_static_minmax_range with per_tensor granularity (quant.py:134-137, :223-262): per input,
    the mean over the calibration tensors of each tensor's min and max, taken in fp32 on the host."""
    mins, maxs = [], []
    for tensors in reshape_batch_tensors(act_tensors):
        mn = torch.stack([torch.min(t).detach().cpu().to(torch.float32) for t in tensors])
        mx = torch.stack([torch.max(t).detach().cpu().to(torch.float32) for t in tensors])
        mins.append(mn.mean(dim=0))
        maxs.append(mx.mean(dim=0))
    return mins, maxs


def static_moving_minmax_range(act_tensors, alpha=0.01):
    """get_static_moving_minmax_range with per_tensor granularity (quant.py:523-542): an
    exponential moving average over the calibration tensors, in the tensors' dtype."""
    mins, maxs = [], []
    for tensors in reshape_batch_tensors(act_tensors):
        m_min = m_max = None
        for t in tensors:
            mn, mx = torch.min(t), torch.max(t)
            if m_min is None:
                m_min, m_max = mn, mx
            else:
                m_min = m_min + alpha * (mn - m_min)
                m_max = m_max + alpha * (mx - m_max)
        mins.append(m_min)
        maxs.append(m_max)
    return mins, maxs


def _hist_quantization_error(histogram, min_val, max_val, next_start_bin, next_end_bin, bins, dst_nbins):
    """get_quantization_error with get_norm (quant.py:264-330)."""
    bin_width = (max_val.item() - min_val.item()) / bins
    dst_bin_width = bin_width * (next_end_bin - next_start_bin + 1) / dst_nbins
    if dst_bin_width == 0.0:
        return 0.0

    def get_norm(delta_begin, delta_end, density):
        norm = (delta_end * delta_end * delta_end - delta_begin * delta_begin * delta_begin) / 3
        return density * norm
    src_bin = torch.arange(bins, device=histogram.device)
    src_bin_begin = (src_bin - next_start_bin) * bin_width
    src_bin_end = src_bin_begin + bin_width
    dst_bin_of_begin = torch.clamp(torch.div(src_bin_begin, dst_bin_width, rounding_mode='floor'), 0, dst_nbins - 1)
    dst_bin_of_begin_center = (dst_bin_of_begin + 0.5) * dst_bin_width
    dst_bin_of_end = torch.clamp(torch.div(src_bin_end, dst_bin_width, rounding_mode='floor'), 0, dst_nbins - 1)
    density = histogram / bin_width
    norm = torch.zeros(bins, device=histogram.device)
    delta_begin = src_bin_begin - dst_bin_of_begin_center
    delta_end = dst_bin_width / 2
    norm += get_norm(delta_begin, torch.ones(bins, device=histogram.device) * delta_end, density)
    norm += (dst_bin_of_end - dst_bin_of_begin - 1) * get_norm(
        torch.tensor(-dst_bin_width / 2), torch.tensor(dst_bin_width / 2), density)
    dst_bin_of_end_center = dst_bin_of_end * dst_bin_width + dst_bin_width / 2
    delta_begin = -dst_bin_width / 2
    delta_end = src_bin_end - dst_bin_of_end_center
    norm += get_norm(torch.tensor(delta_begin), delta_end, density)
    return norm.sum().item()


def _hist_threshold(histogram, min_val, max_val, bins, dst_nbins):
    """get_hist_threshold (quant.py:402-459)."""
    bin_width = (max_val - min_val) / bins
    total = torch.sum(histogram).item()
    cSum = torch.cumsum(histogram, dim=0)
    stepsize, alpha, beta = 1e-8, 0.0, 1.0
    start_bin, end_bin, norm_min = 0, bins - 1, float('inf')
    while alpha < beta:
        next_alpha, next_beta = alpha + stepsize, beta - stepsize
        left, right = start_bin, end_bin
        while left < end_bin and cSum[left] < next_alpha * total:
            left = left + 1
        while right > start_bin and cSum[right] > next_beta * total:
            right = right - 1
        next_start_bin, next_end_bin = start_bin, end_bin
        if (left - start_bin) > (end_bin - right):
            next_start_bin = left
            alpha = next_alpha
        else:
            next_end_bin = right
            beta = next_beta
        if next_start_bin == start_bin and next_end_bin == end_bin:
            continue
        norm = _hist_quantization_error(histogram, min_val, max_val, next_start_bin, next_end_bin, bins, dst_nbins)
        if norm > norm_min:
            break
        norm_min, start_bin, end_bin = norm, next_start_bin, next_end_bin
    return min_val + bin_width * start_bin, min_val + bin_width * (end_bin + 1)


def _hist_combine(orig_hist, orig_min, orig_max, update_hist, update_min, update_max, bins, upsample_rate=16):
    """_combine_histograms with _upscale_histogram (quant.py:332-400)."""
    if update_min == orig_min and update_max == orig_max:
        return orig_hist + update_hist
    if orig_min == orig_max:
        bin_value = torch.sum(update_hist)
        return torch.histc(orig_min, bins=bins, min=update_min, max=update_max) * bin_value + update_hist
    assert update_min <= orig_min and update_max >= orig_max
    histogram = orig_hist.repeat_interleave(upsample_rate) / upsample_rate
    bin_size = (orig_max - orig_min) / (bins * upsample_rate)
    mid_points = (torch.linspace(orig_min, orig_max, bins * upsample_rate + 1, device=orig_min.device)[:-1]
                  .to(histogram.device) + 0.5 * bin_size)
    boundaries = torch.linspace(update_min, update_max, bins + 1, device=update_min.device).to(histogram.device)
    bucket = torch.bucketize(mid_points, boundaries, right=True) - 1
    bucket[bucket >= bins] = bins - 1
    bucket[bucket < 0] = 0
    return update_hist + torch.bincount(bucket, weights=histogram, minlength=bins)


def static_hist_range(act_tensors, bit, bins=2048):
    """get_static_hist_range (quant.py:461-521), per_tensor: per input, a running 2048-bin histogram over the
    calibration tensors (torch.histc on each tensor's fp32 copy, on the tensor's device; the running
    histogram itself lives on the CPU), then the threshold search."""
    dst_nbins = 2 ** bit
    mins_out, maxs_out = [], []
    for tensors in reshape_batch_tensors(act_tensors):
        t_min = [t.min().detach().cpu().to(torch.float32) for t in tensors]       # get_minmax_stats
        t_max = [t.max().detach().cpu().to(torch.float32) for t in tensors]
        min_val = max_val = None
        histogram = torch.zeros(bins)
        for idx, tensor in enumerate(tensors):
            tensor = tensor.float()
            x_min, x_max = t_min[idx], t_max[idx]
            if min_val is None:
                histogram = torch.histc(tensor, bins, min=x_min.item(), max=x_max.item()).cpu()
                min_val, max_val = x_min, x_max
            else:
                new_min, new_max = torch.min(min_val, x_min), torch.max(max_val, x_max)
                update = torch.histc(tensor, bins, min=new_min.item(), max=new_max.item()).cpu()
                if new_min == min_val and new_max == max_val:
                    histogram = histogram + update
                else:
                    histogram = _hist_combine(histogram, min_val, max_val, update, new_min, new_max, bins)
                min_val, max_val = new_min, new_max
        new_min, new_max = _hist_threshold(histogram, min_val, max_val, bins, dst_nbins)
        mins_out.append(new_min)
        maxs_out.append(new_max)
    return mins_out, maxs_out


def batch_tensors_qparams(act_tensors, bit, sym, calib_algo, alpha=0.01):
    """get_batch_tensors_qparams (quant.py:560-585)."""
    if calib_algo == 'static_hist':
        mins, maxs = static_hist_range(act_tensors, bit)
    elif calib_algo == 'static_minmax':
        mins, maxs = static_minmax_range(act_tensors)
    elif calib_algo == 'static_moving_minmax':
        mins, maxs = static_moving_minmax_range(act_tensors, alpha)
    else:
        raise ValueError(f'Unsupported calibration algorithm: {calib_algo}')
    return [int_qparams_from_range(mn, mx, bit, sym) for mn, mx in zip(mins, maxs)]


def mse_range(g, bit, sym, maxshrink=0.8, mse_grid=100, norm=2.4):
    """get_mse_range (quant.py:147-205) on a grouped tensor (G, group); returns fp32 (min, max), (G, 1).
    The reference keeps its best range in the very tensors it shrinks from (views of min_val /
    max_val written in place), so step i shrinks the best range found so far; stated here with
    explicit copies."""
    t = g.float()
    cur_min = t.amin(dim=-1, keepdim=True)
    cur_max = t.amax(dim=-1, keepdim=True)
    best = torch.full([t.shape[0]], float('inf'), device=t.device)
    for i in range(int(maxshrink * mse_grid)):
        p = 1 - i / mse_grid
        xmin, xmax = p * cur_min, p * cur_max
        s, z, qmax, qmin = int_qparams_from_range(xmin, xmax, bit, sym)
        q = int_dequant(int_quant(t, s, z, qmax, qmin), s, z)
        q -= t
        q.abs_()
        q.pow_(norm)
        err = torch.sum(q, 1)
        better = err < best
        if torch.any(better):
            best[better] = err[better]
            cur_min, cur_max = cur_min.clone(), cur_max.clone()
            cur_min[better] = xmin[better]
            cur_max[better] = xmax[better]
    return cur_min, cur_max


def int_fake_quant_mse(w, bit, sym, granularity, group_size=None, **kw):
    """fake_quant_weight_dynamic with calib_algo 'mse' (quant.py:689-696, :832-868): fp32 range and
    qparams, the quant / dequant ops promote the tensor to fp32, the result returns to w's dtype."""
    g = group_view(w, granularity, group_size)
    mn, mx = mse_range(g, bit, sym, **kw)
    s, z, qmax, qmin = int_qparams_from_range(mn, mx, bit, sym)
    out = int_dequant(int_quant(g, s, z, qmax, qmin), s, z)
    return out.reshape(w.shape).to(w.dtype)


def int_real_quant_dynamic(w, bit, sym, granularity, group_size=None):
    """real_quant_weight_dynamic (quant.py:915-952): codes, scales (R,-1), zeros (R,-1)|None."""
    g = group_view(w, granularity, group_size)
    s, z, qmax, qmin = int_qparams(g, bit, sym)
    q = int_quant(g, s, z, qmax, qmin).reshape(w.shape)
    if bit == 8:
        dt = torch.int8 if sym else torch.uint8
    else:
        dt = torch.int32
    q = q.to(dt)
    zeros = None if sym else z.to(dt).view(w.shape[0], -1)
    return q, s.view(w.shape[0], -1), zeros


def e4m3_round(x_f32):
    """Stand-in for qtorch.quant.float_quantize(x, 4, 3, 'nearest') (quant.py:1065).

    PARITY UNPINNED: qtorch is not vendored with the reference.  Restated as a
    round-to-nearest-even cast onto the float8_e4m3fn grid, subnormals included,
    which is the conversion the reference itself applies next in
    real_quant_weight_* (quant.py:1182, :1210).
    """
    return x_f32.to(torch.float8_e4m3fn).float()


def fp8_qparams(g):
    """FloatQuantizer.get_tensor_qparams with use_qtorch (quant.py:1042-1058, :544-551)."""
    mx = g.amax(dim=-1, keepdim=True)
    mn = g.amin(dim=-1, keepdim=True)
    a = torch.max(mx.abs(), mn.abs()).clamp(min=1e-5)
    s = a / torch.tensor(448.0)
    s[s == 0] = 1           # quant.py:1061
    return s


def fp8_fake_quant_dynamic(w):
    """FloatQuantizer.fake_quant_{weight,act}_dynamic, e4m3, per_channel/per_token
    (quant.py:1099-1108, :1141-1158, :1060-1080).  q stays fp32 (the cast at :1068 is
    discarded), so the dequant product is fp32 and rounded once to the input dtype."""
    s = fp8_qparams(w)
    u = w / s + torch.tensor(0.0)
    q = e4m3_round(u.float())
    return ((q - torch.tensor(0.0)) * s).reshape(w.shape).to(w.dtype)


def fp8_real_quant_dynamic(w):
    """FloatQuantizer.real_quant_weight_dynamic (quant.py:1194-1220): e4m3 codes, scales (R,-1)."""
    s = fp8_qparams(w)
    u = w / s + torch.tensor(0.0)
    q = e4m3_round(u.float())
    return q.to(torch.float8_e4m3fn), s.view(w.shape[0], -1)


def fp8_block_view(w, block=128):
    """reshape_tensor, per_block (quant.py:637-641): zero-pad to whole blocks, view (mb, block, nb, block)."""
    m, n = w.shape
    mp, np_ = -(-m // block) * block, -(-n // block) * block
    t = torch.zeros((mp, np_), dtype=w.dtype, device=w.device)
    t[:m, :n] = w
    return t.view(-1, block, np_ // block, block)


def fp8_block_scales(t):
    """per_block range (quant.py:138-140) and symmetric qparams (:544-551): fp32, shape (mb, 1, nb, 1)."""
    mn = t.abs().float().amin(dim=(1, 3), keepdim=True)
    mx = t.abs().float().amax(dim=(1, 3), keepdim=True)
    s = torch.max(mx.abs(), mn.abs()).clamp(min=1e-5) / torch.tensor(448.0)
    s[s == 0] = 1
    return s


def fp8_block_fake_quant(w, block=128):
    """FloatQuantizer('e4m3', True, 'per_block').fake_quant_weight_dynamic (quant.py:1141-1158, :1060-1075)."""
    t = fp8_block_view(w, block)
    s = fp8_block_scales(t)
    q = e4m3_round((t / s + torch.tensor(0.0)).float())
    out = (q - torch.tensor(0.0)) * s
    return out.reshape(-1, out.shape[2] * block)[:w.shape[0], :w.shape[1]].to(w.dtype)


def fp8_block_real_quant(w, block=128):
    """weight_cast_to_fp8 (quant.py:36-45 -> real_quant_weight_dynamic :1194-1220): codes, scales (mb, nb)."""
    t = fp8_block_view(w, block)
    s = fp8_block_scales(t)
    q = e4m3_round((t / s + torch.tensor(0.0)).float())
    q = q.reshape(-1, q.shape[2] * block)[:w.shape[0], :w.shape[1]]
    return q.to(torch.float8_e4m3fn), s.view(s.shape[0], s.shape[2])


def fp8_block_dequant(codes, scales, block=128):
    """weight_cast_to_bf16 (quant.py:20-33): float(codes) * block scale, to bf16."""
    t = fp8_block_view(codes.float(), block)
    out = (t - 0) * scales.view(scales.shape[0], 1, scales.shape[1], 1)
    return out.reshape(-1, out.shape[2] * block)[:codes.shape[0], :codes.shape[1]].to(torch.bfloat16)


def fp8_act_quant(x, block=128):
    """act_quant (kernel.py:7-53): per group of `block` values s = max|x| / 448 in fp32 (no floor),
    y = e4m3(x / s).  Returns (y, s) with s of shape (*x.shape[:-1], x.shape[-1] // block).
    The Triton kernel's division by the constant is a multiplication by its fp32 reciprocal (checked against
    the kernel's own output on a B200: every scale equal, against 41 % for the exactly rounded quotient).
    Its x / s is an approximate division: within an ulp of the midpoint of two e4m3 values its code can
    differ from the one computed here (one element in 2e5 in the GPU test against the kernel itself)."""
    g = x.float().reshape(-1, block)
    s = g.abs().amax(dim=-1, keepdim=True) * torch.tensor(1.0 / 448.0, dtype=torch.float32)
    y = (g / s).to(torch.float8_e4m3fn)
    return y.reshape(x.shape), s.reshape(*x.shape[:-1], x.shape[-1] // block)


def fp8_block_gemm(a, a_s, b, b_s, block=128):
    """fp8_gemm (kernel.py:153-242): per k block the exact product of the e4m3 values, times the row scale
    of a and the block scale of b, accumulated in fp32."""
    K = a.shape[-1]
    a2, as2 = a.float().reshape(-1, K), a_s.reshape(-1, K // block)
    bf = b.float()
    acc = torch.zeros((a2.shape[0], b.shape[0]), dtype=torch.float32, device=a.device)
    col_blk = torch.arange(b.shape[0], device=a.device) // block
    for kb in range(K // block):
        part = a2[:, kb * block:(kb + 1) * block] @ bf[:, kb * block:(kb + 1) * block].t()
        acc += part * (as2[:, kb:kb + 1] * b_s[col_blk, kb][None, :])
    return acc.reshape(*a.shape[:-1], b.shape[0])


def pack_int4_rows(codes_u8):
    """Two 4-bit codes per byte along the input dim, low nibble first (the nibble order of
    the compressed-tensors packer used by the reference's export path,
    module_utils.py:931-955, which packs 8 nibbles per int32 little-nibble first)."""
    c = codes_u8.to(torch.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def pack_compressed_tensors(codes_signed, num_bits=4):
    """VllmRealQuantLinear.pack (module_utils.py:931-955): (q + 2^(b-1)) packed 32/b per int32 along
    the input dim, first element in the lowest bits."""
    import numpy as np
    offset = 2 ** num_bits // 2
    w = (codes_signed + offset).to(torch.uint8).cpu().numpy().astype(np.uint32)
    pf = 32 // num_bits
    packed = np.zeros((w.shape[0], -(-w.shape[1] // pf)), dtype=np.uint32)
    w = np.pad(w, [(0, 0), (0, packed.shape[1] * pf - w.shape[1])])
    for i in range(pf):
        packed |= w[:, i::pf] << (num_bits * i)
    return torch.from_numpy(packed.view(np.int32))


def pack_autoawq(int_t, bit=4):
    """The packing loops of AutoawqRealQuantLinear.gemm_pack (module_utils.py:1130-1158):
    int_t is (in, out) int32 (already transposed); returns (in, out/8) int32."""
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    pack_num = 32 // bit
    q = torch.zeros((int_t.shape[0], int_t.shape[1] // 32 * bit), dtype=torch.int32)
    for col in range(int_t.shape[1] // pack_num):
        for i in range(pack_num):
            q[:, col] |= int_t[:, col * pack_num + order[i]] << (i * bit)
    return q
