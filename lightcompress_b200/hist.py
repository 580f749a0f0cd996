"""Host side of calib_algo 'static_hist': combining the per-tensor histograms of a calibration batch
and searching the clipping thresholds.

The reference keeps all of this on the CPU (BaseQuantizer.get_static_hist_range and the helpers under
it, llmc/compression/quantization/quant.py:264-521: the running histogram is a CPU tensor and every
per-tensor histogram is moved to it); only the pass over the activations -- torch.histc per calibration
tensor -- touches device memory, and that pass is what lc_act_hist_per_tensor replaces.  The functions
here restate the reference's 2048-bin vector arithmetic op for op (same dtypes, same order), so that the
thresholds come out bit-identical given the same histograms.
"""
import torch


def quantization_error(histogram, min_val, max_val, next_start_bin, next_end_bin, bins, dst_nbins):
    """get_quantization_error (quant.py:279-330): L2 error of quantising the bins
    [next_start_bin, next_end_bin] of `histogram` onto dst_nbins levels."""
    bin_width = (max_val.item() - min_val.item()) / bins
    dst_bin_width = bin_width * (next_end_bin - next_start_bin + 1) / dst_nbins
    if dst_bin_width == 0.0:
        return 0.0
    src_bin = torch.arange(bins, device=histogram.device)
    src_bin_begin = (src_bin - next_start_bin) * bin_width
    src_bin_end = src_bin_begin + bin_width
    dst_bin_of_begin = torch.clamp(torch.div(src_bin_begin, dst_bin_width, rounding_mode='floor'), 0, dst_nbins - 1)
    dst_bin_of_begin_center = (dst_bin_of_begin + 0.5) * dst_bin_width
    dst_bin_of_end = torch.clamp(torch.div(src_bin_end, dst_bin_width, rounding_mode='floor'), 0, dst_nbins - 1)
    density = histogram / bin_width

    def norm_of(delta_begin, delta_end):
        # integral of x^2 between the deltas, times the density (quant.py:264-277)
        return density * ((delta_end * delta_end * delta_end - delta_begin * delta_begin * delta_begin) / 3)
    norm = torch.zeros(bins, device=histogram.device)
    norm += norm_of(src_bin_begin - dst_bin_of_begin_center, torch.ones(bins, device=histogram.device) * (dst_bin_width / 2))
    norm += (dst_bin_of_end - dst_bin_of_begin - 1) * norm_of(torch.tensor(-dst_bin_width / 2),
                                                              torch.tensor(dst_bin_width / 2))
    dst_bin_of_end_center = dst_bin_of_end * dst_bin_width + dst_bin_width / 2
    norm += norm_of(torch.tensor(-dst_bin_width / 2), src_bin_end - dst_bin_of_end_center)
    return norm.sum().item()


def hist_threshold(histogram, min_val, max_val, bins, dst_nbins):
    """get_hist_threshold (quant.py:402-459): shrink the range from whichever end gives up fewer bins,
    one 1e-8 quantile step at a time, while the quantisation error keeps falling."""
    assert histogram.size()[0] == bins, 'bins mismatch'
    bin_width = (max_val - min_val) / bins
    total = torch.sum(histogram).item()
    c_sum = torch.cumsum(histogram, dim=0)
    stepsize = 1e-8
    alpha, beta = 0.0, 1.0
    start_bin, end_bin = 0, bins - 1
    norm_min = float('inf')
    while alpha < beta:
        next_alpha, next_beta = alpha + stepsize, beta - stepsize
        left, right = start_bin, end_bin
        while left < end_bin and c_sum[left] < next_alpha * total:
            left = left + 1
        while right > start_bin and c_sum[right] > next_beta * total:
            right = right - 1
        next_start_bin, next_end_bin = start_bin, end_bin
        if (left - start_bin) > (end_bin - right):
            next_start_bin, alpha = left, next_alpha
        else:
            next_end_bin, beta = right, next_beta
        if next_start_bin == start_bin and next_end_bin == end_bin:
            continue
        norm = quantization_error(histogram, min_val, max_val, next_start_bin, next_end_bin, bins, dst_nbins)
        if norm > norm_min:
            break
        norm_min, start_bin, end_bin = norm, next_start_bin, next_end_bin
    return min_val + bin_width * start_bin, min_val + bin_width * (end_bin + 1)


def upscale_histogram(histogram, orig_min, orig_max, update_min, update_max, bins, upsample_rate):
    """_upscale_histogram (quant.py:332-366): the old histogram re-binned into the widened range."""
    histogram = histogram.repeat_interleave(upsample_rate) / upsample_rate
    bin_size = (orig_max - orig_min) / (bins * upsample_rate)
    mid_points = (torch.linspace(orig_min, orig_max, bins * upsample_rate + 1, device=orig_min.device)[:-1]
                  .to(histogram.device) + 0.5 * bin_size)
    boundaries = torch.linspace(update_min, update_max, bins + 1, device=update_min.device).to(histogram.device)
    assign = torch.bucketize(mid_points, boundaries, right=True) - 1
    assign[assign >= bins] = bins - 1
    assign[assign < 0] = 0
    return torch.bincount(assign, weights=histogram, minlength=bins)


def combine_histograms(orig_hist, orig_min, orig_max, update_hist, update_min, update_max, bins, upsample_rate):
    """_combine_histograms (quant.py:368-400)."""
    if update_min == orig_min and update_max == orig_max:
        return orig_hist + update_hist
    if orig_min == orig_max:
        bin_value = torch.sum(update_hist)
        return torch.histc(orig_min, bins=bins, min=update_min, max=update_max) * bin_value + update_hist
    assert update_min <= orig_min
    assert update_max >= orig_max
    return update_hist + upscale_histogram(orig_hist, orig_min, orig_max, update_min, update_max, bins, upsample_rate)


def static_hist_range(per_tensor_hists, running_min, running_max, bins, upsample_rate, dst_nbins):
    """The loop of get_static_hist_range (quant.py:461-521) over the tensors of one input, given what the
    device pass produced: per_tensor_hists[i] = histc of tensor i over [running_min[i], running_max[i]]
    (the running range after tensor i, fp32 host vectors).  Returns (new_min, new_max)."""
    histogram = per_tensor_hists[0].clone()
    min_val, max_val = running_min[0], running_max[0]
    for i in range(1, len(per_tensor_hists)):
        new_min, new_max = running_min[i], running_max[i]
        update = per_tensor_hists[i]
        if new_min == min_val and new_max == max_val:
            histogram = histogram + update
        else:
            histogram = combine_histograms(histogram, min_val, max_val, update, new_min, new_max, bins, upsample_rate)
        min_val, max_val = new_min, new_max
    return hist_threshold(histogram, min_val, max_val, bins, dst_nbins)
