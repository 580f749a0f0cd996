"""Host-side mirrors of the reference quantizer objects.

`IntegerQuantizer` and `FloatQuantizer` keep the constructor signature, attributes and method
names of llmc/compression/quantization/quant.py (BaseQuantizer :48-103, IntegerQuantizer
:660-959, FloatQuantizer :962-1228) so that the algorithm classes and replacement modules that
call them work unchanged, but every method body is one launch of a fused sm_100a kernel through
the C ABI.  Configurations outside the accelerated path (calib_algo other than 'minmax', for
integer weights 'mse', and for per_tensor activations 'static_minmax' / 'static_moving_minmax';
per_head granularity, per_tensor weights, round_zp=False, mixed-precision index args) raise
NotImplementedError: there is no fallback.
"""
import ctypes

import torch

from . import _lib as L

_INT_GRANS = ('per_group', 'per_channel', 'per_token')
_STATIC_ALGOS = ('static_minmax', 'static_moving_minmax', 'static_hist')


class BaseQuantizer(object):
    """Constructor contract of quant.py:48-103."""

    def __init__(self, bit, symmetric, granularity, **kwargs):
        self.bit = bit
        self.sym = symmetric
        self.granularity = granularity
        self.kwargs = kwargs
        self.calib_algo = kwargs.get('calib_algo', 'minmax')
        if granularity == 'per_group':
            self.group_size = kwargs['group_size']
        elif granularity == 'per_head':
            self.head_num = kwargs['head_num']
        elif granularity == 'per_block':
            self.block_size = kwargs['block_size']
        self.round_zp = kwargs.get('round_zp', True)
        self.mse_b_num = kwargs.get('mse_b_num', 1)
        self.maxshrink = kwargs.get('maxshrink', 0.8)
        self.mse_grid = kwargs.get('mse_grid', 100)
        self.ste = kwargs.get('ste', False)
        self.ste_all = bool(kwargs.get('ste_all', False))
        self.bins = kwargs.get('bins', 2048)          # static_hist (quant.py:83-87)
        self.upsample_rate = 16

    def _check_supported(self, allow_mse=False, per_tensor=False):
        """per_tensor: the caller is one of the static per-tensor activation methods."""
        ok = (self.calib_algo == 'minmax' or (allow_mse and self.calib_algo == 'mse')
              or (per_tensor and self.calib_algo in _STATIC_ALGOS))
        if not ok:
            raise NotImplementedError(f"calib_algo '{self.calib_algo}' is outside the B200 hot path")
        if self.granularity not in _INT_GRANS and not (per_tensor and self.granularity == 'per_tensor'):
            raise NotImplementedError(f"granularity '{self.granularity}' is outside the B200 hot path")
        if not self.round_zp:
            raise NotImplementedError('round_zp=False is outside the B200 hot path')

    def _group_len(self, last_dim):
        """Group length along the last dim, 0 = whole row; mirrors reshape_tensor (quant.py:611-641)."""
        if self.granularity == 'per_group':
            if last_dim >= self.group_size:
                if last_dim % self.group_size:
                    raise ValueError(
                        f'Dimension {last_dim} not divisible by group size {self.group_size}')
                return self.group_size
        return 0

    def reshape_tensor(self, tensor, allow_padding=False):
        g = self._group_len(tensor.shape[-1])
        if self.granularity == 'per_group' and g:
            return tensor.reshape(-1, g)
        if self.granularity in _INT_GRANS or self.granularity == 'per_tensor':
            return tensor
        raise NotImplementedError(self.granularity)

    def restore_tensor(self, tensor, shape):
        return tensor if tensor.shape == shape else tensor.reshape(shape)


def _as_2d(t):
    t = t if t.is_contiguous() else t.contiguous()
    return t, t.reshape(-1, t.shape[-1])


class IntegerQuantizer(BaseQuantizer):
    """quant.py:660-959 over lc_rtn_int_quant."""

    def __init__(self, bit, symmetric, granularity, **kwargs):
        super().__init__(bit, symmetric, granularity, **kwargs)
        self.quant_type = 'int-quant'
        if 'int_range' in kwargs:
            raise NotImplementedError('int_range is outside the B200 hot path')
        if self.sym:
            self.qmin = torch.tensor(-(2 ** (bit - 1)))
            self.qmax = torch.tensor(2 ** (bit - 1) - 1)
        else:
            self.qmin = torch.tensor(0.0)
            self.qmax = torch.tensor(2 ** bit - 1)
        self.dst_nbins = 2 ** bit

    # ---- one fused launch ------------------------------------------------------------------
    def _launch(self, t2d, group, scales_in=None, zeros_in=None, fake=False, codes=L.LC_CODES_NONE,
                params=False):
        self._check_supported(allow_mse=scales_in is not None,
                              per_tensor=scales_in is not None and self.granularity == 'per_tensor')
        L.require_cuda(t2d, scales_in, zeros_in)
        rows, cols = t2d.shape
        g = group if group else cols
        n_groups = rows * (cols // g) if cols else 0
        dev, dt = t2d.device, t2d.dtype
        fake_out = torch.empty_like(t2d) if fake else None
        codes_out = None
        if codes == L.LC_CODES_I32:
            codes_out = torch.empty((rows, cols), dtype=torch.int32, device=dev)
        elif codes == L.LC_CODES_I8:
            codes_out = torch.empty((rows, cols), dtype=torch.int8 if self.sym else torch.uint8, device=dev)
        elif codes == L.LC_CODES_PACK4:
            codes_out = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
        s_out = torch.empty((n_groups, 1), dtype=dt, device=dev) if params else None
        z_out = torch.empty((n_groups, 1), dtype=dt, device=dev) if params and not self.sym else None
        if scales_in is not None:
            scales_in = scales_in.to(dt).contiguous()
            if scales_in.numel() != n_groups:
                raise NotImplementedError('static scales must hold one value per group')
            if zeros_in is not None and not self.sym:
                zeros_in = zeros_in.to(dt).contiguous()
                if zeros_in.numel() != n_groups:
                    raise NotImplementedError('static zeros must hold one value per group')
            else:
                zeros_in = None
        L.call('lc_rtn_int_quant', L.ptr(t2d), L.lc_dtype(t2d), rows, cols, group, int(self.bit), int(self.sym),
               L.ptr(scales_in), L.ptr(zeros_in), L.ptr(fake_out), L.ptr(codes_out), codes, L.ptr(s_out),
               L.ptr(z_out), L.stream_of(t2d))
        return fake_out, codes_out, s_out, z_out

    def _code_fmt(self):
        return L.LC_CODES_I8 if self.bit == 8 else L.LC_CODES_I32

    # ---- calib_algo 'mse' (quant.py:147-205) --------------------------------------------------
    def get_mse_range(self, tensor, norm=2.4, bs=256):
        """(min, max) of the grouped tensor after the shrink-grid search, fp32, one value per group:
        one launch of lc_rtn_mse_range (the reference: about a dozen tensor ops per grid step)."""
        if self.quant_type != 'int-quant':
            raise NotImplementedError('the MSE range kernel covers the integer quantizer')
        self._check_supported(allow_mse=True)
        L.require_cuda(tensor)
        if tensor.shape[0] % self.mse_b_num:
            raise AssertionError('Batch number must be divisible by tensor.shape[0],')
        t, t2d = _as_2d(tensor)
        rows, cols = t2d.shape
        mn = torch.empty((rows, 1), dtype=torch.float32, device=t.device)
        mx = torch.empty((rows, 1), dtype=torch.float32, device=t.device)
        L.call('lc_rtn_mse_range', L.ptr(t2d), L.lc_dtype(t2d), rows, cols, 0, int(self.bit), int(self.sym),
               float(self.maxshrink), int(self.mse_grid), float(norm), L.ptr(mn), L.ptr(mx), L.stream_of(t2d))
        return mn, mx

    def get_tensor_range(self, tensor, args={}):
        """Range of an already grouped tensor (quant.py:124-132)."""
        if self.calib_algo == 'mse':
            return self.get_mse_range(tensor)
        raise NotImplementedError("get_tensor_range is only a separate step for calib_algo 'mse'; "
                                  'the minmax range is fused into the quantisation kernels')

    def get_qparams(self, tensor_range, device):
        """scales / zeros from a (min, max) pair (quant.py:544-558): a handful of ops on one value per
        group, in the range's dtype."""
        mn, mx = tensor_range
        qmin, qmax = self.qmin.to(device), self.qmax.to(device)
        if self.sym:
            scales = torch.maximum(mx.abs(), mn.abs()).clamp(min=1e-5) / qmax
            return scales, torch.tensor(0.0), qmax, qmin
        scales = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
        zeros = (qmin - torch.round(mn / scales)).clamp(qmin, qmax)
        return scales, zeros, qmax, qmin

    def _mse_params(self, tensor):
        grouped = self.reshape_tensor(tensor if tensor.is_contiguous() else tensor.contiguous())
        scales, zeros, qmax, qmin = self.get_qparams(self.get_mse_range(grouped), tensor.device)
        return grouped, scales, zeros, qmax, qmin

    def _fake_mse(self, weight):
        # fp32 parameters make the reference's quant / dequant ops run in fp32 on the promoted tensor;
        # the result returns to the weight's dtype (quant.py:832-868)
        grouped, scales, zeros, _, _ = self._mse_params(weight)
        g32 = grouped.float()
        fake, _, _, _ = self._launch(g32, g32.shape[-1], scales, None if self.sym else zeros, fake=True)
        return fake.reshape(weight.shape).to(weight.dtype)

    # ---- reference API ---------------------------------------------------------------------
    def get_tensor_qparams(self, tensor, args={}):
        if self.calib_algo == 'mse':
            return self._mse_params(tensor)
        t, t2d = _as_2d(tensor)
        group = self._group_len(t.shape[-1])
        _, _, s, z = self._launch(t2d, group, params=True)
        shape = s.shape if group else (*t.shape[:-1], 1)
        s = s.reshape(shape)
        z = torch.tensor(0.0) if self.sym else z.reshape(shape)
        return self.reshape_tensor(t), s, z, self.qmax, self.qmin

    def _static_2d(self, tensor):
        t, t2d = _as_2d(tensor)
        return t, t2d, (t2d.shape[-1] if t2d.shape[-1] else 0)

    def quant(self, tensor, scales, zeros, qmax, qmin):
        """tensor is already grouped (rows, group); scales/zeros hold one value per row."""
        t, t2d, g = self._static_2d(tensor)
        _, codes, _, _ = self._launch(t2d, g, scales, None if self.sym else zeros, codes=L.LC_CODES_I32)
        return codes.to(t.dtype).reshape(t.shape)

    def dequant(self, tensor, scales, zeros):
        # Not on the hot path: the fused kernels never materialise codes as floats.
        return (tensor - zeros) * scales

    def quant_dequant(self, tensor, scales, zeros, qmax, qmin, output_scale_factor=1):
        if output_scale_factor != 1:
            raise NotImplementedError('output_scale_factor is outside the B200 hot path')
        t, t2d, g = self._static_2d(tensor)
        fake, _, _, _ = self._launch(t2d, g, scales, None if self.sym else zeros, fake=True)
        return fake.reshape(t.shape)

    def _reject_args(self, args, allowed=()):
        # keys the base class always passes with value None (lowbound_factor / upbound_factor,
        # base_blockwise_quantization.py:50-56) carry no request
        bad = [k for k in args if k not in allowed and args[k] is not None]
        if bad:
            raise NotImplementedError(f'args {bad} are outside the B200 hot path')

    def _fake_masked(self, tensor, args):
        """Mixed precision (quant.py:753-782, :832-868 with int_indices / fp_indices): rows quantised over
        their integer columns, floating-point columns passed through, in one kernel.  `current_bit` is
        accepted and, as in the reference, changes nothing: qmin / qmax were fixed by the constructor."""
        self._reject_args(args, ('int_indices', 'fp_indices', 'current_bit'))
        self._check_supported()
        if self.granularity == 'per_group':
            raise NotImplementedError('int_indices with per_group (groups over the gathered column order) is '
                                      'outside the B200 hot path')
        L.require_cuda(tensor)
        t, t2d = _as_2d(tensor)
        rows, cols = t2d.shape
        int_ids, fp_ids = args['int_indices'], args['fp_indices']
        key = (int_ids.data_ptr(), fp_ids.data_ptr(), int(int_ids.numel()), int(fp_ids.numel()), cols, str(t.device))
        cache = self.__dict__.setdefault('_mask_cache', {})
        mask = cache.get(key)
        if mask is None:
            mask = torch.full((cols,), 2, dtype=torch.uint8, device=t.device)
            mask[int_ids.to(t.device)] = 0
            mask[fp_ids.to(t.device)] = 1          # the reference scatters the fp part last
            if len(cache) > 256:
                cache.clear()
            # the index tensors are held so that their addresses cannot be reused under the cached key
            cache[key] = (mask, int_ids, fp_ids)
        else:
            mask = mask[0]
        out = torch.empty_like(t2d)
        L.call('lc_rtn_int_fake_quant_masked', L.ptr(t2d), L.lc_dtype(t2d), rows, cols, int(self.bit), int(self.sym),
               L.ptr(mask), L.ptr(out), L.stream_of(t2d))
        return out.reshape(t.shape)

    def fake_quant_weight_dynamic(self, weight, args={}):
        if 'int_indices' in args:
            return self._fake_masked(weight, args)
        self._reject_args(args)
        if self.calib_algo == 'mse':
            return self._fake_mse(weight)
        t, t2d = _as_2d(weight)
        fake, _, _, _ = self._launch(t2d, self._group_len(t.shape[-1]), fake=True)
        return fake.reshape(t.shape)

    def fake_quant_act_dynamic(self, act, args={}):
        if 'int_indices' in args:
            return self._fake_masked(act, args)
        self._reject_args(args)
        t, t2d = _as_2d(act)
        fake, _, _, _ = self._launch(t2d, self._group_len(t.shape[-1]), fake=True)
        return fake.reshape(t.shape)

    def fake_quant_weight_static(self, weight, args):
        self._reject_args(args, ('scales', 'zeros', 'qmax', 'qmin'))
        t, t2d = _as_2d(weight)
        fake, _, _, _ = self._launch(t2d, self._group_len(t.shape[-1]), args['scales'],
                                     None if self.sym else args.get('zeros'), fake=True)
        return fake.reshape(t.shape)

    def fake_quant_act_static(self, act, args={}):
        """quant.py:718-751.  per_tensor (the only granularity the reference allows for static
        activations, base_blockwise_quantization.py:183-186): the scalar scale / zero point enter the
        row kernel as one value per row.  They are first cast to the activation dtype, which is what the
        reference's tensor ops do with the 0-dim CUDA buffers the calibration registered."""
        if self.granularity != 'per_tensor':
            return self.fake_quant_weight_static(act, args)
        self._reject_args(args, ('scales', 'zeros', 'qmax', 'qmin'))
        t, t2d = _as_2d(act)
        rows = t2d.shape[0]
        scales, zeros = args['scales'], args.get('zeros')
        if scales.numel() != 1:
            raise NotImplementedError('per_tensor static quantisation takes one scale')
        s_rows = scales.to(device=t.device, dtype=t.dtype).reshape(1).expand(rows).contiguous()
        z_rows = None
        if not self.sym:
            z_rows = zeros.to(device=t.device, dtype=t.dtype).reshape(1).expand(rows).contiguous()
        fake, _, _, _ = self._launch(t2d, 0, s_rows, z_rows, fake=True)
        return fake.reshape(t.shape)

    # ---- static per-tensor activation ranges (quant.py:105-122, :134-137, :223-262, :523-585) ----
    def _tensor_ranges(self, tensors):
        """(mins, maxs) of a list of CUDA tensors of one dtype: fp32 device vectors, one launch."""
        self._check_supported(per_tensor=True)
        if self.granularity != 'per_tensor':
            raise NotImplementedError('batched activation ranges are per_tensor (the reference allows no other '
                                      'granularity for static activations)')
        tensors = [t if t.is_contiguous() else t.contiguous() for t in tensors]
        L.require_cuda(*tensors)
        n = len(tensors)
        if any(t.dtype != tensors[0].dtype or t.device != tensors[0].device for t in tensors):
            raise NotImplementedError('calibration tensors of one input must share dtype and device')
        dev = tensors[0].device
        mins = torch.empty(n, dtype=torch.float32, device=dev)
        maxs = torch.empty(n, dtype=torch.float32, device=dev)
        ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors])
        numels = (ctypes.c_int64 * n)(*[t.numel() for t in tensors])
        L.call('lc_act_range_per_tensor', ptrs, numels, n, L.lc_dtype(tensors[0]), L.ptr(mins), L.ptr(maxs),
               L.stream_of(tensors[0]))
        return mins, maxs, tensors

    def get_minmax_range(self, tensor):
        """per_tensor (quant.py:135-137): 0-dim (min, max) in the tensor's dtype.  For the other
        granularities the range never leaves the fused quantisation kernels."""
        mins, maxs, _ = self._tensor_ranges([tensor])
        return mins[0].to(tensor.dtype), maxs[0].to(tensor.dtype)

    def reshape_batch_tensors(self, act_tensors):
        """quant.py:105-122."""
        assert len(act_tensors) > 0, (
            'Calibration data is insufficient. Please provide more data to ensure '
            'all experts in the MOE receive an adequate number of tokens.')
        if isinstance(act_tensors[0], tuple):
            return [torch.stack(list(ts)) for ts in zip(*act_tensors)]
        if len(act_tensors) == 1:
            return [[act_tensors[0][i] for i in range(act_tensors[0].size(0))]]
        return [act_tensors]

    def get_minmax_stats(self, act_tensors):
        """quant.py:223-250: per input, the (N,) fp32 host vectors of every tensor's min and max."""
        stats = {}
        for idx, tensors in enumerate(act_tensors):
            mins, maxs, _ = self._tensor_ranges(list(tensors))
            stats[idx] = {'min': mins.cpu(), 'max': maxs.cpu()}
        return stats

    def get_static_minmax_range(self, act_tensors):
        """quant.py:252-262: the mean of the per-tensor ranges, on the host in fp32 like the reference."""
        stats = self.get_minmax_stats(self.reshape_batch_tensors(act_tensors))
        return ([r['min'].mean(dim=0) for r in stats.values()], [r['max'].mean(dim=0) for r in stats.values()])

    def get_static_moving_minmax_range(self, act_tensors, alpha):
        """quant.py:523-542: exponential moving average of the per-tensor ranges in the tensors' dtype;
        one launch for the ranges, one single-warp launch for the average."""
        mins_out, maxs_out = [], []
        for tensors in self.reshape_batch_tensors(act_tensors):
            mins, maxs, ts = self._tensor_ranges(list(tensors))
            out2 = torch.empty(2, dtype=torch.float32, device=mins.device)
            L.call('lc_act_range_moving', L.ptr(mins), L.ptr(maxs), len(ts), L.lc_dtype(ts[0]), float(alpha),
                   L.ptr(out2), L.stream_of(ts[0]))
            mins_out.append(out2[0].to(ts[0].dtype))
            maxs_out.append(out2[1].to(ts[0].dtype))
        return mins_out, maxs_out

    def get_static_hist_range(self, act_tensors):
        """quant.py:461-521.  Per input: the tensors' ranges (one launch), the running range after each
        tensor (two tiny cumulative ops on the per-tensor values), every tensor's 2048-bin histogram over its
        running range (one launch over the whole batch; the reference calls torch.histc per tensor on an
        fp32 copy), then the reference's own host-side histogram merging and threshold search (hist.py)."""
        from . import hist as HH
        mins_out, maxs_out = [], []
        for tensors in self.reshape_batch_tensors(act_tensors):
            mins, maxs, ts = self._tensor_ranges(list(tensors))
            run_min, run_max = torch.cummin(mins, 0).values, torch.cummax(maxs, 0).values
            n = len(ts)
            hists = torch.empty((n, self.bins), dtype=torch.float32, device=mins.device)
            ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
            numels = (ctypes.c_int64 * n)(*[t.numel() for t in ts])
            L.call('lc_act_hist_per_tensor', ptrs, numels, n, L.lc_dtype(ts[0]), L.ptr(run_min), L.ptr(run_max),
                   int(self.bins), L.ptr(hists), L.stream_of(ts[0]))
            hists, run_min, run_max = hists.cpu(), run_min.cpu(), run_max.cpu()
            new_min, new_max = HH.static_hist_range([hists[i] for i in range(n)], run_min, run_max, self.bins,
                                                    self.upsample_rate, self.dst_nbins)
            mins_out.append(new_min)
            maxs_out.append(new_max)
        return mins_out, maxs_out

    def get_batch_tensors_qparams(self, act_tensors, alpha=0.01, args={}):
        """quant.py:560-585."""
        if self.calib_algo == 'static_hist':
            assert self.sym is True and self.granularity == 'per_tensor', \
                'Only support per tensor static symmetric int quantize.'
            min_vals, max_vals = self.get_static_hist_range(act_tensors)
        elif self.calib_algo == 'static_minmax':
            min_vals, max_vals = self.get_static_minmax_range(act_tensors)
        elif self.calib_algo == 'static_moving_minmax':
            min_vals, max_vals = self.get_static_moving_minmax_range(act_tensors, alpha)
        else:
            raise ValueError(f'Unsupported calibration algorithm: {self.calib_algo}')
        scales_list, zeros_list, qmin_list, qmax_list = [], [], [], []
        for mn, mx in zip(min_vals, max_vals):
            scales, zeros, qmax, qmin = self.get_qparams((mn, mx), mn.device)
            scales_list.append(scales)
            zeros_list.append(zeros)
            qmin_list.append(qmin)
            qmax_list.append(qmax)
        return scales_list, zeros_list, qmin_list, qmax_list

    def _real(self, weight, scales=None, zeros=None):
        t, t2d = _as_2d(weight)
        if t.dim() != 2:
            raise NotImplementedError('real quant expects a 2-D weight')
        dyn = scales is None
        _, codes, s, z = self._launch(t2d, self._group_len(t.shape[-1]), scales, zeros,
                                      codes=self._code_fmt(), params=dyn)
        if not dyn:
            s, z = scales, (None if self.sym else zeros)
        s = s.reshape(t.shape[0], -1)
        z = None if self.sym else z.to(codes.dtype).reshape(t.shape[0], -1)
        return codes, s, z

    def real_quant_weight_dynamic(self, weight, args={}):
        self._reject_args(args)
        return self._real(weight)

    def real_quant_weight_static(self, weight, args):
        self._reject_args(args, ('scales', 'zeros', 'qmax', 'qmin'))
        return self._real(weight, args['scales'], args.get('zeros'))

    # ---- additions (no counterpart on the reference quantizer) -------------------------------
    def quant_all_dynamic(self, weight, packed=False):
        """One pass producing everything: (fake, codes, scales, zeros).  With packed=True (4-bit)
        the codes are two nibbles per byte, low nibble first, stored as q - qmin."""
        t, t2d = _as_2d(weight)
        fmt = L.LC_CODES_PACK4 if packed else self._code_fmt()
        fake, codes, s, z = self._launch(t2d, self._group_len(t.shape[-1]), fake=True, codes=fmt, params=True)
        return fake.reshape(t.shape), codes, s.reshape(t2d.shape[0], -1), (
            None if self.sym else z.reshape(t2d.shape[0], -1))

    def __repr__(self):
        return (f'IntegerQuantizer(bit={self.bit}, sym={self.sym}, granularity={self.granularity}, '
                f'kwargs={self.kwargs}, qmin={self.qmin}, qmax={self.qmax})')


class FloatQuantizer(BaseQuantizer):
    """quant.py:962-1228 (use_qtorch path, e4m3): per_channel / per_token / per_group over lc_fp8_e4m3_quant
    (scales in the tensor's dtype), per_block weights over lc_fp8_e4m3_block_quant (fp32 scales, one per
    128 x 128 block)."""

    def __init__(self, bit, symmetric, granularity, **kwargs):
        super().__init__(bit, symmetric, granularity, **kwargs)
        self.sym = True
        self.quant_type = 'float-quant'
        self.e_bits = int(self.bit[1])
        self.m_bits = int(self.bit[-1])
        self.sign_bits = 1
        self.num_bits = self.e_bits + self.m_bits + self.sign_bits
        self.use_qtorch = kwargs.get('use_qtorch')
        if self.bit != 'e4m3' or not self.use_qtorch or 'float_range' in kwargs:
            raise NotImplementedError('only e4m3 with use_qtorch=True is on the B200 hot path')
        finfo = torch.finfo(torch.float8_e4m3fn)
        self.qmin, self.qmax = torch.tensor(finfo.min), torch.tensor(finfo.max)

    def _launch(self, t2d, fake=False, codes=False, scales=False):
        if self.calib_algo != 'minmax' or self.granularity not in ('per_channel', 'per_token', 'per_group'):
            raise NotImplementedError(f'{self.calib_algo}/{self.granularity} is outside the B200 hot path')
        L.require_cuda(t2d)
        shape = t2d.shape
        if self.granularity == 'per_group' and shape[-1] >= self.group_size:
            if shape[-1] % self.group_size:
                raise ValueError(f'Dimension {shape[-1]} not divisible by group size {self.group_size}')
            t2d = t2d.reshape(-1, self.group_size)      # every group is a row of the kernel
            fake_out, codes_out, s_out = self._launch_rows(t2d, fake, codes, scales)
            return (None if fake_out is None else fake_out.reshape(shape),
                    None if codes_out is None else codes_out.reshape(shape), s_out)
        return self._launch_rows(t2d, fake, codes, scales)

    def _launch_rows(self, t2d, fake, codes, scales):
        rows, cols = t2d.shape
        fake_out = torch.empty_like(t2d) if fake else None
        codes_out = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=t2d.device) if codes else None
        s_out = torch.empty((rows, 1), dtype=t2d.dtype, device=t2d.device) if scales else None
        L.call('lc_fp8_e4m3_quant', L.ptr(t2d), L.lc_dtype(t2d), rows, cols, L.ptr(fake_out), L.ptr(codes_out),
               L.ptr(s_out), L.stream_of(t2d))
        return fake_out, codes_out, s_out

    def _launch_block(self, weight, fake=False, codes=False):
        """per_block (quant.py:637-641, :138-140): one launch over the 2-D weight, fp32 block scales."""
        if self.calib_algo != 'minmax':
            raise NotImplementedError(f'{self.calib_algo}/per_block is outside the B200 hot path')
        if self.block_size != 128:
            raise NotImplementedError('the block-wise FP8 kernel has 128 x 128 blocks')
        L.require_cuda(weight)
        if weight.dim() != 2:
            raise ValueError('per_block quantisation expects a 2-D weight')
        m, n = weight.shape
        if m % 128 and n % 128:
            # the reference's restore_tensor cannot undo padding in both dimensions (quant.py:646-650)
            raise RuntimeError(f'per_block: a {m} x {n} weight is ragged in both dimensions')
        w = weight if weight.is_contiguous() else weight.contiguous()
        fake_out = torch.empty_like(w) if fake else None
        codes_out = torch.empty((m, n), dtype=torch.float8_e4m3fn, device=w.device) if codes else None
        s_out = torch.empty((-(-m // 128), -(-n // 128)), dtype=torch.float32, device=w.device)
        L.call('lc_fp8_e4m3_block_quant', L.ptr(w), L.lc_dtype(w), m, n, 128, L.ptr(fake_out), L.ptr(codes_out),
               L.ptr(s_out), L.stream_of(w))
        return fake_out, codes_out, s_out

    def get_tensor_qparams(self, tensor, args={}):
        if self.granularity == 'per_block':
            raise NotImplementedError('per_block: use fake_quant_weight_dynamic / real_quant_weight_dynamic')
        t, t2d = _as_2d(tensor)
        _, _, s = self._launch(t2d, scales=True)
        if self.granularity == 'per_group' and t.shape[-1] >= self.group_size:
            return t.reshape(-1, self.group_size), s, torch.tensor(0.0), self.qmax, self.qmin
        return t, s.reshape(*t.shape[:-1], 1), torch.tensor(0.0), self.qmax, self.qmin

    def fake_quant_weight_dynamic(self, weight, args={}):
        if any(v is not None for v in args.values()):
            raise NotImplementedError(f'args {list(args)} are outside the B200 hot path')
        if self.granularity == 'per_block':
            return self._launch_block(weight, fake=True)[0]
        t, t2d = _as_2d(weight)
        return self._launch(t2d, fake=True)[0].reshape(t.shape)

    fake_quant_act_dynamic = fake_quant_weight_dynamic

    def real_quant_weight_dynamic(self, weight, args={}):
        if any(v is not None for v in args.values()):
            raise NotImplementedError(f'args {list(args)} are outside the B200 hot path')
        if self.granularity == 'per_block':
            _, codes, s = self._launch_block(weight, codes=True)
            return codes, s, None
        t, t2d = _as_2d(weight)
        _, codes, s = self._launch(t2d, codes=True, scales=True)
        return codes.reshape(t.shape), s.reshape(t.shape[0], -1), None

    def __repr__(self):
        return (f'FloatQuantizer(bit={self.bit}, e_bits={self.e_bits}, m_bits={self.m_bits}, '
                f'granularity={self.granularity}, kwargs={self.kwargs}, qmin={self.qmin}, qmax={self.qmax})')


class _W48Level(ctypes.Structure):
    """lc_w48_level of the C ABI."""
    _fields_ = [('qmin', ctypes.c_float), ('qmax', ctypes.c_float), ('symmetric', ctypes.c_int),
                ('scales_min', ctypes.c_float), ('scales_max', ctypes.c_float),
                ('zeros_min', ctypes.c_float), ('zeros_max', ctypes.c_float)]


class Weight48IntegerQuantizer(BaseQuantizer):
    """quant.py:1230-1367 over lc_rtn_w48_fake_quant: weights to 8 bits per row, those codes to 4 bits
    per group, and back, in one pass.  The constructor keeps the reference's `bit_settings` (same keys,
    including its use of scales_bit for the zero-point limits, quant.py:1272-1281)."""

    def __init__(self, bit, bit4, bit8, **kwargs):
        super().__init__(bit, None, None, **kwargs)
        self.quant_type = 'int-quant-w48'
        assert self.bit == 48, 'Only support 48-bit quantization'
        self.bit_settings = {4: dict(bit4), 8: dict(bit8)}
        for b in (4, 8):
            st = self.bit_settings[b]
            if 'int_range' in st:
                st['qmin'], st['qmax'] = st['int_range'][0], st['int_range'][1]
            elif st['symmetric']:
                st['qmin'], st['qmax'] = -(2 ** (b - 1)), 2 ** (b - 1) - 1
            else:
                st['qmin'], st['qmax'] = 0, 2 ** b - 1
            st['qmin'], st['qmax'] = torch.tensor(st['qmin']), torch.tensor(st['qmax'])
            if 'scales_bit' in st:
                if st['scales_symmetric']:
                    st['scales_qmin'], st['scales_qmax'] = -(2 ** (st['scales_bit'] - 1)), 2 ** (st['scales_bit'] - 1) - 1
                else:
                    st['scales_qmin'], st['scales_qmax'] = 0, 2 ** st['scales_bit'] - 1
            else:
                st['scales_qmin'], st['scales_qmax'] = -torch.inf, torch.inf
            if 'zeros_bit' in st:
                if st['zeros_symmetric']:
                    st['zeros_qmin'], st['zeros_qmax'] = -(2 ** (st['scales_bit'] - 1)), 2 ** (st['scales_bit'] - 1) - 1
                else:
                    st['zeros_qmin'], st['zeros_qmax'] = 0, 2 ** st['scales_bit'] - 1
            else:
                st['zeros_qmin'], st['zeros_qmax'] = st['qmin'], st['qmax']

    def _level(self, b):
        st = self.bit_settings[b]
        return _W48Level(float(st['qmin']), float(st['qmax']), int(bool(st['symmetric'])),
                         float(st['scales_qmin']), float(st['scales_qmax']),
                         float(st['zeros_qmin']), float(st['zeros_qmax']))

    def fake_quant_weight_dynamic(self, weight, args={}):
        if any(v is not None for v in args.values()):
            raise NotImplementedError(f'args {list(args)} are outside the B200 hot path')
        if self.calib_algo != 'minmax':
            raise NotImplementedError(f"calib_algo '{self.calib_algo}' is outside the B200 hot path")
        g8, g4 = self.bit_settings[8].get('granularity'), self.bit_settings[4].get('granularity')
        if g8 == 'per_group' or g4 != 'per_group':
            # the kernel is built for the layout the reference ships (rows to 8 bits, groups to 4 bits)
            raise NotImplementedError('the two-level kernel takes a row-wise 8-bit and a per_group 4-bit level')
        L.require_cuda(weight)
        t, t2d = _as_2d(weight)
        rows, cols = t2d.shape
        group = int(self.bit_settings[4]['group_size'])
        if cols % group:
            raise ValueError(f'Dimension {cols} not divisible by group size {group}')
        out = torch.empty_like(t2d)
        l8, l4 = self._level(8), self._level(4)
        L.call('lc_rtn_w48_fake_quant', L.ptr(t2d), L.lc_dtype(t2d), rows, cols, group, ctypes.byref(l8),
               ctypes.byref(l4), L.ptr(out), L.stream_of(t2d))
        return out.reshape(t.shape)

    def __repr__(self):
        return f'Weight48IntegerQuantizer(bit_settings={self.bit_settings})'


def weight_cast_to_fp8(weight, block_size=128):
    """quant.py:36-45 (kernel.py:73-83 when Triton is usable): (e4m3 weight, fp32 scales per block)."""
    q = FloatQuantizer('e4m3', True, 'per_block', block_size=block_size, use_qtorch=True)
    codes, scales, _ = q.real_quant_weight_dynamic(weight)
    return codes, scales


def weight_cast_to_bf16(weight, scale, block_size=128):
    """quant.py:20-33 (kernel.py:115-131): e4m3 weight * its block scale, as bf16."""
    if block_size != 128:
        raise NotImplementedError('the block-wise FP8 kernel has 128 x 128 blocks')
    L.require_cuda(weight, scale)
    w = weight if weight.is_contiguous() else weight.contiguous()
    s = scale.to(torch.float32).contiguous()
    m, n = w.shape
    if s.shape != (-(-m // 128), -(-n // 128)):
        raise ValueError('scale must hold one value per 128 x 128 block')
    out = torch.empty((m, n), dtype=torch.bfloat16, device=w.device)
    L.call('lc_fp8_e4m3_block_dequant', L.ptr(w), L.ptr(s), m, n, 128, L.ptr(out), L.LC_BF16, L.stream_of(out))
    return out
