"""SpQR on the B200 kernels: host mirror of llmc/compression/quantization/spqr.py.

Same per-layer methods as the reference's registered `SpQR` class (layer_init, add_batch, layer_transform,
w_qdq, free); the Hessian, the act-order sort, dampening and the inverse Cholesky factor are the GPTQ
solver's (spqr.py:117-160 and :287-316 are the GPTQ steps with two differences handled here: the damp is a
fraction of mean|diag| taken before dead columns are set, and those get a diagonal of exactly 1), the
column loop with outlier detection is `lc_spqr_weight_transform`, the deploy-time weight `lc_spqr_dequant`.

Supported: the configuration of the reference's spqr_w_only.yml — asymmetric integer weights, per_group
with groups of 16, round_zp False, blocksize 128, second-level statistics in groups of 16 — with any
relative_threshold (inf: no outliers), simplified_outliers on or off, act-order on or off.  Anything else
raises NotImplementedError.
"""
import math

import torch

from . import _lib as L
from .gptq import GPTQ


class SpQR(GPTQ):
    def __init__(self, wquantizer, special=None, model_dtype=torch.bfloat16):
        special = dict(special or {})
        self.relative_threshold = special.get('relative_threshold', 0.2)
        if self.relative_threshold == 'inf':                      # spqr.py:46-47
            self.relative_threshold = math.inf
        self.simplified_outliers = bool(special.get('simplified_outliers', False))
        self.stat_configs = (special.get('scale'), special.get('zero'))
        gptq_special = {k: v for k, v in special.items() if k in (
            'actorder', 'percdamp', 'blocksize', 'true_sequential', 'factorization', 'own_cholesky_min', 'trailing',
            'hessian_batch', 'hessian_ksplit', 'shared_inverse', 'shared_inverse_min')}
        gptq_special.setdefault('percdamp', 1)
        super().__init__(wquantizer, gptq_special, model_dtype)
        self.need_perm = bool(self.actorder)                       # spqr.py:43-44
        self.prep_flags = L.LC_H_LATE_DEAD

    def _check_config(self):
        wq = self.wquantizer
        self.per_channel = False
        if (wq.granularity != 'per_group' or wq.group_size != 16 or wq.sym or wq.round_zp or self.blocksize != 128
                or getattr(wq, 'calib_algo', 'minmax') != 'minmax'):
            raise NotImplementedError('SpQR kernels need asymmetric per_group weights with group_size 16, '
                                      'round_zp False and blocksize 128')
        for cfg in self.stat_configs:
            # the reference hands the statistic quantizers (rows, 1) tensors, on which any per_group quantizer
            # with unrounded zero points degenerates to the same arithmetic; that is what the kernel restates
            if cfg is not None and (cfg.get('granularity') != 'per_group' or cfg.get('symmetric', False)
                                    or cfg.get('round_zp', True) or int(cfg.get('bit', 3)) != 3):
                raise NotImplementedError('SpQR kernels need 3-bit asymmetric per_group statistic quantizers with '
                                          'round_zp False')

    def uses_static(self):
        return False

    @torch.no_grad()
    def outlier_threshold(self, Wp, U):
        """relative_threshold * mean(var(W, dim 0) / diag(U)^2) (spqr.py:205-207) as a device scalar: the
        product is formed in double and rounded to fp32 like the reference's Python float against an fp32
        tensor."""
        if self.relative_threshold == math.inf:
            return torch.full((1,), math.inf, dtype=torch.float32, device=Wp.device)
        scale = (Wp.var(dim=0) / torch.diag(U).square()).mean()
        return (scale.double() * float(self.relative_threshold)).float().reshape(1)

    @torch.no_grad()
    def solve(self, W, H, hscale=1.0, rows=None, factor=None, static=None, threshold=None):
        wq = self.wquantizer
        fac = factor or self.factorize(H, hscale)
        H, perm, invperm, U = fac['H'], fac['perm'], fac['invperm'], fac['U']
        L.require_cuda(W, H)
        W = W if W.is_contiguous() else W.contiguous()
        R_all, C = W.shape
        if C % 128:
            raise NotImplementedError('SpQR kernels need columns % 128 == 0')
        dev, stream = W.device, L.stream_of(W)
        # the threshold is a statistic of all rows of the permuted weight, also when only a row range is solved
        Wp_all = torch.empty((R_all, C), dtype=torch.float32, device=dev)
        L.call('lc_gptq_permute_damp', L.ptr(W), L.lc_dtype(W), L.ptr(H), L.ptr(perm), R_all, C, 1.0, 0.0, 0,
               L.ptr(Wp_all), None, None, stream)
        thr = threshold if threshold is not None else self.outlier_threshold(Wp_all, U)
        Wp = Wp_all if rows is None else Wp_all[rows[0]:rows[1]].contiguous()
        R = Wp.shape[0]
        n_groups = C // 16
        err = torch.empty((128, R), dtype=torch.float32, device=dev)
        scales = torch.empty((R * n_groups, 1), dtype=torch.float32, device=dev)
        zeros = torch.empty((R * n_groups, 1), dtype=torch.float32, device=dev)
        mask = torch.zeros((R, C), dtype=torch.uint8, device=dev)
        loss_rows = torch.empty(R, dtype=torch.float32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        tc = fac.get('U_lo') is not None and R % 4 == 0
        panel = torch.empty((2, 1024, R), dtype=torch.float32, device=dev) if tc else None
        L.call('lc_spqr_weight_transform', L.ptr(Wp), L.ptr(U), L.ptr(fac['U_lo']) if tc else None, R, C, int(wq.bit),
               L.ptr(thr), int(self.simplified_outliers), L.ptr(err), L.ptr(panel[0]) if tc else None,
               L.ptr(panel[1]) if tc else None, L.ptr(scales), L.ptr(zeros), L.ptr(mask), L.ptr(loss_rows),
               L.ptr(status), stream)
        self._pending_status.append(status)
        out = torch.empty((R, C), dtype=torch.float32, device=dev)
        L.call('lc_gptq_unpermute', L.ptr(Wp), L.ptr(perm), R, C, L.ptr(out), L.LC_F32, stream)
        mask_o = mask if invperm is None else mask[:, invperm].contiguous()
        return {'weight': out, 'buf_scales': scales, 'buf_zeros': zeros, 'buf_perm': perm, 'buf_invperm': invperm,
                'mask': mask_o, 'loss_rows': loss_rows, 'threshold': thr}

    def _install(self, layer, res):
        layer.weight.data = res['weight'].reshape(layer.weight.shape)
        wq = self.wquantizer
        for k in ('buf_scales', 'buf_zeros', 'buf_perm', 'buf_invperm'):
            v = res.get(k)
            if v is None:
                continue
            if k in layer._buffers:
                layer._buffers[k] = v
            else:
                layer.register_buffer(k, v)
        for k, v in (('buf_qmax', wq.qmax), ('buf_qmin', wq.qmin)):
            if k not in layer._buffers:
                layer.register_buffer(k, v.to(layer.weight.device))
        # spqr.py:181: the mask is kept as a sparse float tensor; the dense bytes stay beside it for w_qdq
        sparse = res['mask'].float().to_sparse()
        if 'buf_mask' in layer._buffers:
            layer._buffers['buf_mask'] = sparse
        else:
            layer.register_buffer('buf_mask', sparse)
        layer._lc_mask = (res['mask'], layer.weight.data.data_ptr())
        layer._lc_codes = None

    @torch.no_grad()
    def w_qdq(self, module, wquantizer):
        """spqr.py:367-390 in one kernel."""
        weight = module.weight.data
        kept = getattr(module, '_lc_mask', None)
        if kept is not None and kept[1] == weight.data_ptr():
            mask = kept[0]
        else:
            mask = (module.buf_mask.to_dense() != 0).to(torch.uint8)
        w32 = weight.float().contiguous()
        R, C = w32.shape
        out = torch.empty((R, C), dtype=self.model_dtype, device=w32.device)
        L.call('lc_spqr_dequant', L.ptr(w32), L.ptr(module.buf_scales), L.ptr(module.buf_zeros), L.ptr(mask.contiguous()),
               L.ptr(module.buf_invperm) if self.need_perm else None, R, C, int(wquantizer.bit), L.ptr(out),
               L.lc_dtype(out), L.stream_of(w32))
        return out
