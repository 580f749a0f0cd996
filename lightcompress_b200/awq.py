"""Host-side mirror of the reference AWQ algorithm's hot methods.

Follows llmc/compression/quantization/awq.py (get_act_scale :74-85, get_scales :88-108,
fake_quantize_weight :147-164, calculate_loss :134-145, search_scale_subset :179-278,
block_transform :281-296, subset_transform :299-372), the scale application of
base_blockwise_quantization.py (scale_ln_fcs :773-801, scale_fc_fc :655-723, scaling_input :900-912,
update_input_feat :915-920) and auto_clip.py (AutoClipper.run :44-81, auto_clip_layer :84-191,
apply_clip :194-212) for the configuration on the hot path: trans_version v2, no GQA, weight-only,
clip_version v1, one calibration batch (calib.bs = -1).

What runs where: the per-candidate work on full tensors -- scaling + fake-quantising the
weights, scaling the activations, the output error, and the whole clip search -- is one fused
kernel each (C ABI).  The inspect-module forwards are the block's own torch modules.  The
candidate scale vectors (length in_features) are formed with the reference's own tiny torch
expressions so that their bf16 rounding is identical.  The 20 losses stay on the device; the
winning candidate is selected there (first minimum, like the reference's strict `<`), so a subset
costs no host synchronisation.
"""
import contextlib

import torch

from . import _lib as L
from . import block_ops, parallel
from .blockwise import PhaseTimer


def _is_norm(m):
    # norm layers: anything with a 1-D weight and no in_features (RMSNorm / LayerNorm)
    return hasattr(m, 'weight') and m.weight.dim() == 1


class Awq:
    def __init__(self, wquantizer, special=None, calib_seq_len=512):
        special = dict(special or {})
        self.wquantizer = wquantizer
        self.trans = special.get('trans', True)
        self.trans_version = special.get('trans_version', 'v2')
        self.weight_clip = special.get('weight_clip', True)
        self.clip_version = special.get('clip_version', 'v1')
        self.clip_sym = special.get('clip_sym', wquantizer.sym)
        self.n_grid = 20
        self.clip_n_grid, self.clip_max_shrink = 20, 0.5
        self.n_sample_token = calib_seq_len
        self.fused_block_ops = special.get('fused_block_ops', True)
        # clip search: the sums of the rounded products on the tensor cores ('tensor': MMAs against a matrix of
        # ones) or on the CUDA cores ('cuda_cores'); same products, another order of the fp32 additions
        self.clip_sums = special.get('clip_sums', 'tensor')
        self.phases = PhaseTimer()      # off unless a caller switches it on (bench.py)
        if self.trans_version != 'v2' or self.clip_version != 'v1':
            raise NotImplementedError('only trans_version v2 / clip_version v1 are on the B200 hot path')
        if wquantizer.granularity != 'per_group':
            raise NotImplementedError('the AWQ kernels need per_group weights')
        wquantizer._check_supported()

    # ---- kernels ---------------------------------------------------------------------------
    def get_act_scale(self, x):
        """mean |x| over all tokens (awq.py:74-76)."""
        L.require_cuda(x)
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        T, C = x2.shape
        out = torch.empty(C, dtype=x.dtype, device=x.device)
        splits = min(64, (T + 255) // 256)
        scratch = torch.empty(splits * C, dtype=torch.float32, device=x.device)
        L.call('lc_awq_act_mean', L.ptr(x2), L.lc_dtype(x2), T, C, L.ptr(out), L.ptr(scratch), scratch.numel(),
               L.stream_of(x2))
        if parallel.world()[1] > 1:
            # token shards: the kernel's fp32 partial sums of |x| are added over the ranks and divided by the
            # total token count, rounded to the activation dtype once -- the mean over all the data
            total, n = parallel.sum_and_count(scratch.view(splits, C).sum(0), T)
            out = (total / float(n)).to(x.dtype)
        return out

    def get_scales(self, x_mean, ratio):
        """trans_version v2 (awq.py:104-107); a handful of length-C torch ops, kept verbatim."""
        s = x_mean.pow(ratio).clamp(min=1e-4).view(-1)
        return s / (s.max() * s.min()).sqrt()

    def fake_quantize_weight(self, weight, scales, out=None):
        """qdq(weight * scales) without modifying `weight` (awq.py:40-46, :147-164)."""
        wq = self.wquantizer
        w = weight if weight.is_contiguous() else weight.contiguous()
        out = torch.empty_like(w) if out is None else out
        L.call('lc_awq_scale_quant', L.ptr(w), L.ptr(scales.to(w.dtype).contiguous()), L.lc_dtype(w), w.shape[0],
               w.shape[1], wq.group_size, int(wq.bit), int(wq.sym), L.ptr(out), L.stream_of(w))
        return out

    def scaling_input(self, x, scales, out=None):
        """x / scales (base_blockwise_quantization.py:900-912)."""
        x = x if x.is_contiguous() else x.contiguous()
        out = torch.empty_like(x) if out is None else out
        C = x.shape[-1]
        L.call('lc_awq_div_cols', L.ptr(x), L.ptr(scales.to(x.dtype).contiguous()), L.lc_dtype(x), x.numel() // C, C,
               L.ptr(out), L.stream_of(x))
        return out

    def calculate_loss(self, org_out, out, loss_slot, scratch):
        """mean((org_out - out)^2) into the device scalar `loss_slot` (awq.py:134-136)."""
        a = org_out if org_out.is_contiguous() else org_out.contiguous()
        b = out if out.is_contiguous() else out.contiguous()
        L.call('lc_awq_loss', L.ptr(a), L.ptr(b), L.lc_dtype(a), a.numel(), L.ptr(loss_slot), L.ptr(scratch),
               scratch.numel(), L.stream_of(a))

    # ---- scale search ------------------------------------------------------------------------
    @torch.no_grad()
    def search_scale_subset(self, layers, x, inspect_module, kwargs):
        """search_scale_subset for one input batch (awq.py:179-278).  Returns (best_scales, losses)
        with `losses` the n_grid errors as a device tensor."""
        L.require_cuda(x)
        dev = x.device
        org = [l.weight.data for l in layers]
        tmp = [torch.empty_like(w) for w in org]
        out = inspect_module(x, **kwargs)
        org_out = out[0] if isinstance(out, tuple) else out
        x_mean = self.get_act_scale(x)
        losses = torch.empty(self.n_grid, dtype=torch.float32, device=dev)
        scratch = torch.empty(1024, dtype=torch.float64, device=dev)
        cand = torch.empty((self.n_grid, x.shape[-1]), dtype=x.dtype, device=dev)
        x_tmp = torch.empty_like(x)
        for n in range(self.n_grid):
            s = self.get_scales(x_mean, n / self.n_grid)
            cand[n] = s
            for l, w, t in zip(layers, org, tmp):
                l.weight.data = self.fake_quantize_weight(w, s, out=t)
            self.scaling_input(x, s, out=x_tmp)
            out = inspect_module(x_tmp, **kwargs)
            out = out[0] if isinstance(out, tuple) else out
            self.calculate_loss(org_out, out, losses[n:n + 1], scratch)
            del out
        for l, w in zip(layers, org):
            l.weight.data = w
        if parallel.world()[1] > 1:
            # every rank evaluated the grid on its own tokens: squared-error sums and element counts are added
            # over the ranks, so all ranks pick the grid point of the whole calibration set
            n_el = org_out.numel()
            sums, total = parallel.sum_and_count(losses * float(n_el), n_el)
            losses = sums / float(total)
        best = torch.argmin(losses)            # first minimum == the reference's strict `<` update
        return cand.index_select(0, best.view(1)).view(-1), losses

    @torch.no_grad()
    def scale_ln_fcs(self, ln, fcs, scales):
        """base_blockwise_quantization.py:773-801."""
        scales = scales.to(ln.weight.dtype)
        ln.weight.div_(scales)
        if getattr(ln, 'bias', None) is not None:
            ln.bias.div_(scales)
        for fc in fcs:
            fc.weight.mul_(scales.view(1, -1))

    @torch.no_grad()
    def scale_fc_fc(self, fc1, fc2, scales):
        """base_blockwise_quantization.py:684-701, :723 (fc1.out_features == fc2.in_features)."""
        if fc1.out_features != fc2.in_features:
            raise NotImplementedError('only equal-width fc -> fc scaling is on the B200 hot path')
        if getattr(fc1, 'bias', None) is not None:
            fc1.bias.div_(scales.view(-1))
        fc1.weight.div_(scales.view(-1, 1))
        fc2.weight.mul_(scales.view(1, -1))

    def apply_scale(self, scales, prev_op, layers):
        if _is_norm(prev_op):
            self.scale_ln_fcs(prev_op, layers, scales)
        else:
            assert len(layers) == 1
            self.scale_fc_fc(prev_op, layers[0], scales)

    # ---- clip search -------------------------------------------------------------------------
    @torch.no_grad()
    def auto_clip_layer(self, weight, x, apply=True):
        """auto_clip_layer + apply_clip (auto_clip.py:84-212): returns (best_max, best_min), each
        (out_features, n_groups, 1); with apply=True `weight` is clamped in place."""
        wq = self.wquantizer
        L.require_cuda(weight, x)
        w = weight if weight.is_contiguous() else weight.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        R, C = w.shape
        n_tok_all = x2.shape[0]
        step = max(1, n_tok_all // self.n_sample_token)
        n_g = C // wq.group_size
        best_max = torch.empty((R, n_g, 1), dtype=w.dtype, device=w.device)
        best_min = torch.empty((R, n_g, 1), dtype=w.dtype, device=w.device)
        multi = parallel.world()[1] > 1
        L.call('lc_awq_clip_search' if self.clip_sums == 'tensor' else 'lc_awq_clip_search_cuda_cores',
               L.ptr(w), L.ptr(x2), L.lc_dtype(w), R, C, n_tok_all, step, wq.group_size,
               int(wq.bit), int(wq.sym), int(self.clip_sym), self.clip_n_grid, float(self.clip_max_shrink),
               L.ptr(best_max), L.ptr(best_min), L.ptr(w) if apply and not multi else None, L.stream_of(w))
        if multi:
            # AutoClipper.run averages the ranks' thresholds before clamping (auto_clip.py:72-76, :194-212)
            parallel.average_over_ranks(best_max)
            parallel.average_over_ranks(best_min)
            if apply:
                wg = w.view(R, n_g, wq.group_size)
                lo = -best_max if self.clip_sym else best_min
                w.copy_(torch.clamp(wg, lo, best_max).view(R, C))
        if apply and w.data_ptr() != weight.data_ptr():
            weight.copy_(w)
        return best_max, best_min

    # ---- one Llama-layout block ----------------------------------------------------------------
    @torch.no_grad()
    def block_transform(self, block, x, kwargs):
        """Awq.block_transform on a block with the Llama layout (subsets of llmc/models/llama.py:52-91):
        four scale searches with their scale application, then the clip search on v, o, gate, up,
        down (q / k are skipped, auto_clip.py:56-60).  x: (B, T, C) hidden states, one batch.
        Modifies the block in place; returns a report dict."""
        a, m = block.self_attn, block.mlp
        dtype, dev = a.q_proj.weight.dtype, a.q_proj.weight.device
        with contextlib.ExitStack() as stack:
            if self.fused_block_ops:
                # the inspect-module forwards run 80 times per block: their rotary embedding and gated
                # activation go through one kernel each, bit-identical to the modules' own tensor ops
                stack.enter_context(block_ops.fused_rotary(a, dev, dtype))
                stack.enter_context(block_ops.fused_gated_mlp(m))
            return self._block_transform(block, x, kwargs)

    @torch.no_grad()
    def _block_transform(self, block, x, kwargs):
        a, m = block.self_attn, block.mlp
        feats, hooks = {}, []
        for name, mod in (('q', a.q_proj), ('o', a.o_proj), ('gate', m.gate_proj), ('down', m.down_proj)):
            def hook(mod_, inp, out, name=name):
                feats[name] = inp[0].data
            hooks.append(mod.register_forward_hook(hook))
        out = block(x, **kwargs)
        for h in hooks:
            h.remove()
        report = {'scales': {}, 'losses': {}, 'clip': {}, 'output': out[0] if isinstance(out, tuple) else out}
        if self.trans:
            plan = (('qkv', [a.q_proj, a.k_proj, a.v_proj], 'q', a, kwargs, block.input_layernorm),
                    ('o', [a.o_proj], 'o', a.o_proj, {}, a.v_proj),
                    ('gate_up', [m.gate_proj, m.up_proj], 'gate', m, {}, block.post_attention_layernorm),
                    ('down', [m.down_proj], 'down', m.down_proj, {}, m.up_proj))
            for key, layers, f, inspect, kw, prev in plan:
                with self.phases('scale_search'):
                    s, ls = self.search_scale_subset(layers, feats[f], inspect, kw)
                    self.apply_scale(s, prev, layers)
                    feats[f] = self.scaling_input(feats[f], s)
                report['scales'][key], report['losses'][key] = s, ls
        if self.weight_clip:
            for name, mod, f in (('v', a.v_proj, 'q'), ('o', a.o_proj, 'o'), ('gate', m.gate_proj, 'gate'),
                                 ('up', m.up_proj, 'gate'), ('down', m.down_proj, 'down')):
                with self.phases('clip_search'):
                    report['clip'][name] = self.auto_clip_layer(mod.weight.data, feats[f])
        return report
