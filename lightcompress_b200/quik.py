"""Host-side mirror of the reference QUIK algorithm (llmc/compression/quantization/quik.py): the
outlier feature columns of every linear, picked by a per-channel max |x| over the calibration
activations, stay in floating point in both the weight and the activation fake quant.

The statistic is one kernel per hooked call on the device (lc_quik_col_absmax) instead of an abs / max /
host copy per call, and w_qdq / a_qdq are one masked row kernel each (lc_rtn_int_fake_quant_masked)
instead of gather -> quantise -> two scatters.  Index selection (a sort of `hidden` values per linear)
is host logic, as in the reference.
"""
import functools

import torch
import torch.nn as nn

from . import _lib as L


class QUIK:
    def __init__(self, wquantizer, aquantizer, special, quant_config=None):
        self.wquantizer = wquantizer
        self.aquantizer = aquantizer
        self.fp_relative = special['fp_relative']
        self.fp_features = special['fp_features']
        self.fp_threshold = special['fp_threshold']
        # quik.py:23-24 looks for last_fc_bit at the top level of the quant config and reads it from `special`
        if quant_config is not None and 'last_fc_bit' in quant_config:
            self.last_fc_bit = special['last_fc_bit']
        self.act_scales = {}

    # ---- statistic (quik.py:30-89) --------------------------------------------------------------
    @torch.no_grad()
    def get_tensor_scale(self, name, tensor):
        hidden = tensor.shape[-1]
        x = tensor.detach().reshape(-1, hidden)
        x = x if x.is_contiguous() else x.contiguous()
        L.require_cuda(x)
        run = self.act_scales.get(name)
        if run is None:
            run = self.act_scales[name] = torch.zeros(hidden, dtype=torch.float32, device=x.device)
        L.call('lc_quik_col_absmax', L.ptr(x), L.lc_dtype(x), x.shape[0], hidden, L.ptr(run), L.stream_of(x))

    def stat_input_hook(self, m, x, y, name):
        if isinstance(x, tuple):
            x = x[0]
        self.get_tensor_scale(name, x)

    def register_hooks(self, root, prefix=''):
        """Forward hooks on every nn.Linear under `root`, keyed like the reference keys them
        (module path from the model root); returns the handles."""
        hooks = []
        for name, m in root.named_modules():
            if isinstance(m, nn.Linear):
                full = f'{prefix}.{name}' if prefix else name
                hooks.append(m.register_forward_hook(functools.partial(self.stat_input_hook, name=full)))
        return hooks

    # ---- column selection (quik.py:91-126) ------------------------------------------------------
    @torch.no_grad()
    def block_opt(self, layers_dict, block_prefix, hidden_size=None):
        """layers_dict: name -> linear of one block (get_block_linears); block_prefix: e.g.
        'model.layers.3'.  Registers buf_int_ids / buf_fp_ids (and buf_current_bit) like the reference.
        fp_relative scales the outlier count by in_features / hidden_size of the linear (the reference
        reads `block.in_features`, which a decoder block does not have)."""
        for n, m in layers_dict.items():
            layer_name = f'{block_prefix}.{n}'
            if self.fp_relative:
                outlier_num = int(m.in_features / hidden_size) * self.fp_features
            else:
                outlier_num = self.fp_features
            layer_scales = None
            if outlier_num > 0:
                layer_scales = self.act_scales[layer_name].float().cpu()
                max_val = layer_scales.abs().max()
                fp_threshold = self.fp_threshold
                if hasattr(self, 'last_fc_bit'):
                    if 'dense_4h_to_h' in n or 'down_proj' in n:
                        fp_threshold = self.fp_threshold * 2
                        m.register_buffer('buf_current_bit', torch.tensor(self.last_fc_bit))
                if max_val <= fp_threshold:
                    outlier_num = 0
                    layer_scales = None
            if layer_scales is None:
                # the reference calls torch.sort(None) here and stops with a TypeError
                raise TypeError(f'QUIK: no outlier columns for {layer_name} (fp_features = 0 or every activation '
                                'scale is at or below fp_threshold); the reference cannot proceed either')
            order = torch.sort(layer_scales)[1]
            dev = m.weight.device
            m.register_buffer('buf_int_ids', order[:-outlier_num].to(dev))
            m.register_buffer('buf_fp_ids', order[-outlier_num:].to(dev))
            del self.act_scales[layer_name]

    # ---- deploy-time fake quant (quik.py:128-151) -----------------------------------------------
    def _args(self, module):
        args = {'int_indices': module.buf_int_ids, 'fp_indices': module.buf_fp_ids}
        if hasattr(module, 'buf_current_bit'):
            args['current_bit'] = module.buf_current_bit
        return args

    def w_qdq(self, module, wquantizer):
        return self.wquantizer.fake_quant_weight_dynamic(module.weight, self._args(module))

    def a_qdq(self, act, module, aquantizer):
        return self.aquantizer.fake_quant_act_dynamic(act, self._args(module))
