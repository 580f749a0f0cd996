"""Binds the B200 kernels into LightCompress's own plugin classes.

    import lightcompress_b200.plugin as plugin
    plugin.install()            # after `llmc` is importable; before the algorithm object is constructed
    ...                         # llmc/__main__.py runs unchanged: ALGO_REGISTRY[method](model, quant_config,
                                # input, padding_mask, config).run_block_loop(); .deploy('fake_quant')

What `install()` changes, all of it on the imported `llmc` modules of this process (no file is edited):

  * the names `IntegerQuantizer`, `FloatQuantizer`, `Weight48IntegerQuantizer` that
    `BaseBlockwiseQuantization.set_quant_config` instantiates from the YAML dicts
    (llmc/compression/quantization/base_blockwise_quantization.py:156-193) become the classes of
    `lightcompress_b200.quant` (same constructor keywords, attributes and method names);
  * `ALGO_REGISTRY['GPTQ' | 'Awq' | 'RTN' | 'SpQR']` become subclasses of the registered classes.  Item
    assignment goes through `Register.__setitem__` (llmc/utils/registry_factory.py:23-24), which does
    not run the duplicate-name check of the decorator.  Constructor signature, YAML keys, the `buf_*`
    buffers left on every linear and the replacement modules in the blocks stay the reference's.

GPTQ: `layer_init`, `add_batch`, `layer_transform`, `w_qdq` and `free` forward to
`lightcompress_b200.GPTQ` (Hessian on tcgen05, factorisation, 128-column solver, fused deploy
weight).  `block_opt` runs the per-block schedule through `lightcompress_b200.GPTQBlockwise` (one
Hessian per subset, every module of a Llama-layout block evaluated once); `quant.special.b200_schedule:
'reference'` keeps the reference's own `block_opt` / `run` / `block_transform` / `rehook_next_subset`
and only swaps the methods above.
Awq: `block_transform` runs the fused scale + clip search of `lightcompress_b200.Awq` for blocks with
the Llama layout and one calibration batch (`calib.bs: -1`); other cases raise.
RTN: nothing to override beyond the quantizer classes (llmc/compression/quantization/rtn.py:10-28).
SpQR: the per-layer methods forward to `lightcompress_b200.SpQR`; its block loop stays the reference's.

`uninstall()` restores every name.
"""
import gc

import torch

from . import quant as _quant
from .awq import Awq as _B200Awq
from .blockwise import GPTQBlockwise, is_llama_layout
from .gptq import GPTQ as _B200GPTQ
from .spqr import SpQR as _B200SpQR

_saved = {}


def _to_device(v, dev):
    if torch.is_tensor(v):
        return v.to(dev)
    if isinstance(v, tuple):
        return tuple(_to_device(t, dev) for t in v)
    return v


def _subset_pairs(block, subsets):
    """The adapter's subsets (dicts with 'layers': {name: module}, llmc/models/llama.py:52-91) as the
    (parent, attribute) pairs the block schedule swaps modules through."""
    from collections import OrderedDict
    out = []
    for sub in subsets:
        d = OrderedDict()
        for name in sub['layers']:
            parent_name, _, attr = name.rpartition('.')
            d[name] = (block.get_submodule(parent_name) if parent_name else block, attr)
        out.append(d)
    return out


def _make_gptq(RefGPTQ, rmu):
    class GPTQ(RefGPTQ):
        """The registered GPTQ algorithm (llmc/compression/quantization/gptq.py:22) over the B200 kernels."""

        def __init__(self, model, quant_config, input, padding_mask, config, modality='language'):
            super().__init__(model, quant_config, input, padding_mask, config, modality)
            # the constructor re-creates the dict after add_quant_config (gptq.py:31)
            self.layers_cache = self._b200.layers_cache

        @torch.no_grad()
        def add_quant_config(self):
            super().add_quant_config()
            special = dict(self.quant_config['special'])
            self._b200 = _B200GPTQ(self.wquantizer, special, self.model_dtype)
            self._schedule = special.get('b200_schedule', 'b200')
            self._runner = GPTQBlockwise(
                self.wquantizer, special, self.model_dtype, quant_out=self.quant_out, solver=self._b200,
                fake_linear=lambda m: rmu.FakeQuantLinear.new(
                    m, **self.get_replacement_params(mode='fake_quant', w_only=self.w_only, name=None)))

        # ---- per-layer hot methods (gptq.py:298-308, :254-295, :114-117, :425-452, :466-471) ----
        @torch.no_grad()
        def layer_init(self, layer, name):
            self._b200.layer_init(layer, name)

        @torch.no_grad()
        def add_batch(self, layer, name, inp, out):
            self._b200.add_batch(layer, name, inp, out)

        @torch.no_grad()
        def layer_transform(self, layer, name):
            if self.owq and not self._b200.n_out_dict:
                self._b200.n_out_dict = dict(self.n_out_dict)
            self._b200.layer_transform(layer, name)
            self._b200.check_status()

        @torch.no_grad()
        def w_qdq(self, module, wquantizer):
            return self._b200.w_qdq(module, wquantizer)

        @torch.no_grad()
        def free(self, name):
            self._b200.layers_cache.pop(name, None)

        # ---- per-block schedule (base_blockwise_quantization.py:403-432, :447-549) ----
        @torch.no_grad()
        def block_opt(self, block):
            if (self._schedule == 'reference' or self.data_free or self.act_static or self.quant_kvcache
                    or self.quant_attn or self.quant_act_fn or self.online_rotate
                    or self._is_ignored_block(self.block_idx)):
                return super().block_opt(block)
            block = block.cuda()
            dev = next(block.parameters()).device
            data, kwargs = self.input['data'], self.input['kwargs']
            for i in range(len(data)):
                data[i] = data[i].to(dev)
                kwargs[i] = {k: _to_device(v, dev) for k, v in kwargs[i].items()}
            subsets = self.model.get_subsets_in_block(block)
            pairs = None if is_llama_layout(block) and len(subsets) == 4 else _subset_pairs(block, subsets)
            if self.owq and not self._b200.n_out_dict:
                self._b200.set_block_linears(list(self.model.get_block_linears(block)))
            self.input['data'] = self._runner.block_opt(block, data, kwargs, subsets=pairs)
            block = block.cpu()
            gc.collect()

    GPTQ.__name__ = GPTQ.__qualname__ = 'GPTQ'
    return GPTQ


def _make_awq(RefAwq):
    class Awq(RefAwq):
        """The registered Awq algorithm (llmc/compression/quantization/awq.py:29) over the B200 kernels."""

        def __init__(self, model, quant_config, input, padding_mask, config):
            super().__init__(model, quant_config, input, padding_mask, config)
            special = dict(self.quant_config.get('special', {}))
            special.setdefault('clip_sym', self.wquantizer.sym)
            self._b200 = _B200Awq(self.wquantizer, special, calib_seq_len=self.config.calib.get('seq_len', 512))

        @torch.no_grad()
        def block_opt(self, block):
            if self.data_free or self.act_static or self.quant_kvcache or self._is_ignored_block(self.block_idx):
                return super().block_opt(block)
            if (not is_llama_layout(block) or len(self.input['data']) != 1 or not self.w_only
                    or self.save_scale or getattr(self, 'save_clip', False)):
                raise NotImplementedError('the B200 AWQ path covers Llama-layout blocks, weight-only, one calibration '
                                          'batch (calib.bs: -1), without save_scale / save_clip')
            block = block.cuda()
            dev = next(block.parameters()).device
            x = self.input['data'][0].to(dev)
            kw = {k: _to_device(v, dev) for k, v in self.input['kwargs'][0].items()}
            self.input['kwargs'][0] = kw
            report = self._b200.block_transform(block, x, kw)
            if self.quant_out:
                # run() forwards once more through the fake-quantised block (:474-484)
                self.model.replace_module_block(
                    _saved['rmu'].FakeQuantLinear, block, self.block_idx,
                    self.get_replacement_params(mode='fake_quant', w_only=self.w_only, name=None))
                out = block(x, **kw)
                self.input['data'] = [out[0] if isinstance(out, tuple) else out]
            else:
                self.input['data'] = [report['output']]
            block = block.cpu()
            gc.collect()

    Awq.__name__ = Awq.__qualname__ = 'Awq'
    return Awq


def _make_spqr(RefSpQR):
    class SpQR(RefSpQR):
        """The registered SpQR algorithm (llmc/compression/quantization/spqr.py:19) over the B200 kernels:
        the per-layer methods forward to `lightcompress_b200.SpQR`; the block loop (hooks, true_sequential
        re-forwards, module replacement, spqr.py:60-112) stays the reference's."""

        def __init__(self, model, quant_config, input, padding_mask, config):
            super().__init__(model, quant_config, input, padding_mask, config)
            self.layers_cache = self._b200.layers_cache        # the constructor re-creates the dict (spqr.py:29)

        @torch.no_grad()
        def add_quant_config(self):
            super().add_quant_config()
            self._b200 = _B200SpQR(self.wquantizer, dict(self.quant_config['special']), self.model_dtype)

        @torch.no_grad()
        def layer_init(self, layer, name):
            self._b200.layer_init(layer, name)

        @torch.no_grad()
        def add_batch(self, layer, name, inp, out):
            self._b200.add_batch(layer, name, inp, out)

        @torch.no_grad()
        def layer_transform(self, layer, name):
            self._b200.layer_transform(layer, name)
            self._b200.check_status()

        @torch.no_grad()
        def w_qdq(self, module, wquantizer):
            return self._b200.w_qdq(module, wquantizer)

        @torch.no_grad()
        def free(self, name):
            self._b200.layers_cache.pop(name, None)

    SpQR.__name__ = SpQR.__qualname__ = 'SpQR'
    return SpQR


def _make_rtn(RefRTN):
    class RTN(RefRTN):
        """llmc/compression/quantization/rtn.py:10-28: no transform; `deploy` calls w_qdq / w_q / a_qdq of the
        base class, which call the (swapped) quantizer objects."""

    RTN.__name__ = RTN.__qualname__ = 'RTN'
    return RTN


def install():
    """Idempotent.  Needs `llmc` importable (the reference's checkout on sys.path)."""
    if _saved:
        return _saved['classes']
    import llmc.compression.quantization.awq as rawq
    import llmc.compression.quantization.base_blockwise_quantization as rbase
    import llmc.compression.quantization.gptq as rgptq
    import llmc.compression.quantization.module_utils as rmu
    import llmc.compression.quantization.rtn as rrtn
    import llmc.compression.quantization.spqr as rspqr
    from llmc.utils.registry_factory import ALGO_REGISTRY
    _saved['rmu'] = rmu
    _saved['quantizers'] = {n: getattr(rbase, n) for n in
                            ('IntegerQuantizer', 'FloatQuantizer', 'Weight48IntegerQuantizer')}
    _saved['algos'] = {n: ALGO_REGISTRY[n] for n in ('GPTQ', 'Awq', 'RTN', 'SpQR')}
    _saved['rbase'], _saved['registry'] = rbase, ALGO_REGISTRY
    for n in _saved['quantizers']:
        setattr(rbase, n, getattr(_quant, n))
    classes = {'GPTQ': _make_gptq(rgptq.GPTQ, rmu), 'Awq': _make_awq(rawq.Awq), 'RTN': _make_rtn(rrtn.RTN),
               'SpQR': _make_spqr(rspqr.SpQR)}
    for n, c in classes.items():
        ALGO_REGISTRY[n] = c
    _saved['classes'] = classes
    return classes


def uninstall():
    if not _saved:
        return
    for n, c in _saved['quantizers'].items():
        setattr(_saved['rbase'], n, c)
    for n, c in _saved['algos'].items():
        _saved['registry'][n] = c
    _saved.clear()


def installed():
    return bool(_saved)


__all__ = ['install', 'uninstall', 'installed']
