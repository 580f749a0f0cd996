"""Packing of 4-bit codes into the two export layouts the reference writes
(llmc/compression/quantization/module_utils.py: VllmRealQuantLinear.pack :931-955,
AutoawqRealQuantLinear.gemm_pack :1099-1158)."""
import torch

from . import _lib as L


def pack_compressed_tensors_int4(weight, wquantizer):
    """Symmetric int4 real quant + compressed-tensors packing in one pass over the weight:
    returns (packed int32 (rows, cols/8), scales (rows, n_groups))."""
    if not wquantizer.sym or wquantizer.bit != 4:
        raise NotImplementedError('compressed-tensors int4 packing is for symmetric 4-bit weights')
    fake, packed, s, z = wquantizer.quant_all_dynamic(weight, packed=True)
    if packed.shape[1] % 4:
        raise ValueError('in_features must be a multiple of 8')
    return packed.view(torch.int32), s


def pack_compressed_tensors_int4_static(weight, scales, wquantizer):
    """The same with given scales (real_quant_weight_static, quant.py:870-913, then the packer): the
    export step of a GPTQ layer solved with static_groups, whose weight is the fp32 compensated weight
    and whose scales are the layer's buf_scales.  Returns (packed int32 (rows, cols/8), scales
    (rows, n_groups))."""
    if not wquantizer.sym or wquantizer.bit != 4:
        raise NotImplementedError('compressed-tensors int4 packing is for symmetric 4-bit weights')
    if weight.dim() != 2 or weight.shape[1] % 8:
        raise ValueError('in_features must be a multiple of 8')
    w = weight if weight.is_contiguous() else weight.contiguous()
    _, packed, _, _ = wquantizer._launch(w, wquantizer._group_len(w.shape[-1]), scales, None, codes=L.LC_CODES_PACK4)
    return packed.view(torch.int32), scales.reshape(w.shape[0], -1)


def pack_autoawq_gemm(codes_u8, zeros_u8):
    """AutoAWQ GEMM layout: codes (out, in) uint8 -> qweight (in, out/8) int32; zeros (out, n_groups)
    uint8 -> qzeros (n_groups, out/8) int32."""
    L.require_cuda(codes_u8, zeros_u8)
    outs = []
    for t in (codes_u8, zeros_u8):
        t = t.contiguous()
        R, C = t.shape
        o = torch.empty((C, R // 8), dtype=torch.int32, device=t.device)
        L.call('lc_pack_int4_awq', L.ptr(t), R, C, L.ptr(o), L.stream_of(t))
        outs.append(o)
    return outs[0], outs[1]


# ---- quantization_config / compression_config entries of the exported model's config.json ----------
# (llmc/utils/export_vllm.py:4-125, llmc/utils/export_autoawq.py:4-30).  `weight` and `act` are the
# `quant.weight` / `quant.act` sections of the YAML config as plain dicts.

def vllm_quant_config(weight, act=None, ignore=(), quant_method='compressed-tensors'):
    """Returns (key, entry): the key of config.json to set ('quantization_config' for the fp8
    checkpoints vLLM loads natively, else 'compression_config') and its value."""
    w_type = weight.get('quant_type', 'int-quant')
    a_type = act.get('quant_type', 'int-quant') if act is not None else None
    if act is not None and a_type != w_type:
        raise AssertionError('weights and activations must use the same quant_type')
    a_bits = None
    if a_type == 'float-quant':
        if act.get('static', False):
            return 'quantization_config', {'activation_scheme': 'static', 'ignored_layers': [list(ignore)],
                                           'quant_method': 'fp8'}
        if weight.get('granularity', 'per_block'):
            # (the reference tests the granularity string's truthiness, so every dynamic fp8 config lands here)
            bs = weight['block_size']
            return 'quantization_config', {'activation_scheme': 'dynamic', 'fmt': 'e4m3', 'quant_method': 'fp8',
                                           'weight_block_size': [bs, bs]}
        fmt, kind, w_bits, a_bits = 'float-quantized', 'float', 8, 8
    elif weight.get('need_pack', False):
        fmt, kind, w_bits = 'pack-quantized', 'int', weight['bit']
    elif w_type == 'float-quant':
        fmt, kind, w_bits = 'float-quantized', 'float', 8
    else:
        fmt, kind, w_bits = 'int-quantized', 'int', weight['bit']
        if act is not None:
            a_bits = act['bit']
    per_group = weight['granularity'] == 'per_group'
    inputs = None
    if act is not None:
        if a_bits is None:
            raise NameError('a_num_bits')     # the reference leaves it unset for packed / float weights with acts
        inputs = {'dynamic': not act['static'] if 'static' in act else True, 'group_size': None,
                  'num_bits': a_bits, 'observer': 'minmax', 'observer_kwargs': {},
                  'strategy': 'token' if act['granularity'] == 'per_token' else 'tensor',
                  'symmetric': act['symmetric'], 'type': kind}
    weights = {'dynamic': False, 'group_size': weight['group_size'] if per_group else None, 'num_bits': w_bits,
               'observer': 'minmax', 'observer_kwargs': {}, 'strategy': 'group' if per_group else 'channel',
               'symmetric': weight['symmetric'], 'type': kind}
    entry = {'config_groups': {'group_0': {'targets': ['Linear'], 'input_activations': inputs, 'weights': weights}},
             'format': fmt, 'ignore': list(ignore), 'quant_method': quant_method}
    return 'compression_config', entry


def autoawq_quant_config(weight):
    return {'bits': weight['bit'],
            'group_size': weight['group_size'] if weight['granularity'] == 'per_group' else -1,
            'modules_to_not_convert': None, 'quant_method': 'awq',
            'version': weight['pack_version'].split('_')[0], 'zero_point': not weight['symmetric']}


def update_config_json(save_quant_path, key, entry, drop_quantization_config=False):
    """Sets config.json[key] = entry in the exported model directory (indent 4, like the reference)."""
    import json
    import os
    path = os.path.join(save_quant_path, 'config.json')
    with open(path) as f:
        cfg = json.load(f)
    if drop_quantization_config and 'quantization_config' in cfg:
        del cfg['quantization_config']
    cfg[key] = entry
    with open(path, 'w') as f:
        json.dump(cfg, f, indent=4)


def update_vllm_quant_config(save_quant_path, weight, act=None, ignore=(), vllm_quant_method='compressed-tensors'):
    key, entry = vllm_quant_config(weight, act, ignore, vllm_quant_method)
    int_weights = weight.get('quant_type', 'int-quant') == 'int-quant'
    update_config_json(save_quant_path, key, entry,
                       drop_quantization_config=(key == 'compression_config' and int_weights))


def update_autoawq_quant_config(save_quant_path, weight):
    update_config_json(save_quant_path, 'quantization_config', autoawq_quant_config(weight),
                       drop_quantization_config=True)
