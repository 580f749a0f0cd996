"""Oracle restatement of the reference's per-block GPTQ schedule (test infrastructure).

Follows llmc/compression/quantization/base_blockwise_quantization.py (block_opt :403-432, run
:447-485, block_transform :487-527, rehook_next_subset :529-549) with GPTQ's hooks
(gptq.py:247-251, :298-322) and the Llama subsets (llmc/models/llama.py:52-91), literally: every
linear accumulates its own Hessian in the first pass, later subsets are re-initialised and
re-accumulated after the earlier ones were replaced by fake-quant linears.
"""
import torch
import torch.nn.functional as F

from . import gptq_ref


class _FakeQuantLinear(torch.nn.Module):
    """module_utils.py:679-771 reduced to what the schedule needs."""

    def __init__(self, weight_q, bias):
        super().__init__()
        self.tmp_weight = weight_q
        self.bias = bias

    def forward(self, x):
        return F.linear(x, self.tmp_weight, self.bias)


def llama_subsets(block):
    a, m = block.self_attn, block.mlp
    return [[('self_attn.q_proj', a, 'q_proj'), ('self_attn.k_proj', a, 'k_proj'), ('self_attn.v_proj', a, 'v_proj')],
            [('self_attn.o_proj', a, 'o_proj')],
            [('mlp.gate_proj', m, 'gate_proj'), ('mlp.up_proj', m, 'up_proj')],
            [('mlp.down_proj', m, 'down_proj')]]


@torch.no_grad()
def _forward(block, inputs, kwargs):
    outs = []
    for x in inputs:
        o = block(x, **kwargs)
        outs.append(o[0] if isinstance(o, tuple) else o)
    return outs


@torch.no_grad()
def gptq_block(block, inputs, kwargs, bit=4, sym=False, percdamp=0.01, actorder=True,
               true_sequential=True, quant_out=True, model_dtype=torch.bfloat16, capture=None, subsets=None):
    """Runs one decoder block through the schedule.  Returns (per-linear results, next inputs).
    Each result is gptq_ref.quantize_layer's dict plus 'w_qdq' (the deployed weight).
    capture: a dict that receives, per linear, the list of input tensors its final Hessian was
    accumulated from (for teacher-forced comparisons of a single linear).
    subsets: another adapter's subsets, e.g. llmc/models/opt.py:53-90."""
    # subsets: lists of (name, parent module, attribute) in schedule order, as the model adapters'
    # get_subsets_in_block give them (default: the Llama adapter's, llmc/models/llama.py:52-91)
    subsets = subsets if subsets is not None else llama_subsets(block)
    states, handles = {}, []

    def hook_layers(items):
        hs = []
        for name, parent, attr in items:
            layer = getattr(parent, attr)
            states[name] = gptq_ref.hessian_init(layer.weight.shape[1], layer.weight.device)
            if capture is not None:
                capture[name] = []                  # re-initialised with the Hessian (subset_init)
            def hook(m, inp, out, name=name):       # must return None: a value would replace the output
                gptq_ref.add_batch(states[name], inp[0].data)
                if capture is not None:
                    capture[name].append(inp[0].data)
            hs.append(layer.register_forward_hook(hook))
        return hs

    handles = hook_layers([it for s in subsets for it in s])      # block_init + register_hooks
    first_out = _forward(block, inputs, kwargs)
    for h in handles:
        h.remove()
    results = {}
    for i, subset in enumerate(subsets):
        for name, parent, attr in subset:
            layer = getattr(parent, attr)
            res = gptq_ref.quantize_layer(layer.weight.data, states[name]['H'], bit, sym, 128, 128, percdamp, actorder)
            res['w_qdq'] = gptq_ref.w_qdq(res, model_dtype, bit, sym)
            results[name] = res
        if true_sequential and i + 1 < len(subsets):
            for name, parent, attr in subset:
                setattr(parent, attr, _FakeQuantLinear(results[name]['w_qdq'], getattr(getattr(parent, attr), 'bias', None)))
            hs = hook_layers(subsets[i + 1])                       # subset_init re-zeroes the next subset
            _forward(block, inputs, kwargs)
            for h in hs:
                h.remove()
    if quant_out:
        for subset in subsets:
            for name, parent, attr in subset:
                mod = getattr(parent, attr)
                if not isinstance(mod, _FakeQuantLinear):
                    setattr(parent, attr, _FakeQuantLinear(results[name]['w_qdq'], getattr(mod, 'bias', None)))
        outs = _forward(block, inputs, kwargs)
    else:
        outs = first_out
    return results, outs
