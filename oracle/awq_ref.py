"""Oracle restatement of the reference AWQ scale + clip search (test infrastructure).

Follows llmc/compression/quantization/awq.py (get_act_scale :74-85, get_scales :88-108,
scaling_weight :40-46, fake_quantize_weight :147-164, calculate_loss :134-145,
search_scale_subset :179-278, subset_transform :299-372), base_blockwise_quantization.py
(scale_ln_fcs :773-801, scale_fc_fc :655-723 equal-width branch, scaling_input :900-912,
update_input_feat :915-920) and auto_clip.py (run :44-81, auto_clip_layer :84-191,
fake_quantize_weight :258-262, apply_clip :194-212), for the configuration on the hot path:
trans_version v2, no GQA, weight-only, clip_version v1, one calibration batch (bs = -1), one rank.

Written with plain torch ops in the order the reference applies them, so that on bf16 tensors
every intermediate is rounded exactly where the reference rounds it.  Device-agnostic: the tests
run it on the CPU and, for arbitration, on the GPU next to the kernels.
"""
import torch

from . import quant_ref as Q


# ---- scale search ---------------------------------------------------------------------------------
def act_scale(x):
    """get_act_scale (awq.py:74-76): mean over all tokens of |x|, in x's dtype."""
    return x.abs().view(-1, x.shape[-1]).mean(0)


def scales_for_ratio(x_mean, ratio):
    """get_scales, trans_version v2 (awq.py:104-107)."""
    s = x_mean.pow(ratio).clamp(min=1e-4).view(-1)
    return s / (s.max() * s.min()).sqrt()


def fake_quant_scaled_weight(w, scales, bit, sym, group_size):
    """scaling_weight + fake_quant_weight_dynamic (awq.py:40-46, :147-164); returns a new tensor."""
    ws = w.clone().mul_(scales.view(1, -1))
    return Q.int_fake_quant_dynamic(ws, bit, sym, 'per_group', group_size)


def loss(org_out, out):
    """calculate_loss, single batch (awq.py:134-136)."""
    return (org_out - out).float().pow(2).mean().item()


@torch.no_grad()
def search_scale(layers, x, inspect, kwargs, bit=4, sym=False, group_size=128, n_grid=20):
    """search_scale_subset for one input batch (awq.py:179-278).  `layers` are the nn.Linear of the
    subset, `inspect` the module whose output is compared, `x` the cached input (B, T, C).
    Returns (best_scales, list of the n_grid losses)."""
    org = [l.weight.data.clone() for l in layers]
    org_out = inspect(x, **kwargs)
    org_out = org_out[0] if isinstance(org_out, tuple) else org_out
    x_mean = act_scale(x)
    best_err, best_scales, losses = float('inf'), None, []
    for n in range(n_grid):
        s = scales_for_ratio(x_mean, n / n_grid)
        for l, w in zip(layers, org):
            l.weight.data = fake_quant_scaled_weight(w, s, bit, sym, group_size)
        out = inspect(x / s.view(1, -1), **kwargs)
        out = out[0] if isinstance(out, tuple) else out
        e = loss(org_out, out)
        losses.append(e)
        for l, w in zip(layers, org):
            l.weight.data = w            # load_state_dict(org_sd)
        if e < best_err:
            best_err, best_scales = e, s
    return best_scales, losses


@torch.no_grad()
def apply_scale_ln_fcs(ln, fcs, scales):
    """scale_ln_fcs (base_blockwise_quantization.py:773-801)."""
    scales = scales.to(ln.weight.dtype)
    ln.weight.div_(scales)
    for fc in fcs:
        fc.weight.mul_(scales.view(1, -1))


@torch.no_grad()
def apply_scale_fc_fc(fc1, fc2, scales):
    """scale_fc_fc, fc1.out_features == fc2.in_features (base_blockwise_quantization.py:684-701, :723)."""
    fc1.weight.div_(scales.view(-1, 1))
    fc2.weight.mul_(scales.view(1, -1))


# ---- clip search ------------------------------------------------------------------------------------
@torch.no_grad()
def auto_clip_layer(w, x, bit=4, sym=False, group_size=128, clip_sym=False, n_grid=20, max_shrink=0.5,
                    n_sample_token=512):
    """auto_clip_layer, clip_version v1, one input tensor (auto_clip.py:84-191).
    w (oc, ic), x (..., ic).  Returns (best_max_val, best_min_val), each (oc, n_groups, 1)."""
    w = w.reshape(w.shape[0], 1, -1, group_size)
    oc_batch = 256 if w.shape[0] % 256 == 0 else 64
    assert w.shape[0] % oc_batch == 0
    x = x.view(-1, x.shape[-1])
    x = x.reshape(1, x.shape[0], -1, group_size)
    step = max(1, x.shape[1] // n_sample_token)
    x = x[:, 0::step]
    best_max_all, best_min_all = [], []
    for b in range(w.shape[0] // oc_batch):
        wb = w[b * oc_batch:(b + 1) * oc_batch]
        org_max = wb.abs().amax(dim=-1, keepdim=True) if clip_sym else wb.amax(dim=-1, keepdim=True)
        org_min = wb.amin(dim=-1, keepdim=True)
        best_max, best_min = org_max.clone(), org_min.clone()
        min_errs = torch.ones_like(org_max) * 1e9
        org_out = (x * wb).sum(dim=-1)
        for i_s in range(int(max_shrink * n_grid)):
            max_val = org_max * (1 - i_s / n_grid)
            min_val = -max_val if clip_sym else org_min * (1 - i_s / n_grid)
            cur_w = torch.clamp(wb, min_val, max_val)
            q_w = Q.int_fake_quant_dynamic(cur_w, bit, sym, 'per_group', group_size)
            cur_out = (x * q_w).sum(dim=-1)
            err = (cur_out - org_out).pow(2).mean(dim=1).view(min_errs.shape)
            err_mean = 0 + err
            err_mean /= 1
            better = err_mean < min_errs
            min_errs[better] = err_mean[better]
            best_max[better] = max_val[better]
            best_min[better] = min_val[better]
        best_max_all.append(best_max)
        best_min_all.append(best_min)
    return torch.cat(best_max_all, dim=0).squeeze(1), torch.cat(best_min_all, dim=0).squeeze(1)


@torch.no_grad()
def apply_clip(weight, min_val, max_val, clip_sym=False):
    """apply_clip v1 (auto_clip.py:194-212): clamp each group to its searched range."""
    shape = weight.shape
    w = weight.reshape(*max_val.shape[:2], -1)
    if clip_sym:
        min_val = -max_val
    return torch.clamp(w, min_val, max_val).reshape(shape)


# ---- one Llama decoder block ------------------------------------------------------------------------
@torch.no_grad()
def awq_block(block, x, kwargs, bit=4, sym=False, group_size=128, clip_sym=None, weight_clip=True,
              n_sample_token=512):
    """Awq.block_transform on a Llama-layout block (awq.py:281-372; subsets llama.py:52-91).
    x: (B, T, C) hidden states (one batch).  Modifies the block in place; returns a dict with the
    per-subset best scales and losses and the per-linear clip ranges."""
    clip_sym = sym if clip_sym is None else clip_sym
    a, m = block.self_attn, block.mlp
    feats = {}
    hooks = []
    for name, mod in (('q', a.q_proj), ('o', a.o_proj), ('gate', m.gate_proj), ('down', m.down_proj)):
        def hook(mod_, inp, out, name=name):
            feats[name] = inp[0].data
        hooks.append(mod.register_forward_hook(hook))
    block(x, **kwargs)
    for h in hooks:
        h.remove()
    report = {'scales': {}, 'losses': {}, 'clip': {}}

    s, ls = search_scale([a.q_proj, a.k_proj, a.v_proj], feats['q'], a, kwargs, bit, sym, group_size)
    apply_scale_ln_fcs(block.input_layernorm, [a.q_proj, a.k_proj, a.v_proj], s)
    feats['q'] = feats['q'] / s.view(1, -1)
    report['scales']['qkv'], report['losses']['qkv'] = s, ls

    s, ls = search_scale([a.o_proj], feats['o'], a.o_proj, {}, bit, sym, group_size)
    apply_scale_fc_fc(a.v_proj, a.o_proj, s)
    feats['o'] = feats['o'] / s.view(1, -1)
    report['scales']['o'], report['losses']['o'] = s, ls

    s, ls = search_scale([m.gate_proj, m.up_proj], feats['gate'], m, {}, bit, sym, group_size)
    apply_scale_ln_fcs(block.post_attention_layernorm, [m.gate_proj, m.up_proj], s)
    feats['gate'] = feats['gate'] / s.view(1, -1)
    report['scales']['gate_up'], report['losses']['gate_up'] = s, ls

    s, ls = search_scale([m.down_proj], feats['down'], m.down_proj, {}, bit, sym, group_size)
    apply_scale_fc_fc(m.up_proj, m.down_proj, s)
    feats['down'] = feats['down'] / s.view(1, -1)
    report['scales']['down'], report['losses']['down'] = s, ls

    if weight_clip:
        # AutoClipper.run skips names containing q_ / k_ (auto_clip.py:56-60)
        for name, mod, f in (('v', a.v_proj, 'q'), ('o', a.o_proj, 'o'), ('gate', m.gate_proj, 'gate'),
                             ('up', m.up_proj, 'gate'), ('down', m.down_proj, 'down')):
            mx, mn = auto_clip_layer(mod.weight.data, feats[f], bit, sym, group_size, clip_sym,
                                     n_sample_token=n_sample_token)
            mod.weight.data = apply_clip(mod.weight.data, mn, mx, clip_sym)
            report['clip'][name] = (mx, mn)
    return report
