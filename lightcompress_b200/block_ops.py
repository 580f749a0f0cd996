"""Fused element-wise pieces of the calibration block forward.

The reference's block_forward (llmc/compression/quantization/base_blockwise_quantization.py:378-401)
runs the decoder block's stock module code.  Three chains of small tensor ops in that code -- the
RMS norms, the rotary embedding of q and k and the gated activation of the MLP -- cost more HBM
passes than all quantisation kernels together, so the staged Llama schedule swaps them for one
kernel each.  The kernels round after every op of the chain they replace (the RMS norm also
associates its sum of squares like torch's row reduction); before a swap is used it is compared
bit for bit with the stock code on random data, and the stock code is kept if they differ (another
rotary convention, activation or norm, or a torch build that reduces in another order).
"""
import contextlib
import sys

import numpy as np
import torch

from . import _lib as L

_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
_checked = {}


def rejected():
    """The self-checks that failed so far, i.e. the module kinds for which the stock tensor ops were kept
    because the fused kernel did not reproduce them bit for bit: [(kind, detail), ...].  Empty on the
    Llama block this library is built for; a benchmark or a caller that expects the fused path reads this
    instead of guessing."""
    return [(k[0], str(k[1])) for k, ok in _checked.items() if not ok]


def rope_apply_one(x, cos, sin):
    """x: (B, H, T, D) view of a (B, T, H, D) contiguous tensor; cos, sin: (B, T, D) or (1, T, D)
    contiguous.  Returns the embedded tensor with x's shape and memory layout."""
    B, H, T, D = x.shape
    mem = x.transpose(1, 2)
    out = torch.empty_like(mem)
    L.call('lc_rope_apply', L.ptr(mem), L.ptr(cos), L.ptr(sin), L.lc_dtype(x), B * T, H, D, cos.shape[0] * T,
           L.ptr(out), L.stream_of(x))
    return out.transpose(1, 2)


def _rope_fits(q, k, cos, sin, unsqueeze_dim):
    if unsqueeze_dim != 1 or not q.is_cuda or q.dtype not in _DTYPES or q.dim() != 4 or k.dim() != 4:
        return False
    if not (k.dtype == cos.dtype == sin.dtype == q.dtype):
        return False
    B, _, T, D = q.shape
    if cos.shape not in ((B, T, D), (1, T, D)) or sin.shape != cos.shape or k.shape[0] != B \
            or k.shape[2:] != (T, D):
        return False
    if D % (8 if q.dtype == torch.float32 else 16):
        return False
    return (q.transpose(1, 2).is_contiguous() and k.transpose(1, 2).is_contiguous() and cos.is_contiguous()
            and sin.is_contiguous() and all(t.data_ptr() % 16 == 0 for t in (q, k, cos, sin)))


def _make_rope(orig):
    def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1, **kw):
        if kw or not _rope_fits(q, k, cos, sin, unsqueeze_dim):
            return orig(q, k, cos, sin, unsqueeze_dim=unsqueeze_dim, **kw)
        return rope_apply_one(q, cos, sin), rope_apply_one(k, cos, sin)
    return apply_rotary_pos_emb


def _rope_matches(orig, device, dtype):
    """True if `orig` is the rotate-half convention the kernel implements (checked on random data)."""
    key = ('rope', id(orig), str(device), dtype)
    if key not in _checked:
        g = torch.Generator().manual_seed(7)
        q = torch.randn(2, 5, 3, 32, generator=g).to(dtype).to(device).transpose(1, 2)
        k = torch.randn(2, 5, 1, 32, generator=g).to(dtype).to(device).transpose(1, 2)
        cos = torch.randn(2, 5, 32, generator=g).to(dtype).to(device)
        sin = torch.randn(2, 5, 32, generator=g).to(dtype).to(device)
        try:
            rq, rk = orig(q, k, cos, sin)
            ok = torch.equal(rq, rope_apply_one(q, cos, sin)) and torch.equal(rk, rope_apply_one(k, cos, sin))
        except (TypeError, RuntimeError, ValueError):
            ok = False
        _checked[key] = ok
    return _checked[key]


@contextlib.contextmanager
def fused_rotary(attn_module, device, dtype):
    """While active, the Python module that defines `attn_module`'s class applies the rotary
    embedding through lc_rope_apply.  Yields whether the swap took place."""
    mod = sys.modules.get(type(attn_module).__module__)
    orig = getattr(mod, 'apply_rotary_pos_emb', None)
    if orig is None or dtype not in _DTYPES or not _rope_matches(orig, device, dtype):
        yield False
        return
    mod.apply_rotary_pos_emb = _make_rope(orig)
    try:
        yield True
    finally:
        mod.apply_rotary_pos_emb = orig


def silu_mul(gate, up):
    out = torch.empty_like(gate)
    L.call('lc_silu_mul', L.ptr(gate), L.ptr(up), L.lc_dtype(gate), gate.numel(), L.ptr(out), L.stream_of(gate))
    return out


def gated_act(act_fn, gate, up):
    """act_fn(gate) * up; through lc_silu_mul when act_fn is SiLU (verified once per activation type,
    device and dtype on random data) and the tensors fit the kernel, else with the stock ops."""
    fits = (gate.is_cuda and gate.dtype in _DTYPES and up.dtype == gate.dtype and gate.shape == up.shape
            and gate.is_contiguous() and up.is_contiguous() and gate.numel() % 8 == 0
            and gate.data_ptr() % 16 == 0 and up.data_ptr() % 16 == 0)
    if fits:
        key = ('act', type(act_fn), str(gate.device), gate.dtype)
        if key not in _checked:
            g = torch.Generator().manual_seed(11)
            a = (torch.randn(4096, generator=g) * 4).to(gate.dtype).to(gate.device)
            b = torch.randn(4096, generator=g).to(gate.dtype).to(gate.device)
            _checked[key] = torch.equal(act_fn(a) * b, silu_mul(a, b))
        if _checked[key]:
            return silu_mul(gate, up)
    return act_fn(gate) * up


def _rms_raw(x, weight, eps):
    x2 = x.reshape(-1, x.shape[-1])
    rows, C = x2.shape
    out = torch.empty_like(x2)
    # 1/C the way the mean it replaces forms it: fp32 rows / fp32 (rows * C)
    factor = float(np.float32(rows) / np.float32(rows * C))
    L.call('lc_rmsnorm', L.ptr(x2), L.ptr(weight), L.lc_dtype(x2), rows, C, factor, float(eps), L.ptr(out),
           L.stream_of(x2))
    return out.view(x.shape)


def rms_norm(module, x):
    """module(x) for a Llama-style RMS norm (weight, variance_epsilon) through lc_rmsnorm when the
    kernel reproduces the module bit for bit (checked once per module type, width, dtype and device
    on random rows that include the row count of `x`), else the module itself."""
    w = getattr(module, 'weight', None)
    eps = getattr(module, 'variance_epsilon', None)
    C = x.shape[-1]
    fits = (w is not None and eps is not None and x.is_cuda and x.dtype in _DTYPES and w.dtype == x.dtype
            and w.dim() == 1 and w.shape[0] == C and C % 128 == 0 and 128 <= C < 8192 and x.is_contiguous()
            and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.numel() > 0)
    if not fits:
        return module(x)
    rows = x.numel() // C
    key = ('rms', type(module), C, rows, float(eps), str(x.device), x.dtype)
    if key not in _checked:
        g = torch.Generator().manual_seed(13)
        t = torch.randn(rows, C, generator=g)
        t[: rows // 2] *= torch.rand(rows // 2, 1, generator=g) * 30     # a spread of row norms
        wt = torch.randn(C, generator=g) * 0.5 + 1
        saved = module.weight.data
        ok = True
        try:
            # in fp32 nothing hides a differently associated sum; then the dtype actually used
            for dt in (torch.float32, x.dtype):
                module.weight.data = wt.to(dt).to(x.device)
                td = t.to(dt).to(x.device).view(x.shape)
                ok = ok and torch.equal(module(td), _rms_raw(td, module.weight.data, eps))
        finally:
            module.weight.data = saved
        _checked[key] = ok
    if _checked[key]:
        return _rms_raw(x, w.data, eps)
    return module(x)


@contextlib.contextmanager
def fused_gated_mlp(mlp):
    """While active, `type(mlp).forward` is down_proj(act_fn(gate_proj(x)) * up_proj(x)) with the
    activation and the product in one kernel (gated_act).  Only swapped in if the class's own forward
    gives the same bits on random data for this module's layout; yields whether it was."""
    cls = type(mlp)
    need = all(hasattr(mlp, a) for a in ('gate_proj', 'up_proj', 'down_proj', 'act_fn'))
    w = getattr(getattr(mlp, 'gate_proj', None), 'weight', None)
    if not need or w is None or not w.is_cuda or w.dtype not in _DTYPES:
        yield False
        return
    orig = cls.forward

    def forward(self, x):
        return self.down_proj(gated_act(self.act_fn, self.gate_proj(x), self.up_proj(x)))
    key = ('mlp', cls, str(w.device), w.dtype)
    if key not in _checked:
        g = torch.Generator().manual_seed(17)
        t = torch.randn(2, 24, w.shape[1], generator=g).to(w.dtype).to(w.device)
        with torch.no_grad():
            _checked[key] = torch.equal(orig(mlp, t), forward(mlp, t))
    if not _checked[key]:
        yield False
        return
    cls.forward = forward
    try:
        yield True
    finally:
        cls.forward = orig
