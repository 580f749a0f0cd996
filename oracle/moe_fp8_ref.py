"""Oracle restatement of the FP8 fake-quantised MoE layer (test infrastructure): every expert
linear as an EffcientFakeQuantLinear (llmc/compression/quantization/module_utils.py:774-852) with
FloatQuantizer e4m3 per_channel weights and per_token dynamic inputs (quant.py:1099-1158), evaluated
expert by expert with plain torch.  PARITY UNPINNED for the e4m3 rounding call (see quant_ref)."""
import torch
import torch.nn.functional as F

from . import quant_ref as Q


def fake_quant_linear(x, w):
    """EffcientFakeQuantLinear.forward (module_utils.py:799-813): a_qdq(x) then F.linear with w_qdq(w)."""
    return F.linear(Q.fp8_fake_quant_dynamic(x), Q.fp8_fake_quant_dynamic(w))


@torch.no_grad()
def moe_forward(x, gate, w_gate, w_up, w_down, s_gate, s_up, s_down, top_k):
    scores = torch.softmax((x @ gate.t()).float(), dim=-1)
    w, idx = torch.topk(scores, top_k, dim=-1)
    w = w.to(x.dtype)
    out = torch.zeros_like(x, dtype=torch.float32)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // top_k
    e_sorted = flat_e[order]
    wsel = w.reshape(-1)[order]
    for e in range(gate.shape[0]):
        m = e_sorted == e
        if not bool(m.any()):
            continue
        xe = x[tok[m]]
        h = F.silu(fake_quant_linear(xe, w_gate[e])) * fake_quant_linear(xe, w_up[e])
        y = fake_quant_linear(h, w_down[e])
        out.index_add_(0, tok[m], (y * wsel[m].unsqueeze(1)).float())
    hs = F.silu(fake_quant_linear(x, s_gate)) * fake_quant_linear(x, s_up)
    out += fake_quant_linear(hs, s_down).float()
    return out.to(x.dtype)
