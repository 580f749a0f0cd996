"""Oracle restatement of the reference SpQR layer solver (test infrastructure).

Follows llmc/compression/quantization/spqr.py: add_batch :287-316 (the GPTQ Hessian), layer_transform
:117-182, weight_transform :184-285 (with its nested `outliers`), get_group_qparams :325-346,
set_model_qparams :348-356 and the deploy-time w_qdq :367-390; the quantizer arithmetic with
round_zp False is quant.py:544-558 (get_qparams) and :698-711 (quant / dequant).

What the reference's second-level statistics really do is restated as it is: the group's scales and
zeros arrive as (rows, 1) tensors, whose last dimension (1) is below the statistic quantizers' group
size, so reshape_tensor (quant.py:611-641) leaves them alone and every value forms a "group" by itself:
range 0, scale clamp(1e-5) / 7, value reproduced up to the rounding of (v / c) * c.
"""
import math

import torch


def _qparams(t, bit):
    """Asymmetric integer qparams with round_zp False over the last dim (quant.py:134-145, :544-558)."""
    qmin, qmax = torch.tensor(0.0), torch.tensor(2 ** bit - 1)
    mx = t.amax(dim=-1, keepdim=True)
    mn = t.amin(dim=-1, keepdim=True)
    s = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
    z = qmin - (mn / s)
    return s, z, qmax, qmin


def _qdq(t, s, z, qmax, qmin):
    """quant + dequant with round_zp False (quant.py:698-711)."""
    q = torch.clamp(torch.round(t / s.clamp_min(1e-9) + z), qmin.to(t.device), qmax.to(t.device))
    return (q - z) * s


def second_level(v, bit=3):
    """scale_quantizer / zero_quantizer on a (rows, 1) tensor (spqr.py:328-339): get_tensor_qparams then
    fake_quant_weight_static, per_group with a last dimension of 1."""
    s, z, qmax, qmin = _qparams(v, bit)
    return _qdq(v, s, z, qmax, qmin)


def group_qparams(G, bit, stat_bit=3):
    """get_group_qparams (spqr.py:325-346): first-level qparams of the (rows, group) slice, then the
    second-level fake quantisation of both."""
    s, z, qmax, qmin = _qparams(G, bit)
    return second_level(s, stat_bit), second_level(z, stat_bit), qmax, qmin


def outlier_gain(G, hinv_gd, bit):
    """`outliers` nested in weight_transform (spqr.py:185-203): per element of the group, how much the
    group's weighted quantisation error falls when that element is left out."""
    n = G.shape[1]
    idx = torch.arange(n, device=G.device)
    idx = idx[1:] - (idx[:, None] >= idx[1:]).to(idx.dtype)
    loo = G[:, idx]                                             # rows x n x (n - 1)
    flat = loo.flatten(0, 1)
    s, z, qmax, qmin = _qparams(flat, bit)
    loo_rg = _qdq(flat, s, z, qmax, qmin).reshape(loo.shape)
    loo_err = ((loo_rg - loo) / hinv_gd[idx]).square().sum(-1)
    s, z, qmax, qmin = _qparams(G, bit)
    base = ((_qdq(G, s, z, qmax, qmin) - G) / hinv_gd).square().sum(dim=1, keepdim=True)
    return base - loo_err


def prepare(W, H, percdamp=1.0, actorder=True, perm=None):
    """layer_transform up to the factorisation (spqr.py:117-160): sort, permute, damp (before the dead
    columns are set, so a dead column's diagonal is exactly 1), inverse Cholesky factor."""
    W = W.clone().float()
    H = H.clone()
    C = W.shape[1]
    if perm is None:
        perm = torch.argsort(torch.diag(H), descending=True) if actorder else torch.arange(C, device=H.device)
    W = W[:, perm]
    H = H[perm][:, perm]
    invperm = torch.argsort(perm)
    dead = torch.diag(H) == 0
    if percdamp > 0:
        damp = percdamp * abs(torch.diag(H)).mean()
        d = torch.arange(C, device=H.device)
        H[d, d] += damp
    H[dead, dead] = 1
    W[:, dead] = 0
    H = torch.linalg.cholesky(H)
    H = torch.cholesky_inverse(H)
    U = torch.linalg.cholesky(H, upper=True)
    return W, U, perm, invperm


def outlier_threshold(W, U, relative_threshold):
    """spqr.py:205-207; a Python float (double) like the reference's."""
    outlier_scale = (W.var(dim=0) / torch.diag(U).square()).mean().item()
    return relative_threshold * outlier_scale


def weight_transform(W, U, bit=4, group_size=16, blocksize=128, relative_threshold=0.2, simplified=False,
                     threshold=None):
    """spqr.py:184-285.  W (permuted, fp32) is modified in place like the reference.  Returns the kept
    (error-compensated, unquantised) weights, the outlier mask, per-group scales and zeros lists and the
    squared errors."""
    R, C = W.shape
    if threshold is None:
        threshold = outlier_threshold(W, U, relative_threshold)
    tmp = torch.zeros_like(W)
    Losses = torch.zeros_like(W)
    mask = torch.zeros_like(W, dtype=torch.bool)
    g_scales, g_zeros = [], []
    for i1 in range(0, C, blocksize):
        i2 = min(i1 + blocksize, C)
        Err1 = torch.zeros((R, i2 - i1), device=W.device)
        for i in range(i1, i2):
            if i % group_size == 0:
                G = W[:, i:i + group_size]
                if simplified or threshold == math.inf:
                    s, z, qmax, qmin = group_qparams(G, bit)
                else:
                    E = outlier_gain(G, torch.diag(U)[i:i + group_size], bit)
                    M = (E > threshold).float()
                    mean = torch.sum(G * (1 - M), dim=1, keepdim=True) / torch.sum(1 - M, dim=1,
                                                                                   keepdim=True).clamp_min(1)
                    s, z, qmax, qmin = group_qparams(G * (1 - M) + mean * M, bit)
                g_scales.append(s)
                g_zeros.append(z)
            w = W[:, i]
            q = _qdq(w.unsqueeze(1), s, z, qmax, qmin).squeeze(1)
            err = (w - q) / U[i, i]
            if threshold != math.inf:
                mask[:, i] = err.square() > threshold
                M = mask[:, i].float()
                newq = q * (1 - M) + w * M
                err = (w - newq) / U[i, i]
            tmp[:, i] = w
            Losses[:, i] = err.square()
            W[:, i + 1:i2] -= err.unsqueeze(1).matmul(U[i, i + 1:i2].unsqueeze(0))
            Err1[:, i - i1] = err
        W[:, i2:] -= Err1.matmul(U[i1:i2, i2:])
    return tmp, mask, g_scales, g_zeros, Losses


def quantize_layer(W, H, bit=4, group_size=16, blocksize=128, percdamp=1.0, relative_threshold=0.2,
                   simplified=False, actorder=True, perm=None, threshold=None):
    """layer_transform (spqr.py:117-182): the reference's per-layer results — weight (compensated, fp32,
    original column order), buf_scales / buf_zeros ((rows * n_groups, 1), permuted-group order), the
    outlier mask in original column order, perm, invperm."""
    Wp, U, perm, invperm = prepare(W, H, percdamp, actorder, perm)
    if threshold is None:
        threshold = outlier_threshold(Wp, U, relative_threshold)
    tmp, mask, gs, gz, losses = weight_transform(Wp, U, bit, group_size, blocksize, relative_threshold,
                                                 simplified, threshold)
    return dict(weight=tmp[:, invperm], mask=mask[:, invperm],
                buf_scales=torch.stack(gs, dim=1).reshape(-1, 1), buf_zeros=torch.stack(gz, dim=1).reshape(-1, 1),
                buf_perm=perm, buf_invperm=invperm, loss=float(losses.sum()), threshold=threshold, U=U)


def w_qdq(res, model_dtype, bit=4, group_size=16):
    """Deploy-time weight (spqr.py:367-390): outliers keep their compensated value, the rest is the static
    fake quantisation with the group's second-level-quantised statistics."""
    weight = res['weight']
    maskf = res['mask'].float()
    out = (maskf * weight).to(model_dtype)
    wp = weight[:, res['buf_perm']]
    qmin, qmax = torch.tensor(0.0), torch.tensor(2 ** bit - 1)
    g = wp.reshape(-1, group_size)
    fq = _qdq(g, res['buf_scales'], res['buf_zeros'], qmax, qmin).reshape(wp.shape).to(wp.dtype).to(model_dtype)
    fq = fq[:, res['buf_invperm']]
    return (fq * (1 - maskf) + out).to(model_dtype)
