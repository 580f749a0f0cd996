"""Oracle restatement of the reference GPTQ layer solver (test infrastructure).

Follows llmc/compression/quantization/gptq.py: add_batch :254-295, hessian_sorting
:58-64, process_hessian_and_weights :128-176, weight_transform :199-244,
search_column_qparams :359-366, merge/update qparams :344-356, :398-409 and the
deploy-time w_qdq :425-452.  Only the configuration the hot path covers is restated:
nn.Linear, per_group with group_size == blocksize, static_groups off or on (:224-227, :377-393),
per_channel (:368-375); owq (:44-50, :66-83, :186-188,
:440-447) with fewer outlier columns than a group.
"""
import math
import torch
from . import quant_ref as Q


def hessian_init(columns, device='cpu'):
    """layer_init (gptq.py:298-308)."""
    return {'H': torch.zeros(columns, columns, device=device), 'nsamples': 0}


def add_batch(state, inp):
    """gptq.py:254-295 at world size 1: inp is (b, T, C) or (T, C) in the model dtype."""
    if inp.dim() == 2:
        inp = inp.unsqueeze(0)
    b = inp.shape[0]
    x = inp.reshape(-1, inp.shape[-1]).t()
    state['H'] *= state['nsamples'] / (state['nsamples'] + b)
    state['nsamples'] += b
    x = math.sqrt(2 / state['nsamples']) * x.float()
    state['H'] += x.matmul(x.t())
    return state


def owq_perm(H, n_out):
    """hessian_sorting with owq (gptq.py:66-83; owq switches actorder off, gptq.py:47-50): the n_out
    columns with the largest Hessian diagonal go last, in descending order of it; the others keep
    their order."""
    C = H.shape[0]
    descending_ids = torch.argsort(torch.diag(H), descending=True)
    keep = torch.full([C], True)
    keep[descending_ids[:n_out]] = False
    return torch.cat([torch.arange(C)[keep], descending_ids[:n_out]])


def prepare(W, H, percdamp=0.01, actorder=True, n_out=0, perm=None):
    """hessian_sorting + process_hessian_and_weights (gptq.py:58-83, :128-176).
    Returns permuted fp32 W, upper Cholesky factor U of the damped inverse Hessian, perm, invperm.
    perm: a column order to use instead of the one sorted from diag(H) (an extension for comparisons
    that must not depend on how near-equal diagonal entries happen to sort)."""
    W = W.clone().float()
    H = H.clone()
    C = W.shape[1]
    if perm is not None:
        perm = perm.to(H.device)
    elif n_out:
        perm = owq_perm(H, n_out)
    else:
        perm = torch.argsort(torch.diag(H), descending=True) if actorder else torch.arange(C, device=H.device)
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    W = W[:, perm]
    H = H[perm][:, perm]
    invperm = torch.argsort(perm)
    damp = percdamp * torch.mean(torch.diag(H))
    idx = torch.arange(C, device=H.device)
    H[idx, idx] += damp
    L = torch.linalg.cholesky(H)
    Hinv = torch.cholesky_inverse(L)
    U = torch.linalg.cholesky(Hinv, upper=True)
    return W, U, perm, invperm


def static_group_qparams(W, bit=4, sym=False, group_size=128):
    """The round-to-nearest qparams collect_block_qparams leaves on a layer
    (base_blockwise_quantization.py:349-376), in the weight's dtype: buf_scales / buf_zeros,
    (R * n_groups, 1), which search_group_qparams (gptq.py:377-393) splits per group."""
    g = W if group_size is None else Q.group_view(W, 'per_group', group_size)     # None: per_channel
    s, z, qmax, qmin = Q.int_qparams(g, bit, sym)
    return s, z


def weight_transform(W, U, bit=4, sym=False, group_size=128, blocksize=128, n_out=0, static=None, perm=None):
    """gptq.py:199-244.  W is modified in place like the reference; returns
    (kept weights `tmp`, Losses, per-group scales list, per-group zeros list).  With owq the last
    n_out columns are not quantised (they only receive the error feedback) and `tmp` is zero there."""
    assert group_size == blocksize or static is not None
    R, C = W.shape
    n_nonout = C - n_out
    tmp = torch.zeros_like(W)
    Losses = torch.zeros_like(W)
    g_scales, g_zeros = [], []
    if static is not None:
        # static groups (gptq.py:224-227): column i of the permuted weight uses the group of its original column
        n_g = C // group_size
        st_s = static[0].reshape(R, n_g)
        st_z = None if sym else static[1].reshape(R, n_g)
        qmin, qmax = Q.int_range(bit, sym)
    for i1 in range(0, n_nonout, blocksize):
        i2 = min(i1 + blocksize, n_nonout)
        W1 = W[:, i1:i2].clone()
        U1 = U[i1:i2, i1:i2]
        Err1 = torch.zeros_like(W1)
        for i in range(i2 - i1):
            w = W1[:, i].clone()
            d = U1[i, i]
            if static is not None:
                idx = i1 + i if perm is None else int(perm[i1 + i])
                gi = idx // group_size
                s = st_s[:, gi:gi + 1]
                z = torch.tensor(0.0) if sym else st_z[:, gi:gi + 1]
            elif (i1 + i) % group_size == 0:
                cols = W[:, i1 + i: min(i1 + i + group_size, n_nonout)]
                s, z, qmax, qmin = Q.int_qparams(cols, bit, sym)
                g_scales.append(s)
                g_zeros.append(z)
            q = Q.int_dequant(Q.int_quant(w.unsqueeze(1), s, z, qmax, qmin), s, z).squeeze(1)
            tmp[:, i1 + i] = w
            Losses[:, i1 + i] = (w - q) ** 2 / (2 * d ** 2)
            err = (w - q) / d
            W1[:, i:] -= err.unsqueeze(1).matmul(U1[i, i:].unsqueeze(0))
            Err1[:, i] = err
        W[:, i2:] -= Err1.matmul(U[i1:i2, i2:])
    return tmp, Losses, g_scales, g_zeros


def merge_group_qparams(per_group):
    """merge_qparams for per_group (gptq.py:353-355): list of (R,1) -> (R*n_g, 1)."""
    return torch.stack(per_group, dim=1).reshape(-1, 1)


def quantize_layer(W, H, bit=4, sym=False, group_size=128, blocksize=128,
                   percdamp=0.01, actorder=True, n_out=0, static_groups=False, granularity='per_group', perm=None):
    """layer_transform (gptq.py:114-117, :178-196): returns a dict with the reference's
    per-layer results: weight (compensated, fp32, original column order), buf_scales,
    buf_zeros (permuted-group order), buf_perm, buf_invperm, loss.  n_out > 0 is the owq mode
    (0 < n_out < group_size with C a multiple of group_size, so that the group count stays C / group_size:
    the reference's w_qdq only works then): the outlier columns keep their error-compensated fp32 values
    (gptq.py:186-188)."""
    Wp, U, perm, invperm = prepare(W, H, percdamp, actorder and not n_out, n_out, perm)
    if granularity == 'per_channel':
        # search_layer_qparams (gptq.py:368-375): the layer's per-channel round-to-nearest qparams for every
        # column -- static groups with one group spanning the row
        static_groups, group_size = True, W.shape[1]
        static = static_group_qparams(W, bit, sym, None)
    else:
        static = static_group_qparams(W, bit, sym, group_size) if static_groups else None
    tmp, Losses, gs, gz = weight_transform(Wp, U, bit, sym, group_size, blocksize, n_out, static,
                                           perm if (static_groups and actorder) else None)
    if n_out:
        tmp[:, W.shape[1] - n_out:] = Wp[:, W.shape[1] - n_out:]
    if static_groups:
        # the layer keeps its round-to-nearest buffers (gptq.py:195-196) and deploys without a permutation
        out = {'weight': tmp[:, invperm].contiguous(), 'buf_scales': static[0],
               'buf_zeros': None if sym else static[1], 'buf_perm': torch.arange(W.shape[1]),
               'buf_invperm': torch.arange(W.shape[1]), 'solver_perm': perm, 'loss': float(Losses.sum()), 'U': U,
               'n_nonout': W.shape[1]}
        return out
    out = {
        'weight': tmp[:, invperm].contiguous(),
        'buf_scales': merge_group_qparams(gs),
        'buf_perm': perm, 'buf_invperm': invperm,
        'loss': float(Losses.sum()),
        'U': U, 'n_nonout': W.shape[1] - n_out,
    }
    out['buf_zeros'] = None if sym else merge_group_qparams(gz)
    return out


def codes_permuted(res, bit=4, sym=False, group_size=128):
    """Int codes as the reference defines them on the fake-quant path (gptq.py:425-452 with
    quant.py:698-700): quant(weight[:, perm] grouped, buf_scales, buf_zeros).  (R, C), permuted order."""
    qmin, qmax = Q.int_range(bit, sym)
    w = res['weight'][:, res['buf_perm']]
    z = torch.tensor(0.0) if sym else res['buf_zeros']
    g = w.reshape(-1, group_size)
    return Q.int_quant(g, res['buf_scales'], z, qmax, qmin).reshape(w.shape)


def w_qdq(res, model_dtype, bit=4, sym=False, group_size=128):
    """Deploy-time fake quant (gptq.py:425-452): permute, static qdq, un-permute, model dtype."""
    w = res['weight'][:, res['buf_perm']]
    z = torch.tensor(0.0) if sym else res['buf_zeros']
    out = Q.int_fake_quant_static(w, res['buf_scales'], z, bit, sym, 'per_group', group_size).to(model_dtype)
    n_nonout = res.get('n_nonout', w.shape[1])
    if n_nonout < w.shape[1]:
        out[:, n_nonout:] = w[:, n_nonout:].to(model_dtype)     # owq: the outlier columns stay unquantised
    return out[:, res['buf_invperm']]


def recon_error(W, Wq, X):
    """||W X - Wq X|| / ||W X|| over calibration rows X (T, C), fp64 accumulate."""
    Xd = X.double()
    ref = Xd @ W.double().t()
    return float((Xd @ (W.double() - Wq.double()).t()).norm() / ref.norm())
