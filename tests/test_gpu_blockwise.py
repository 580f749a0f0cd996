"""GPU parity of the per-block GPTQ schedule (GPTQBlockwise) against the oracle's literal
restatement of the reference schedule, on a small Llama decoder block built from the installed
transformers (random-init weights, synthetic hidden states).

The oracle is plain torch, so it runs on the same GPU as the kernels here: both sides then see
bit-identical bf16 forwards (same cuBLAS / SDPA kernels) and every subset must meet the strict
bar, fewer than 0.1 % differing codes, plus a reconstruction error within 1 % of the oracle's.
A second run with the oracle on the CPU reports how far cross-device forward noise alone moves
the later subsets (informative; only the reconstruction bar is asserted there)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make_block(hidden=256, inter=512, heads=4, T=96, n_seq=16, seed=0):
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=1, vocab_size=128, max_position_embeddings=4 * T)
    cfg._attn_implementation = 'sdpa'
    torch.manual_seed(seed)
    block = LlamaDecoderLayer(cfg, 0).to(torch.bfloat16)
    g = torch.Generator().manual_seed(seed + 1)
    for p in block.parameters():
        if p.dim() == 2:
            p.data = (torch.randn(p.shape, generator=g) * 0.02).to(torch.bfloat16)
    rot = LlamaRotaryEmbedding(cfg)
    pos = torch.arange(T)[None]
    cos, sin = rot(torch.zeros(1, T, hidden, dtype=torch.bfloat16), pos)
    kwargs = dict(position_embeddings=(cos, sin), attention_mask=None, position_ids=pos)
    xs = []
    ch = torch.randperm(hidden, generator=g)[:max(1, hidden // 100)]
    for _ in range(n_seq):
        x = torch.randn(1, T, hidden, generator=g)
        x[:, :, ch] *= 20
        xs.append(x.to(torch.bfloat16))
    return block, xs, kwargs


def _to_cuda(kwargs):
    out = {}
    for k, v in kwargs.items():
        if torch.is_tensor(v):
            out[k] = v.cuda()
        elif isinstance(v, tuple):
            out[k] = tuple(t.cuda() for t in v)
        else:
            out[k] = v
    return out


@pytest.mark.parametrize('true_sequential,oracle_device', [(True, 'cuda'), (False, 'cuda'), (True, 'cpu')])
def test_block_schedule_matches_oracle(true_sequential, oracle_device):
    from lightcompress_b200 import FakeQuantLinear, GPTQBlockwise, IntegerQuantizer, llama_subsets
    from oracle import gptq_block_ref, gptq_ref
    block, xs, kwargs = _make_block()
    ref_block = copy.deepcopy(block)
    if oracle_device == 'cuda':
        ref_res, ref_out = gptq_block_ref.gptq_block(ref_block.cuda(), [x.cuda() for x in xs], _to_cuda(kwargs),
                                                     true_sequential=true_sequential)
        ref_res = {n: {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in r.items()} for n, r in ref_res.items()}
        ref_out = [o.cpu() for o in ref_out]
    else:
        ref_res, ref_out = gptq_block_ref.gptq_block(ref_block, xs, kwargs, true_sequential=true_sequential)

    gblock = copy.deepcopy(block).cuda()
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    runner = GPTQBlockwise(wq, {'actorder': True, 'percdamp': 0.01, 'blocksize': 128,
                                'true_sequential': true_sequential, 'hessian_batch': 4, 'stage_plan': False})
    outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
    torch.cuda.synchronize()
    assert runner.forward_passes == (5 if true_sequential else 2)

    for si, subset in enumerate(llama_subsets(gblock)):
        for name, (parent, attr) in subset.items():
            mod = getattr(parent, attr)
            assert isinstance(mod, FakeQuantLinear) and mod.weight.dtype == torch.float32
            r = ref_res[name]
            R, C = r['weight'].shape
            got = {'weight': mod.weight.cpu(), 'buf_scales': mod.buf_scales.cpu(), 'buf_zeros': mod.buf_zeros.cpu(),
                   'buf_perm': mod.buf_perm.cpu(), 'buf_invperm': mod.buf_invperm.cpu()}
            a = torch.empty(R, C)
            b = torch.empty(R, C)
            a[:, got['buf_perm']] = gptq_ref.codes_permuted(got)
            b[:, r['buf_perm']] = gptq_ref.codes_permuted(r)
            mism = float((a != b).float().mean())
            wq_gpu = mod.tmp_weight.cpu().float()
            assert torch.equal(wq_gpu, gptq_ref.w_qdq(got, torch.bfloat16).float())   # deploy path == oracle formula
            W0 = dict(block.named_modules())[name].weight.data.float()
            X = torch.randn(512, C, generator=torch.Generator().manual_seed(si))
            e_ref = gptq_ref.recon_error(W0, r['w_qdq'].float(), X)
            e_gpu = gptq_ref.recon_error(W0, wq_gpu, X)
            print(f'{name}: code mismatch {mism:.4%}  recon(ref) {e_ref:.5f} recon(gpu) {e_gpu:.5f}')
            if si == 0 or oracle_device == 'cuda':
                assert mism < 1e-3, (name, mism)
            assert abs(e_gpu - e_ref) <= 0.01 * e_ref, (name, e_gpu, e_ref)
    o_ref = torch.cat(ref_out).float()
    o_gpu = torch.cat([o.cpu() for o in outs]).float()
    rel = float((o_gpu - o_ref).norm() / o_ref.norm())
    print(f'block output rel diff {rel:.4e}')
    assert rel < 0.05


def test_staged_plan_is_bit_identical_to_reforwarding():
    """The Llama stage plan (every module evaluated once) against the generic re-forwarding
    schedule, with and without early exit: same weights, parameters, permutation and outputs,
    bit for bit."""
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets
    block, xs, kwargs = _make_block(seed=3)
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    results = []
    for special in ({'stage_plan': True}, {'stage_plan': False, 'early_exit': True},
                    {'stage_plan': False, 'early_exit': False}):
        gblock = copy.deepcopy(block).cuda()
        # hessian_ksplit=1: a deterministic Hessian (no atomically combined token splits), so that
        # the three runs can be compared bit for bit
        runner = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'hessian_batch': 8,
                                         'hessian_ksplit': 1}, **special))
        outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
        torch.cuda.synchronize()
        state = {}
        for subset in llama_subsets(gblock):
            for name, (parent, attr) in subset.items():
                mod = getattr(parent, attr)
                state[name] = (mod.weight.clone(), mod.buf_scales.clone(), mod.buf_zeros.clone(), mod.buf_perm.clone())
        results.append((state, torch.cat(outs), runner.forward_passes))
    assert [r[2] for r in results] == [1, 5, 5]
    for state, out, _ in results[1:]:
        assert torch.equal(out, results[0][1])
        for name in state:
            for a, b in zip(state[name], results[0][0][name]):
                assert torch.equal(a, b), name


@pytest.mark.parametrize('mode', ['static_groups', 'owq'])
def test_block_schedule_with_static_groups_and_owq(mode):
    """The two other modes of the solver through the block schedule: staged plan and generic
    re-forwarding agree bit for bit; static groups keep every linear's round-to-nearest buffers, owq
    leaves the outlier columns unquantised in the deployed weight."""
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets
    block, xs, kwargs = _make_block(seed=5)
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    extra = {'static_groups': True} if mode == 'static_groups' else {'owq': True, 'n_outs': [6, 6, 6, 6, 2, 2, 6]}
    results = []
    for plan in (True, False):
        gblock = copy.deepcopy(block).cuda()
        runner = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'hessian_batch': 8, 'hessian_ksplit': 1,
                                         'stage_plan': plan}, **extra))
        outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
        runner.solver.check_status()
        torch.cuda.synchronize()
        results.append((gblock, torch.cat(outs)))
    assert torch.equal(results[0][1], results[1][1])
    gblock = results[0][0]
    orig = dict(block.named_modules())
    for subset in llama_subsets(gblock):
        for name, (parent, attr) in subset.items():
            m = getattr(parent, attr)
            other = dict(results[1][0].named_modules())[name]
            assert torch.equal(m.weight, other.weight) and torch.equal(m.tmp_weight, other.tmp_weight), name
            if mode == 'static_groups':
                _, s, z, _, _ = wq.get_tensor_qparams(orig[name].weight.data.cuda())
                assert torch.equal(m.buf_scales, s) and torch.equal(m.buf_zeros, z), name
                assert m.buf_scales.dtype == torch.bfloat16
            else:
                n_nonout = int(m.buf_n_nonout)
                assert n_nonout == m.weight.shape[1] - (2 if 'gate' in name or 'up' in name else 6), name
                outl = m.buf_perm[n_nonout:]
                assert torch.equal(m.tmp_weight[:, outl], m.weight[:, outl].to(m.tmp_weight.dtype)), name


def _other_family_block(kind, hidden=256, inter=512, heads=4, T=96, n_seq=16, seed=5):
    """A decoder layer of another model family that has Llama's attribute names: Qwen2 (biases on q / k / v,
    the same data flow) or Granite (residual and attention multipliers: another data flow)."""
    if kind == 'qwen2':
        from transformers.models.qwen2.modeling_qwen2 import Qwen2Config as Cfg, Qwen2DecoderLayer as Layer
        from transformers.models.qwen2.modeling_qwen2 import Qwen2RotaryEmbedding as Rot
        extra = {}
    else:
        from transformers.models.granite.modeling_granite import GraniteConfig as Cfg, GraniteDecoderLayer as Layer
        from transformers.models.granite.modeling_granite import GraniteRotaryEmbedding as Rot
        extra = dict(residual_multiplier=0.5, attention_multiplier=0.1)
    cfg = Cfg(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads, num_key_value_heads=heads,
              num_hidden_layers=1, vocab_size=128, max_position_embeddings=4 * T, **extra)
    cfg._attn_implementation = 'sdpa'
    torch.manual_seed(seed)
    block = Layer(cfg, 0).to(torch.bfloat16)
    g = torch.Generator().manual_seed(seed + 1)
    for p in block.parameters():
        p.data = (torch.randn(p.shape, generator=g) * (0.02 if p.dim() == 2 else 0.1)).to(torch.bfloat16) + (
            0 if p.dim() == 2 or p.shape[0] != hidden else 1)
    rot = Rot(cfg)
    pos = torch.arange(T)[None]
    cos, sin = rot(torch.zeros(1, T, hidden, dtype=torch.bfloat16), pos)
    kwargs = dict(position_embeddings=(cos, sin), attention_mask=None, position_ids=pos)
    xs = [torch.randn(1, T, hidden, generator=g).to(torch.bfloat16) for _ in range(n_seq)]
    return block, xs, kwargs


@pytest.mark.parametrize('kind', ['qwen2', 'granite'])
def test_stage_plan_is_only_taken_where_it_reproduces_the_block(kind):
    """The staged plan is chosen by attribute names and then checked against the block's own forward.
    Qwen2's layer (biases) computes what the plan computes: it is taken, one forward.  Granite's layer
    scales the residual branches: the check refuses the plan for that class and the generic re-forwarding
    schedule runs.  Either way the result equals the generic schedule's bit for bit."""
    from lightcompress_b200 import GPTQBlockwise, IntegerQuantizer, llama_subsets
    block, xs, kwargs = _other_family_block(kind)
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    results = []
    for special in ({'stage_plan': True}, {'stage_plan': False}):
        gblock = copy.deepcopy(block).cuda()
        runner = GPTQBlockwise(wq, dict({'actorder': True, 'percdamp': 0.01, 'hessian_ksplit': 1}, **special))
        outs = runner.block_opt(gblock, [x.cuda() for x in xs], _to_cuda(kwargs))
        torch.cuda.synchronize()
        state = {name: (getattr(parent, attr).weight.clone(), getattr(parent, attr).buf_scales.clone(),
                        getattr(parent, attr).buf_perm.clone())
                 for subset in llama_subsets(gblock) for name, (parent, attr) in subset.items()}
        results.append((state, torch.cat(outs), runner.forward_passes, list(runner.stage_plan_rejected)))
    staged, generic = results
    if kind == 'qwen2':
        assert staged[2] == 1 and not staged[3]
    else:
        assert staged[2] == 5 and staged[3] == ['GraniteDecoderLayer']
    assert torch.equal(staged[1], generic[1])
    for name in staged[0]:
        for a, b in zip(staged[0][name], generic[0][name]):
            assert torch.equal(a, b), name
    # and the output is the quantised block's own forward
    with torch.no_grad():
        ys = [gblock(x.cuda(), **_to_cuda(kwargs)) for x in xs]
    want = torch.cat([y[0] if isinstance(y, tuple) else y for y in ys])
    assert torch.equal(want, generic[1])


def test_generic_schedule_on_a_block_of_another_layout():
    """A decoder layer without Llama's attribute names (OPT: q / k / v, out_proj, fc1, fc2 with biases and
    LayerNorms; subsets of llmc/models/opt.py:53-90) goes through the generic hook-and-re-forward schedule
    with the adapter's subsets, against the oracle schedule on the same GPU."""
    from collections import OrderedDict
    from transformers.models.opt.modeling_opt import OPTConfig, OPTDecoderLayer
    from lightcompress_b200 import FakeQuantLinear, GPTQBlockwise, IntegerQuantizer
    from oracle import gptq_block_ref, gptq_ref
    hidden, ffn, T, n_seq = 256, 512, 96, 16
    cfg = OPTConfig(hidden_size=hidden, ffn_dim=ffn, num_attention_heads=4, num_hidden_layers=1, vocab_size=128,
                    max_position_embeddings=4 * T, word_embed_proj_dim=hidden, dropout=0.0, attention_dropout=0.0)
    cfg._attn_implementation = 'sdpa'
    torch.manual_seed(21)
    block = OPTDecoderLayer(cfg, layer_idx=0).to(torch.bfloat16).eval()
    g = torch.Generator().manual_seed(22)
    for p in block.parameters():
        if p.dim() == 2:
            p.data = (torch.randn(p.shape, generator=g) * 0.02).to(torch.bfloat16)
    xs = [torch.randn(1, T, hidden, generator=g).to(torch.bfloat16) for _ in range(n_seq)]
    kwargs = {}

    def names(b):
        a = b.self_attn
        return [[('self_attn.q_proj', a, 'q_proj'), ('self_attn.k_proj', a, 'k_proj'), ('self_attn.v_proj', a, 'v_proj')],
                [('self_attn.out_proj', a, 'out_proj')], [('fc1', b, 'fc1')], [('fc2', b, 'fc2')]]

    ref_block = copy.deepcopy(block).cuda()
    ref_res, ref_out = gptq_block_ref.gptq_block(ref_block, [x.cuda() for x in xs], kwargs, subsets=names(ref_block))
    gblock = copy.deepcopy(block).cuda()
    assert not hasattr(gblock, 'mlp')
    pairs = [OrderedDict((n, (parent, attr)) for n, parent, attr in sub) for sub in names(gblock)]
    wq = IntegerQuantizer(4, False, 'per_group', group_size=128)
    # every subset's column order pinned to the oracle's: the LayerNorm outputs feeding fc1 have near-equal
    # Hessian diagonals, whose argsort order is decided by the last bits of the sums
    pins = {sub[0][0]: ref_res[sub[0][0]]['buf_perm'] for sub in names(gblock)}
    runner = GPTQBlockwise(wq, {'actorder': True, 'percdamp': 0.01, 'blocksize': 128, 'hessian_batch': 4,
                                'pinned_perms': pins})
    outs = runner.block_opt(gblock, [x.cuda() for x in xs], kwargs, subsets=pairs)
    torch.cuda.synchronize()
    assert runner.forward_passes == 5
    with torch.no_grad():
        fp_block = copy.deepcopy(block).cuda()
        ys = [fp_block(x.cuda()) for x in xs]
        o_fp = torch.cat([y[0] if isinstance(y, tuple) else y for y in ys]).float().cpu()
    for si, sub in enumerate(names(gblock)):
        for name, parent, attr in sub:
            mod = getattr(parent, attr)
            assert isinstance(mod, FakeQuantLinear) and mod.bias is not None
            r = ref_res[name]
            R, C = r['weight'].shape
            got = {'weight': mod.weight.cpu(), 'buf_scales': mod.buf_scales.cpu(), 'buf_zeros': mod.buf_zeros.cpu(),
                   'buf_perm': mod.buf_perm.cpu(), 'buf_invperm': mod.buf_invperm.cpu()}
            a, b = torch.empty(R, C), torch.empty(R, C)
            a[:, got['buf_perm']] = gptq_ref.codes_permuted(got)
            b[:, r['buf_perm'].cpu()] = gptq_ref.codes_permuted({k: (v.cpu() if torch.is_tensor(v) else v)
                                                                  for k, v in r.items()})
            mism = float((a != b).float().mean())
            print(f'opt {name}: code mismatch {mism:.4%}')
            assert mism < 1e-3, (name, mism)
    o_ref = torch.cat([o.cpu() for o in ref_out]).float()
    o_gpu = torch.cat([o.cpu() for o in outs]).float()
    e_ref = float((o_ref - o_fp).norm() / o_fp.norm())
    e_gpu = float((o_gpu - o_fp).norm() / o_fp.norm())
    print(f'opt block output error vs the unquantised block: oracle {e_ref:.5f}, ours {e_gpu:.5f}')
    assert abs(e_gpu - e_ref) <= 0.01 * e_ref
