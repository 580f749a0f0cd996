"""Fused RMS norm, rotary embedding and gated activation against the chains of torch ops they replace in the
calibration block forward (the decoder block's stock module code, run by the reference's
block_forward, llmc/compression/quantization/base_blockwise_quantization.py:378-401): bit-exact."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def _rope_chain(q, k, cos, sin):
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return (q * cos) + (_rotate_half(q) * sin), (k * cos) + (_rotate_half(k) * sin)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape', [(1, 2048, 32, 128), (3, 130, 8, 64), (2, 7, 1, 16)])
def test_rope_matches_the_op_chain(dtype, shape):
    from lightcompress_b200 import block_ops
    B, T, H, D = shape
    g = torch.Generator().manual_seed(B * 1000 + T)
    q = torch.randn(B, T, H * D, generator=g).to(dtype).cuda().view(B, T, H, D).transpose(1, 2)
    k = (torch.randn(B, T, H * D, generator=g) * 3).to(dtype).cuda().view(B, T, H, D).transpose(1, 2)
    ang = torch.rand(B, T, D, generator=g) * 6.28
    cos, sin = ang.cos().to(dtype).cuda(), ang.sin().to(dtype).cuda()
    rq, rk = _rope_chain(q, k, cos, sin)
    oq, ok = block_ops.rope_apply_one(q, cos, sin), block_ops.rope_apply_one(k, cos, sin)
    assert oq.shape == rq.shape and (H == 1 or oq.stride() == rq.stride())
    assert torch.equal(oq, rq) and torch.equal(ok, rk)
    # one table shared by all sequences of the batch: cos / sin of shape (1, T, D)
    rq1, _ = _rope_chain(q, k, cos[:1], sin[:1])
    assert torch.equal(block_ops.rope_apply_one(q, cos[:1].contiguous(), sin[:1].contiguous()), rq1)


def test_fused_gated_mlp_swaps_and_restores_the_forward():
    from lightcompress_b200 import block_ops
    import transformers.models.llama.modeling_llama as ml
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=4,
                      num_hidden_layers=1, vocab_size=64)
    mlp = ml.LlamaMLP(cfg).to(torch.bfloat16).cuda()
    x = torch.randn(3, 40, 256).to(torch.bfloat16).cuda()
    orig = ml.LlamaMLP.forward
    with torch.no_grad():
        ref = mlp(x)
        with block_ops.fused_gated_mlp(mlp) as active:
            assert active and ml.LlamaMLP.forward is not orig
            assert torch.equal(mlp(x), ref)
    assert ml.LlamaMLP.forward is orig


def test_rope_patch_swaps_and_restores_the_module_function():
    from lightcompress_b200 import block_ops
    import transformers.models.llama.modeling_llama as ml
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=4,
                      num_hidden_layers=1, vocab_size=64)
    attn = ml.LlamaAttention(cfg, 0)
    orig = ml.apply_rotary_pos_emb
    with block_ops.fused_rotary(attn, torch.device('cuda'), torch.bfloat16) as active:
        assert active and ml.apply_rotary_pos_emb is not orig
        # a layout outside the kernel's (contiguous (B, H, T, D)) goes through the stock function
        q = torch.randn(1, 4, 8, 64).to(torch.bfloat16).cuda()
        cos = torch.randn(1, 8, 64).to(torch.bfloat16).cuda()
        a, _ = ml.apply_rotary_pos_emb(q, q, cos, cos)
        b, _ = orig(q, q, cos, cos)
        assert torch.equal(a, b)
    assert ml.apply_rotary_pos_emb is orig


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
def test_silu_mul_matches_the_op_chain(dtype):
    from lightcompress_b200 import block_ops
    g = torch.Generator().manual_seed(5)
    gate = (torch.randn(2048, 11008, generator=g) * 3)
    gate[0, :16] = torch.tensor([0., -0., 1e-30, -1e-30, 20., -20., 90., -90., 104., -104., float('inf'),
                                 float('-inf'), float('nan'), 1e4, -1e4, 0.5])
    gate = gate.to(dtype).cuda()
    up = torch.randn(2048, 11008, generator=g).to(dtype).cuda()
    ref = F.silu(gate) * up
    out = block_ops.silu_mul(gate, up)
    assert torch.equal(torch.isnan(out), torch.isnan(ref))
    assert torch.equal(torch.nan_to_num(out, nan=0.), torch.nan_to_num(ref, nan=0.))
    assert torch.equal(block_ops.gated_act(torch.nn.SiLU(), gate, up).isnan(), ref.isnan())
    # an activation that is not SiLU keeps the stock ops
    gelu = torch.nn.GELU()
    assert torch.equal(torch.nan_to_num(block_ops.gated_act(gelu, gate, up), nan=0.),
                       torch.nan_to_num(gelu(gate) * up, nan=0.))


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('shape', [(1, 2048, 4096), (2, 500, 5120), (1, 64, 128), (1, 33, 8064), (1, 2048, 2048)])
def test_rmsnorm_matches_the_module(dtype, shape):
    """Bit equality with the stock module includes the association of the sum of squares."""
    from lightcompress_b200 import block_ops
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    g = torch.Generator().manual_seed(shape[1])
    x = torch.randn(*shape, generator=g)
    x[:, ::3] *= 17.0
    x[0, 0] = 0.0
    x = x.to(dtype).cuda()
    mod = LlamaRMSNorm(shape[-1], eps=1e-5).to(dtype).cuda()
    mod.weight.data = (torch.randn(shape[-1], generator=g) * 0.3 + 1).to(dtype).cuda()
    ref = mod(x)
    raw = block_ops._rms_raw(x, mod.weight.data, mod.variance_epsilon)
    assert torch.equal(raw, ref)
    assert torch.equal(block_ops.rms_norm(mod, x), ref)
    # a width outside the kernel's range, or a module that is not an RMS norm, keeps the stock code
    ln = torch.nn.LayerNorm(shape[-1]).to(dtype).cuda()
    assert torch.equal(block_ops.rms_norm(ln, x), ln(x))
