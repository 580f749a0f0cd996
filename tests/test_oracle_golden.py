"""The CPU oracle must reproduce, bit for bit, what the reference produced when the golden
fixtures were generated (tests/golden/make_golden.py ran the reference itself on CPU)."""
import torch

from oracle import gptq_ref, quant_ref


def _eq(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    assert torch.equal(a.view(torch.uint8) if a.dtype == torch.float8_e4m3fn else a,
                       b.view(torch.uint8) if b.dtype == torch.float8_e4m3fn else b)


def test_rtn_int_oracle_matches_reference(golden):
    cases = golden('rtn_int.pt')
    assert len(cases) == 40
    for key, c in cases.items():
        fq = quant_ref.int_fake_quant_dynamic(c['w'], c['bit'], c['sym'], c['granularity'], c['group_size'])
        _eq(fq, c['fake'])
        if 'codes' in c:
            q, s, z = quant_ref.int_real_quant_dynamic(c['w'], c['bit'], c['sym'], c['granularity'], c['group_size'])
            _eq(q, c['codes'])
            _eq(s, c['scales'])
            if c['sym']:
                assert z is None and c['zeros'] is None
            else:
                _eq(z, c['zeros'])


def test_rtn_mse_oracle_matches_reference(golden):
    """calib_algo 'mse': searched ranges (including the reference's in-place compounding of accepted
    shrinks) and the fake-quantised weight."""
    cases = golden('rtn_mse.pt')
    assert len(cases) == 8
    for key, c in cases.items():
        g = quant_ref.group_view(c['w'], c['granularity'], c['group_size'])
        mn, mx = quant_ref.mse_range(g, c['bit'], c['sym'])
        _eq(mn, c['min'])
        _eq(mx, c['max'])
        _eq(quant_ref.int_fake_quant_mse(c['w'], c['bit'], c['sym'], c['granularity'], c['group_size']), c['fake'])


def test_fp8_oracle_matches_reference_with_substituted_rounding(golden):
    for key, c in golden('fp8_e4m3.pt').items():
        assert c['pinned'] is False       # qtorch is not vendored: parity unpinned for the rounding call
        _eq(quant_ref.fp8_fake_quant_dynamic(c['w']), c['fake'])
        q, s = quant_ref.fp8_real_quant_dynamic(c['w'])
        _eq(q.view(torch.uint8), c['codes'])
        _eq(s, c['scales'])
        _eq(quant_ref.fp8_fake_quant_dynamic(c['x']), c['fake_act'])


def test_fp8_block_oracle_matches_reference_with_substituted_rounding(golden):
    """Block-wise FP8 weights (one fp32 scale per 128 x 128 block): the reference's weight_cast_to_fp8 /
    weight_cast_to_bf16 and per_block fake quant, with the same substituted float rounding as above."""
    cases = golden('fp8_block.pt')
    assert len(cases) == 4
    for key, c in cases.items():
        codes, s = quant_ref.fp8_block_real_quant(c['w'])
        assert torch.equal(codes.view(torch.uint8), c['codes']), key
        _eq(s, c['scales'])
        _eq(quant_ref.fp8_block_dequant(codes, s), c['back'])
        _eq(quant_ref.fp8_block_fake_quant(c['w']), c['fake'])


def test_gptq_oracle_matches_reference(golden):
    torch.set_num_threads(1)
    for key, c in golden('gptq_layer.pt').items():
        st = gptq_ref.hessian_init(c['W'].shape[1])
        for i in range(c['X'].shape[0]):
            gptq_ref.add_batch(st, c['X'][i:i + 1])
        _eq(st['H'], c['H'])
        res = gptq_ref.quantize_layer(c['W'], c['H'], bit=c['bit'], sym=c['sym'],
                                      percdamp=c['percdamp'], actorder=c['actorder'])
        _eq(res['buf_perm'], c['buf_perm'])
        _eq(res['weight'], c['weight'])
        _eq(res['buf_scales'], c['buf_scales'])
        if not c['sym']:
            _eq(res['buf_zeros'], c['buf_zeros'])
        codes = gptq_ref.codes_permuted(res, c['bit'], c['sym'])
        assert torch.equal(codes.to(torch.int16), c['codes_perm'])
        _eq(gptq_ref.w_qdq(res, c['W'].dtype, c['bit'], c['sym']), c['w_qdq'])


def test_gptq_static_groups_oracle_matches_reference(golden):
    """static_groups: the solver quantises with the layer's round-to-nearest qparams (by original column
    group under act-order), the buffers stay, and the deploy step needs no permutation."""
    torch.set_num_threads(1)
    cases = golden('gptq_static.pt')
    assert len(cases) == 3
    for key, c in cases.items():
        res = gptq_ref.quantize_layer(c['W'], c['H'], bit=c['bit'], sym=c['sym'], percdamp=c['percdamp'],
                                      actorder=c['actorder'], static_groups=True)
        _eq(res['weight'], c['weight'])
        _eq(res['buf_scales'], c['buf_scales'])
        if not c['sym']:
            _eq(res['buf_zeros'], c['buf_zeros'])
        codes = gptq_ref.codes_permuted(res, c['bit'], c['sym'])
        assert torch.equal(codes.to(torch.int16), c['codes_perm'])
        _eq(gptq_ref.w_qdq(res, c['W'].dtype, c['bit'], c['sym']), c['w_qdq'])


def test_gptq_per_channel_oracle_matches_reference(golden):
    """per_channel weights (the reference's w8a8 GPTQ configs): one fixed scale per row for every column."""
    torch.set_num_threads(1)
    cases = golden('gptq_per_channel.pt')
    assert len(cases) == 2
    for key, c in cases.items():
        res = gptq_ref.quantize_layer(c['W'], c['H'], bit=c['bit'], sym=c['sym'], percdamp=c['percdamp'],
                                      actorder=c['actorder'], granularity='per_channel')
        _eq(res['weight'], c['weight'])
        _eq(res['buf_scales'], c['buf_scales'])
        if not c['sym']:
            _eq(res['buf_zeros'], c['buf_zeros'])
        C = c['W'].shape[1]
        codes = gptq_ref.codes_permuted(res, c['bit'], c['sym'], group_size=C)
        assert torch.equal(codes.to(torch.int16), c['codes_perm'])
        _eq(gptq_ref.w_qdq(res, c['W'].dtype, c['bit'], c['sym'], group_size=C), c['w_qdq'])


def test_gptq_owq_oracle_matches_reference(golden):
    """owq: the n_out columns with the largest Hessian diagonal are permuted to the end and stay
    unquantised (error feedback only); everything else as GPTQ without act-order."""
    torch.set_num_threads(1)
    cases = golden('gptq_owq.pt')
    assert len(cases) == 2
    for key, c in cases.items():
        res = gptq_ref.quantize_layer(c['W'], c['H'], bit=c['bit'], sym=c['sym'], percdamp=c['percdamp'],
                                      actorder=False, n_out=c['n_out'])
        _eq(res['buf_perm'], c['buf_perm'])
        _eq(res['weight'], c['weight'])
        _eq(res['buf_scales'], c['buf_scales'])
        if not c['sym']:
            _eq(res['buf_zeros'], c['buf_zeros'])
        _eq(gptq_ref.w_qdq(res, c['W'].dtype, c['bit'], c['sym']), c['w_qdq'])


def test_spqr_oracle_matches_reference(golden):
    """SpQR: leave-one-out outlier detection, simplified outliers, no outliers, with and without
    act-order — compensated weight, outlier mask, statistics and deploy-time weight, bit for bit."""
    from oracle import spqr_ref
    torch.set_num_threads(1)
    cases = golden('spqr_layer.pt')
    assert len(cases) == 4
    for key, c in cases.items():
        res = spqr_ref.quantize_layer(c['W'], c['H'], bit=c['bit'], group_size=c['group'], percdamp=c['percdamp'],
                                      relative_threshold=c['rel_threshold'], simplified=c['simplified'],
                                      actorder=c['actorder'])
        _eq(res['buf_perm'], c['buf_perm'])
        _eq(res['mask'], c['mask'])
        _eq(res['weight'], c['weight'])
        _eq(res['buf_scales'], c['buf_scales'])
        _eq(res['buf_zeros'], c['buf_zeros'])
        _eq(spqr_ref.w_qdq(res, c['W'].dtype, c['bit'], c['group']), c['w_qdq'])


def test_static_activation_ranges_oracle_matches_reference(golden):
    """calib_algo 'static_minmax' / 'static_moving_minmax' (per_tensor): qparams from a batch of
    calibration activations and the static fake quant that uses them."""
    cases = golden('act_static.pt')
    assert len(cases) == 12
    for key, c in cases.items():
        (s, z, qmax, qmin), = quant_ref.batch_tensors_qparams([a.clone() for a in c['acts']], c['bit'], c['sym'],
                                                              c['algo'])
        _eq(s, c['scales'])
        _eq(z, c['zeros'])
        fq = quant_ref.int_fake_quant_static(c['x'], s, z, c['bit'], c['sym'], 'per_tensor')
        _eq(fq, c['fake'])


def test_w48_oracle_matches_reference(golden):
    """Weight48IntegerQuantizer: 8-bit rows, then 4-bit groups of the codes, and back."""
    cases = golden('rtn_w48.pt')
    assert len(cases) == 12
    for key, c in cases.items():
        _eq(quant_ref.w48_fake_quant(c['w'], c['bit4'], c['bit8']), c['fake'])


def test_quik_mixed_precision_oracle_matches_reference(golden):
    """QUIK: activation statistic, column split and the int / fp mixed fake quant of weight and activation."""
    cases = golden('quik_mixed.pt')
    assert len(cases) == 6
    for key, c in cases.items():
        stat = None
        for a in c['acts']:
            stat = quant_ref.quik_col_absmax(stat, a)
        _eq(stat, c['stat'])
        int_ids, fp_ids = quant_ref.quik_select(stat, c['fp_ids'].numel())
        _eq(int_ids, c['int_ids'])
        _eq(fp_ids, c['fp_ids'])
        _eq(quant_ref.int_fake_quant_mixed(c['w'], c['wbit'], c['sym'], 'per_channel', int_ids, fp_ids), c['fake_w'])
        _eq(quant_ref.int_fake_quant_mixed(c['acts'][0], c['abit'], c['sym'], 'per_token', int_ids, fp_ids),
            c['fake_a'])


def test_group_not_divisible_raises():
    import pytest
    with pytest.raises(ValueError):
        quant_ref.int_fake_quant_dynamic(torch.zeros(2, 200), 4, False, 'per_group', 128)


def _tiny_block(state, hidden=256, inter=512, heads=4, T=64):
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=1, vocab_size=128, max_position_embeddings=4 * T)
    cfg._attn_implementation = 'sdpa'
    block = LlamaDecoderLayer(cfg, 0).to(torch.bfloat16)
    block.load_state_dict(state)
    rot = LlamaRotaryEmbedding(cfg)
    pos = torch.arange(T)[None]
    cos, sin = rot(torch.zeros(1, T, hidden, dtype=torch.bfloat16), pos)
    return block, {'position_embeddings': (cos, sin), 'attention_mask': None, 'position_ids': pos}


def test_awq_oracle_matches_reference_block(golden):
    """The reference's own Awq.block_transform (scale search, scale application, clip search and
    clamp) on a tiny Llama block: the oracle must leave bit-identical weights and norms."""
    from oracle import awq_ref
    torch.set_num_threads(1)
    for key, c in golden('awq_block.pt').items():
        block, kwargs = _tiny_block(c['state0'])
        awq_ref.awq_block(block, c['x'], kwargs, bit=4, sym=c['sym'], clip_sym=c['clip_sym'], n_sample_token=64)
        got = block.state_dict()
        for k, v in c['state1'].items():
            assert torch.equal(got[k], v), (key, k, int((got[k] != v).sum()))
        assert any(not torch.equal(c['state0'][k], c['state1'][k]) for k in c['state1'])


def test_gptq_block_schedule_oracle_matches_the_references_run_block_loop(golden):
    """oracle/gptq_block_ref.py against the reference's own GPTQ run_block_loop() on a two-layer Llama
    (tests/golden/make_golden.py: make_gptq_block): the compensated weight, scales, zeros and
    permutation of all fourteen linears, and the tensors handed on after each block, bit for bit."""
    from oracle import gptq_block_ref
    torch.set_num_threads(1)
    c = golden('gptq_block_loop.pt')
    sh = c['shape']
    inputs = [x.clone() for x in c['x0']]
    assert c['module_classes'].count('FakeQuantLinear') == 1            # quant_out leaves fake-quant linears
    for bi, state in enumerate(c['state0']):
        from transformers.models.llama.modeling_llama import LlamaDecoderLayer
        from oracle import ref_driver as rd
        block = LlamaDecoderLayer(rd.tiny_llama_config(**sh), bi).to(torch.bfloat16)
        block.load_state_dict(state)
        kwargs = c['kwargs']          # as the reference's catcher recorded them (base_model.py:172-191)
        results, inputs = gptq_block_ref.gptq_block(block, inputs, kwargs)
        assert list(results) == list(c['linears'][bi])
        for name, want in c['linears'][bi].items():
            got = results[name]
            for k in ('weight', 'buf_scales', 'buf_zeros', 'buf_perm', 'buf_invperm'):
                assert got[k].dtype == want[k].dtype and torch.equal(got[k], want[k]), (bi, name, k)
    for a, b in zip(inputs, c['next_inputs']):
        assert torch.equal(a, b)


def test_static_hist_oracle_matches_reference(golden):
    """calib_algo 'static_hist': the searched range and the resulting scale of the reference's
    get_static_hist_range / get_batch_tensors_qparams, bit for bit."""
    for key, c in golden('act_hist.pt').items():
        mins, maxs = quant_ref.static_hist_range([a.clone() for a in c['acts']], 8)
        _eq(mins[0], c['min'])
        _eq(maxs[0], c['max'])
        (s, z, qmax, qmin), = quant_ref.batch_tensors_qparams([a.clone() for a in c['acts']], 8, True, 'static_hist')
        _eq(s, c['scales'])
        assert c['max'] < max(a.max() for a in c['acts']).float()       # the search did clip the range
