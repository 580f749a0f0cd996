"""CPU checks of lightcompress_b200.plugin against the reference's own registry and constructors.

Needs the reference's `llmc` package (baseline/_ref/, placed by `python __graft_entry__.py` where the
checkout is present, or LLMC_REFERENCE_ROOT); skipped otherwise.  No kernel runs here: the test
stops where the first kernel would be called."""
import pytest
import torch

from oracle import ref_driver as rd

pytestmark = pytest.mark.skipif(rd.find_reference() is None, reason='no reference checkout / baseline/_ref')


@pytest.fixture(scope='module')
def ref():
    return rd.import_reference()


def test_install_swaps_registry_and_quantizers_and_uninstall_restores(ref):
    import lightcompress_b200 as lcb
    from lightcompress_b200 import plugin
    import llmc.compression.quantization.spqr  # noqa: F401  (registers SpQR)
    stock = {n: ref.ALGO_REGISTRY[n] for n in ('GPTQ', 'Awq', 'RTN', 'SpQR')}
    stock_q = ref.base.IntegerQuantizer
    classes = plugin.install()
    try:
        for n in ('GPTQ', 'Awq', 'RTN', 'SpQR'):
            cls = ref.ALGO_REGISTRY[n]
            assert cls is classes[n] and cls is not stock[n]
            assert issubclass(cls, stock[n]) and cls.__name__ == n          # looked up by class name
        assert ref.base.IntegerQuantizer is lcb.IntegerQuantizer
        assert ref.base.FloatQuantizer is lcb.FloatQuantizer
        assert ref.base.Weight48IntegerQuantizer is lcb.Weight48IntegerQuantizer
        assert plugin.install() is classes                                  # idempotent
    finally:
        plugin.uninstall()
    assert all(ref.ALGO_REGISTRY[n] is stock[n] for n in stock)
    assert ref.base.IntegerQuantizer is stock_q


def test_constructor_takes_the_yaml_dicts_of_gptq_w_only(ref, monkeypatch):
    """ALGO_REGISTRY['GPTQ'](model, quant_config, input, padding_mask, config) with the `quant` section of
    configs/quantization/methods/GPTQ/gptq_w_only.yml (llmc/__main__.py:63-69)."""
    import os
    import yaml
    import lightcompress_b200 as lcb
    from lightcompress_b200 import plugin
    quant = rd.gptq_quant_config()
    yml = os.path.join(ref.root, rd.HOT_PATH_YAMLS[0])
    if os.path.exists(yml):
        y = yaml.safe_load(open(yml))['quant']
        assert y['weight'] == dict(quant['weight']) and y['special'] == dict(quant['special'])
        assert y['quant_out'] == quant['quant_out'] and y['method'] == 'GPTQ'
    model = rd.synth_llama_adapter(ref, rd.tiny_llama_config(layers=1), seed=1)
    calib = rd.calib_ids(2, 32, 128)
    model.collect_first_block_input(calib, None)
    config = rd.AttrDict(model=dict(type='Llama'), calib=dict(bs=1, seq_len=32, n_samples=2), quant=quant)
    plugin.install()
    try:
        cls = ref.ALGO_REGISTRY['GPTQ']
        # the constructor computes round-to-nearest qparams of every linear (gptq.py:325-330): on this
        # GPU-less machine that is where the first kernel is called, and it must refuse loudly
        with pytest.raises(RuntimeError, match='no CPU path'):
            cls(model, quant, model.get_first_block_input(), None, config)
        monkeypatch.setattr(cls, 'collect_model_qparams', lambda self: None)
        algo = cls(model, quant, model.get_first_block_input(), None, config)
        assert isinstance(algo.wquantizer, lcb.IntegerQuantizer)
        assert (algo.wquantizer.bit, algo.wquantizer.sym, algo.wquantizer.group_size) == (4, False, 128)
        assert algo.need_perm and algo.true_sequential and algo.quant_out and algo.n_samples == 2
        assert algo.layers_cache is algo._b200.layers_cache
        assert (algo._b200.percdamp, algo._b200.blocksize, algo._b200.actorder) == (0.01, 128, True)
        for name in ('layer_init', 'add_batch', 'layer_transform', 'w_qdq', 'free', 'block_opt'):
            assert name in cls.__dict__, name                               # overridden, not inherited
        rtn = ref.ALGO_REGISTRY['RTN'](model, rd.rtn_quant_config(), None, None, config)
        assert isinstance(rtn.wquantizer, lcb.IntegerQuantizer) and rtn.data_free
    finally:
        plugin.uninstall()


def test_spqr_constructor_takes_the_yaml_dicts_of_spqr_w_only(ref):
    """ALGO_REGISTRY['SpQR'](...) with the `quant` section of configs/quantization/methods/SpQR/spqr_w_only.yml:
    the plugin's class builds the B200 solver from the same dicts and overrides the per-layer methods only."""
    import math
    import lightcompress_b200 as lcb
    from lightcompress_b200 import plugin
    quant = rd.spqr_quant_config()
    model = rd.synth_llama_adapter(ref, rd.tiny_llama_config(layers=1), seed=1)
    calib = rd.calib_ids(2, 32, 128)
    model.collect_first_block_input(calib, None)
    config = rd.AttrDict(model=dict(type='Llama'), calib=dict(bs=1, seq_len=32, n_samples=2), quant=quant)
    plugin.install()
    try:
        cls = ref.ALGO_REGISTRY['SpQR']
        algo = cls(model, quant, model.get_first_block_input(), None, config)
        assert isinstance(algo._b200, lcb.SpQR) and isinstance(algo.wquantizer, lcb.IntegerQuantizer)
        assert (algo.wquantizer.bit, algo.wquantizer.group_size, algo.wquantizer.round_zp) == (4, 16, False)
        assert (algo._b200.percdamp, algo._b200.relative_threshold, algo._b200.simplified_outliers) == (1, 0.2, False)
        assert algo.layers_cache is algo._b200.layers_cache and algo._b200.need_perm
        for name in ('layer_init', 'add_batch', 'layer_transform', 'w_qdq', 'free'):
            assert name in cls.__dict__, name
        assert 'block_transform' not in cls.__dict__                        # the reference's own block loop
        inf = lcb.SpQR(algo.wquantizer, dict(quant['special'], relative_threshold='inf'))
        assert inf.relative_threshold == math.inf
        with pytest.raises(NotImplementedError):
            lcb.SpQR(lcb.IntegerQuantizer(4, False, 'per_group', group_size=128), dict(quant['special']))
    finally:
        plugin.uninstall()
