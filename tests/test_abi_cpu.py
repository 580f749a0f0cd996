"""CPU checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, and validates arguments without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, 'include', 'lc_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(lc_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_are_exported_and_bound():
    from lightcompress_b200 import _lib
    names = _declared()
    assert 'lc_rtn_int_quant' in names and 'lc_hessian_accum' in names and len(names) >= 12
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f'{n} is declared in include/lc_b200.h but not exported'
        assert n in _lib.SIGNATURES, f'{n} has no ctypes signature'
    assert sorted(_lib.SIGNATURES) == names


def test_status_strings_and_version():
    from lightcompress_b200 import _lib
    assert _lib.lib.lc_version() >= 100
    assert _lib.status_string(0) == 'ok'
    assert 'timed out' in _lib.status_string(_lib.LC_ERR_TIMEOUT)


def test_argument_validation_needs_no_gpu():
    from lightcompress_b200 import _lib
    lib = _lib.lib
    # unknown dtype / bad bits / pack4 with 8 bits / cols not divisible by the group
    assert lib.lc_rtn_int_quant(None, 7, 4, 128, 128, 4, 0, None, None, None, None, 0, None, None, None) == _lib.LC_ERR_ARG
    assert lib.lc_rtn_int_quant(None, 0, 4, 128, 128, 9, 0, None, None, None, None, 0, None, None, None) == _lib.LC_ERR_ARG
    assert lib.lc_rtn_int_quant(ctypes.c_void_p(16), 0, 4, 200, 128, 4, 0, None, None, None, None, 0, None, None, None) == _lib.LC_ERR_SHAPE
    # empty input is a no-op, like the reference on an empty tensor
    assert lib.lc_rtn_int_quant(None, 0, 0, 128, 128, 4, 0, None, None, None, None, 0, None, None, None) == _lib.LC_OK
    assert lib.lc_hessian_accum(ctypes.c_void_p(16), 8, 12, ctypes.c_void_p(16), 1.0, 1.0, 0, None, None) == _lib.LC_ERR_ALIGN
    assert lib.lc_gptq_block_quant(None, None, 1, 128, 0, 128, 4, 0, None, None, None, 1, None, None, None) == _lib.LC_ERR_ARG


def test_cpu_tensors_are_rejected_loudly():
    import torch
    from lightcompress_b200 import IntegerQuantizer
    q = IntegerQuantizer(4, False, 'per_group', group_size=128)
    with pytest.raises(RuntimeError, match='no CPU path'):
        q.fake_quant_weight_dynamic(torch.zeros(4, 128))
    with pytest.raises(ValueError):
        q.fake_quant_weight_dynamic(torch.zeros(4, 200))


def test_unsupported_configurations_raise():
    from lightcompress_b200 import GPTQ, FloatQuantizer, IntegerQuantizer
    with pytest.raises(NotImplementedError):
        IntegerQuantizer(4, False, 'per_group', group_size=128, calib_algo='mse')._check_supported()
    with pytest.raises(NotImplementedError):
        FloatQuantizer('e5m2', True, 'per_channel', use_qtorch=True)
    with pytest.raises(NotImplementedError):
        GPTQ(IntegerQuantizer(4, False, 'per_group', group_size=64))


def test_export_config_writers_match_the_reference(tmp_path):
    """config.json entries for the vLLM (compressed-tensors / fp8) and AutoAWQ exports against what the
    reference's writers produced for the same YAML sections (tests/golden/export_configs.json)."""
    import importlib.util
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    # export.py's packing functions need the GPU library; its config writers are plain Python: load by path
    spec = importlib.util.spec_from_file_location(
        'lightcompress_b200.export', os.path.join(here, '..', 'lightcompress_b200', 'export.py'),
        submodule_search_locations=None)
    import lightcompress_b200  # noqa: F401  (package context for the relative import)
    ex = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ex)
    with open(os.path.join(here, 'golden', 'export_configs.json')) as f:
        cases = json.load(f)
    assert len(cases) == 7
    for name, c in cases.items():
        d = tmp_path / name
        d.mkdir()
        with open(d / 'config.json', 'w') as f:
            json.dump({'model_type': 'llama', 'quantization_config': {'old': 1}}, f)
        if name == 'autoawq':
            ex.update_autoawq_quant_config(str(d), c['in']['weight'])
        else:
            ex.update_vllm_quant_config(str(d), c['in']['weight'], c['in'].get('act'), ignore=['lm_head'])
        with open(d / 'config.json') as f:
            assert json.load(f) == c['config_json'], name
