"""ctypes binding of the C-ABI library (include/lc_b200.h).

The library is the product: if it is missing this module raises at import time -- there is
no CPU or pure-torch fallback.  torch is used only to own device memory and streams; raw
`data_ptr()`s and the current stream handle cross the ABI.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'liblc_b200.so')

LC_OK = 0
LC_ERR_ARG, LC_ERR_SHAPE, LC_ERR_ALIGN, LC_ERR_ARCH = -1, -2, -3, -4
LC_ERR_WORKSPACE, LC_ERR_NOT_PD, LC_ERR_TIMEOUT, LC_ERR_CUDA = -5, -6, -7, -8
LC_F32, LC_BF16, LC_F16 = 0, 1, 2
LC_CODES_NONE, LC_CODES_I32, LC_CODES_I8, LC_CODES_PACK4 = 0, 1, 2, 3
LC_GEMM_UPPER_ONLY, LC_GEMM_B_LOWER, LC_GEMM_A_UPPER = 1, 2, 4
LC_H_REVERSE, LC_H_UPPER, LC_H_LATE_DEAD = 1, 2, 4

_DTYPES = {torch.float32: LC_F32, torch.bfloat16: LC_BF16, torch.float16: LC_F16}

_p, _i, _i64, _f, _d = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_double

# name -> argtypes; every function returns int except those given another restype in _load
SIGNATURES = {
    'lc_version': [],
    'lc_status_string': [_i],
    'lc_set_device': [_i],
    'lc_rtn_int_quant': [_p, _i, _i64, _i64, _i64, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p],
    'lc_fp8_e4m3_quant': [_p, _i, _i64, _i64, _p, _p, _p, _p],
    'lc_hessian_accum': [_p, _i64, _i64, _p, _f, _f, _i, _p, _p],
    'lc_hessian_accum_multi': [_p, _p, _i, _i64, _p, _f, _f, _i, _p, _p],
    'lc_hessian_accum_upper': [_p, _p, _i, _i64, _p, _f, _f, _i, _p, _p],
    'lc_selftest_wait_expiry': [_p, _p],
    'lc_gptq_diag': [_p, _i64, _p, _p],
    'lc_gptq_permute_damp': [_p, _i, _p, _p, _i64, _i64, _f, _f, _i, _p, _p, _p, _p],
    'lc_gptq_flip': [_p, _i64, _p, _p],
    'lc_gptq_block_quant': [_p, _p, _i64, _i64, _i64, _i, _i, _i, _p, _p, _p, _i64, _p, _p, _p],
    'lc_gptq_trailing_update': [_p, _p, _p, _i64, _i64, _i64, _i, _i64, _p],
    'lc_gptq_weight_transform': [_p, _p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p],
    'lc_gptq_weight_transform_owq': [_p, _p, _i64, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p],
    'lc_gptq_weight_transform_tc_owq': [_p, _p, _p, _i64, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    'lc_gptq_weight_transform_static': [_p, _p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p, _p],
    'lc_gptq_weight_transform_tc_static': [_p, _p, _p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    'lc_gptq_weight_transform_noalloc': [_p, _p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p],
    'lc_gptq_split_tf32': [_p, _i64, _p, _p],
    'lc_gptq_panel_update': [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _p],
    'lc_gptq_weight_transform_tc': [_p, _p, _p, _i64, _i64, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    'lc_gptq_unpermute': [_p, _p, _i64, _i64, _p, _i, _p],
    'lc_awq_act_mean': [_p, _i, _i64, _i64, _p, _p, _i64, _p],
    'lc_awq_scale_quant': [_p, _p, _i, _i64, _i64, _i64, _i, _i, _p, _p],
    'lc_awq_div_cols': [_p, _p, _i, _i64, _i64, _p, _p],
    'lc_awq_loss': [_p, _p, _i, _i64, _p, _p, _i64, _p],
    'lc_pack_int4_awq': [_p, _i64, _i64, _p, _p],
    'lc_tf32x3_gemm_tn': [_p, _i64, _p, _p, _i64, _p, _p, _i64, _i64, _i64, _i64, _i, _f, _i, _p, _p],
    'lc_gptq_factor_workspace_floats': [_i64],
    'lc_gptq_factorize': [_p, _i64, _p, _p, _p, _i64, _p, _p],
    'lc_gptq_invert_factor': [_p, _i64, _p, _p, _p, _i64, _p, _p],
    'lc_gptq_factor_split': [_i64],
    'lc_gptq_factor_vt_offset': [_i64],
    'lc_gptq_invert_factor_part': [_p, _i64, _p, _i64, _i64, _i64, _p, _p],
    'lc_gptq_invert_factor_finish': [_i64, _p, _i64, _p, _p, _p],
    'lc_fp8_e4m3_block_quant': [_p, _i, _i64, _i64, _i64, _p, _p, _p, _p],
    'lc_fp8_e4m3_block_quant_triton': [_p, _i, _i64, _i64, _i64, _p, _p, _p, _p],
    'lc_fp8_e4m3_block_dequant': [_p, _p, _i64, _i64, _i64, _p, _i, _p],
    'lc_fp8_e4m3_act_quant': [_p, _i, _i64, _i64, _p, _p, _p],
    'lc_fp8_block_gemm': [_p, _p, _p, _p, _i64, _i64, _i64, _p, _i, _p, _p],
    'lc_gptq_dequant_unpermute': [_p, _p, _p, _p, _i64, _i64, _i, _i, _p, _i, _p],
    'lc_act_range_per_tensor': [_p, _p, _i, _i, _p, _p, _p],
    'lc_act_range_moving': [_p, _p, _i, _i, _d, _p, _p],
    'lc_act_hist_per_tensor': [_p, _p, _i, _i, _p, _p, _i, _p, _p],
    'lc_spqr_weight_transform': [_p, _p, _p, _i64, _i64, _i, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p],
    'lc_spqr_dequant': [_p, _p, _p, _p, _p, _i64, _i64, _i, _p, _i, _p],
    'lc_rtn_w48_fake_quant': [_p, _i, _i64, _i64, _i64, _p, _p, _p, _p],
    'lc_quik_col_absmax': [_p, _i, _i64, _i64, _p, _p],
    'lc_rtn_int_fake_quant_masked': [_p, _i, _i64, _i64, _i, _i, _p, _p, _p],
    'lc_rtn_mse_range': [_p, _i, _i64, _i64, _i64, _i, _i, _d, _i, _f, _p, _p, _p],
    'lc_rope_apply': [_p, _p, _p, _i, _i64, _i, _i, _i64, _p, _p],
    'lc_silu_mul': [_p, _p, _i, _i64, _p, _p],
    'lc_rmsnorm': [_p, _p, _i, _i64, _i64, _f, _f, _p, _p],
    'lc_awq_clip_search': [_p, _p, _i, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _d, _p, _p, _p, _p],
    'lc_awq_clip_search_cuda_cores': [_p, _p, _i, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _i, _d, _p, _p, _p, _p],
}


class LcError(RuntimeError):
    def __init__(self, fn, code, text):
        super().__init__(f'{fn} failed: {text} ({code})')
        self.code = code


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f'{LIB_PATH} is missing: build it with `python __graft_entry__.py` '
            '(nvcc, sm_100a).  There is no fallback implementation.')
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise ImportError(f'{LIB_PATH} is stale (no symbol {name}): rebuild it with '
                              '`python __graft_entry__.py`') from None
        fn.argtypes = argtypes
        fn.restype = {'lc_status_string': ctypes.c_char_p,
                      'lc_gptq_factor_workspace_floats': ctypes.c_int64,
                      'lc_gptq_factor_split': ctypes.c_int64,
                      'lc_gptq_factor_vt_offset': ctypes.c_int64}.get(name, ctypes.c_int)
    return lib


lib = _load()


def status_string(code):
    return lib.lc_status_string(int(code)).decode()


def check(fn, code):
    if code != LC_OK:
        raise LcError(fn, code, status_string(code))


def lc_dtype(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f'unsupported dtype {t.dtype}') from None


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError('lightcompress_b200 kernels need CUDA tensors; there is no CPU path')


def stream_of(t):
    """Selects t's device inside the library and returns torch's current stream on it."""
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    check('lc_set_device', lib.lc_set_device(dev))
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def call(name, *args):
    check(name, getattr(lib, name)(*args))
