"""ctypes binding of libb200mixers.so (include/b200_mixers.h): the kernels of decoder layers that are not softmax attention.

The library is built on first use when it is missing or older than its sources (``build_native.build_mixers``: a handful of small
files, seconds) -- a fresh checkout serves such a model without building the low-bit library.  There is no CPU or PyTorch
fallback: without the library, or on tensors that are not on a CUDA device, the calls raise.
"""
import ctypes
import os

import torch

from ipex_llm_b200.utils.common import invalidInputError

_lib = None
LIB_PATH = None


class MixersNativeError(RuntimeError):
    pass


_c_int, _c_long, _c_float, _c_ptr = ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_void_p
_SIGNATURES = {
    "mixers_embed_rows": [_c_int, _c_ptr, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr],
    "mixers_dyt_residual_norm": [_c_int, _c_ptr, _c_long, _c_int] + [_c_ptr] * 9 + [_c_ptr],
    "mixers_window_qk_prepare": [_c_int, _c_ptr] + [_c_int] * 10 + [_c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                                                 _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_sigmoid_window_attention": [_c_int, _c_ptr, _c_ptr, _c_ptr] + [_c_int] * 9 + [_c_ptr, _c_int, _c_float, _c_ptr, _c_ptr, _c_int,
                                                                                          _c_int, _c_float, _c_ptr, _c_ptr],
    "mixers_short_conv_silu": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_gated_delta_rule": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                                                                 _c_ptr, _c_ptr],
    "mixers_gated_linear_attention": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_gated_rms_norm": [_c_int, _c_ptr, _c_long, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_float, _c_ptr, _c_int, _c_int,
                              _c_float, _c_int, _c_ptr],
    "mixers_short_conv": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_channel_delta_rule": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                                                                   _c_ptr, _c_ptr],
    "mixers_state_space_scan": [_c_int, _c_ptr] + [_c_int] * 6 + [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                                                                 _c_ptr, _c_ptr],
    "mixers_sigmoid_gate": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr],
    "mixers_rms_pair_sum": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_float, _c_long, _c_int, _c_ptr, _c_ptr],
    "mixers_sum_residual_norms": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_long, _c_int,
                                  _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "mixers_gelu_erf": [_c_int, _c_ptr, _c_long, _c_ptr, _c_ptr],
    "mixers_rope_qk_prepare": [_c_int, _c_ptr] + [_c_int] * 14 + [_c_ptr, _c_float, _c_ptr, _c_int, _c_float, _c_ptr, _c_ptr, _c_long, _c_long,
                                                                 _c_long, _c_ptr, _c_long, _c_long, _c_long, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_moe_scatter_scaled": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_long, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "mixers_token_shift_mix": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_wkv": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr,
                   _c_ptr],
    "mixers_layer_norm_residual": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr],
    "mixers_clamped_glu": [_c_int, _c_ptr, _c_long, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr],
    "mixers_wide_qkv_prepare": [_c_int, _c_ptr] + [_c_int] * 10 + [_c_ptr, _c_ptr, _c_float, _c_ptr, _c_long, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                                                _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_scored_router": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                             _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "mixers_poly_norm": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_float, _c_ptr, _c_ptr],
    "mixers_soft_cap": [_c_int, _c_ptr, _c_long, _c_float, _c_ptr, _c_ptr],
    "mixers_embed_pair": [_c_int, _c_ptr, _c_float, _c_ptr, _c_long, _c_long, _c_long, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                          _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "mixers_rms_residual": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr,
                            _c_ptr],
    "mixers_rms_norm_rows": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr],
    "mixers_xielu": [_c_int, _c_ptr, _c_long, _c_ptr, _c_ptr, _c_ptr],
    "mixers_silu_mul": [_c_int, _c_ptr, _c_long, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "mixers_gelu_table_mul": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_latent_prepare": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_float, _c_ptr, _c_ptr,
                              _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_softmax_attention": [_c_int, _c_ptr, _c_long, _c_long, _c_ptr, _c_long, _c_long, _c_long, _c_ptr, _c_long, _c_long, _c_long] + [_c_int] * 8
                                + [_c_ptr, _c_int, _c_int, _c_float, _c_float, _c_ptr, _c_ptr, _c_long, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "mixers_grouped_router": [_c_int, _c_ptr, _c_long, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr],
    "mixers_moe_small": [_c_int, _c_ptr, _c_long, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                         _c_int, _c_int, _c_float, _c_float, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "mixers_moe_sort": [_c_ptr, _c_long, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "mixers_moe_combine": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_long, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
}


def lib():
    global _lib, LIB_PATH
    if _lib is None:
        from ipex_llm_b200 import build_native
        path = os.environ.get("B200_MIXERS_LIB") or build_native.build_mixers()
        try:
            loaded = ctypes.CDLL(path)
        except OSError as e:
            invalidInputError(False, f"Failed to load shared library '{path}': {e}.")
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.argtypes, fn.restype = argtypes, _c_int
        loaded.mixers_softmax_attention_workspace.argtypes = [_c_int] * 7
        loaded.mixers_softmax_attention_workspace.restype = _c_long
        _lib, LIB_PATH = loaded, path
    return _lib


_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def dtype_code(dtype):
    invalidInputError(dtype in _DTYPES, f"the mixer kernels take float32, bfloat16 or float16, not {dtype}")
    return _DTYPES[dtype]


def ptr(t):
    if t is None:
        return None
    invalidInputError(t.device.type == "cuda", "the mixer kernels run on CUDA tensors only (there is no CPU path)")
    invalidInputError(t.numel() > 0, "an empty tensor has no data pointer to hand to a kernel")
    return t.data_ptr()


def stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def call(name, *args):
    rc = getattr(lib(), name)(*args)
    if rc:
        raise MixersNativeError(f"{name}: CUDA error {rc}")
