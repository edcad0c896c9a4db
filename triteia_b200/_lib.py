"""ctypes binding of libtriteia_b200.so (the C ABI declared in include/triteia_b200.h).

The product path has NO fallback: if the shared library is missing or a symbol cannot be
resolved, importing this module raises.  Build it with `python -m triteia_b200.build`.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libtriteia_b200.so")

TRB_OK, ERR_PROB_SHAPE, ERR_KERN_SHAPE, ERR_BAD_ARG, ERR_CUDA, ERR_TIMEOUT, ERR_SCRATCH = range(7)
TRB_F16, TRB_BF16 = 0, 1

_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); must list every function of include/triteia_b200.h
SIGNATURES = {
    "trb_version": (_i, []),
    "trb_status_string": (ctypes.c_char_p, [_i]),
    "trb_device_status": (_i, [_i, ctypes.POINTER(_i)]),
    "trb_selftest_timeout": (_i, [_i, _vp, _i, _vp]),
    "trb_mul_2_4": (_i, [_vp] * 5 + [_i] * 3 + [_vp, _i, _i, _vp] + [_i] * 4),
    "trb_sbmm_2_4": (_i, [_vp] * 8 + [_i] * 4 + [_vp, _i, _i, _vp] + [_i] * 4),
    "trb_bmm_2_4": (_i, [_vp] * 5 + [_i] * 3 + [_vp, _i, _i, _vp] + [_i] * 4),
    "trb_route": (_i, [_vp, _i, _i, _i, _i] + [_vp] * 8 + [_i, _vp]),
    "trb_route_max_tiles": (_i, [_i, _i, _i]),
    "trb_sbmm_indexed_scratch_bytes": (_sz, [_i, _i, _i]),
    "trb_sbmm_indexed_scratch_min_bytes": (_sz, [_i, _i, _i]),
    "trb_sbmm_ksplit_bytes": (_sz, []),
    "trb_sbmm_2_4_ksplit": (_i, [_vp] * 8 + [_i] * 6 + [_vp, _vp, _sz]),
    "trb_sbmm_indexed": (_i, [_vp] * 6 + [_i] * 7 + [_vp, _sz, _i, _vp]),
    "trb_sbmm_indexed_phase": (_i, [_vp] * 6 + [_i] * 7 + [_vp, _sz, _i, _i, _vp]),
    "trb_sbmm_indexed_static_capacity": (_sz, []),
    "trb_sbmm_indexed_static": (_i, [_vp] * 6 + [_i] * 7 + [_i, _vp]),
    "trb_shard_buffer_rows": (_sz, [_i, _i]),
    "trb_shard_dispatch": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _vp]),
    "trb_shard_compute": (_i, [_vp] * 5 + [_i] * 6 + [_vp, _i, _vp, _sz, _i, _vp]),
    "trb_shard_combine": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "trb_unpack_2_4": (_i, [_vp] * 4 + [_i] * 4 + [_vp]),
    "trb_pack_2_4": (_i, [_vp] * 5 + [_i] * 4 + [_vp]),
    "trb_gelu_quick": (_i, [_vp, _vp, ctypes.c_longlong, _i, _i, _vp]),
    "trb_silu_and_mul": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "trb_rotary_embedding": (_i, [_vp] * 5 + [_i, _i, ctypes.c_longlong, ctypes.c_longlong] + [_i] * 6 + [_vp]),
    "trb_row_checksum": (_i, [_vp] * 2 + [_i] * 4 + [_vp]),
    "trb_stack_scratch_bytes": (_sz, [_i, _i]),
    "trb_stack_pass": (_i, [_i] + [_vp] * 5 + [_i, _vp] + [_vp] * 5 + [_i, _i, _vp, _i, _vp, _sz, _i, _vp]),
    "trb_bgmv": (_i, [_vp] * 4 + [_i] * 5 + [_f, _i, _i, _vp]),
    "trb_lora_bgmv_fused": (_i, [_vp] * 5 + [_i] * 6 + [_f, _i, _i, _vp]),
    "trb_lora_indexed": (_i, [_vp] * 5 + [_i] * 6 + [_f, _i, _i, _vp]),
    "trb_base_gemm": (_i, [_vp] * 3 + [_i] * 3 + [_vp, _vp] + [_i] * 4 + [_vp]),
    "trb_sgmv_stacked": (_i, [_vp] * 4 + [_i] * 8 + [_vp]),
    "trb_lora_shrink_rows": (_i, [_vp] * 4 + [_i] * 6 + [_f, _i, _vp]),
    "trb_sgmv_tmp_size": (_sz, [_i]),
    "trb_sgmv": (_i, [_vp] * 5 + [_i] * 6 + [_vp]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m triteia_b200.build`); there is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_of(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def dev_of(t):
    if not t.is_cuda:
        raise RuntimeError("triteia_b200: tensors must live on a CUDA device (there is no CPU path)")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def status_string(code):
    return lib.trb_status_string(int(code)).decode()


def check(code, what):
    if code != TRB_OK:
        raise RuntimeError(f"{what}: {status_string(code)} (status {code})")


def device_status(dev=None):
    """Synchronise `dev` and return (then clear) its device-side error word."""
    d = torch.cuda.current_device() if dev is None else dev
    out = _i(0)
    check(lib.trb_device_status(d, ctypes.byref(out)), "trb_device_status")
    return out.value


def dtype_tag(dtype):
    if dtype == torch.float16:
        return TRB_F16
    if dtype == torch.bfloat16:
        return TRB_BF16
    raise RuntimeError(f"No suitable kernel. dtype={dtype}")
