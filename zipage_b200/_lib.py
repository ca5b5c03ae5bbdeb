"""ctypes binding of libzipage_b200.so (the C ABI declared in include/zipage_b200.h).

The library is the product; there is no Python or CPU fallback.  If the shared
object has not been built, loading raises with the build command.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libzipage_b200.so"

ZP_DTYPE = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}
IMPL = {"auto": 0, "simt": 1, "tcgen05": 2}


class ZipageError(RuntimeError):
    pass


class SelectParams(C.Structure):
    _fields_ = [
        ("top_k", C.c_int32), ("query_cache_len", C.c_int32), ("pooling_size", C.c_int32),
        ("continues_pooling", C.c_int32), ("use_redundancy", C.c_int32),
        ("redundancy_max_norm", C.c_int32), ("sink_len", C.c_int32), ("pad_mask", C.c_int32),
        ("redundancy_lambda", C.c_float), ("redundancy_one_minus_lambda", C.c_float),
        ("redundancy_temperature", C.c_float),
    ]


class CompressParams(C.Structure):
    _fields_ = [
        ("budget_blocks", C.c_int32), ("query_cache_len", C.c_int32), ("use_global_score", C.c_int32),
        ("max_norm", C.c_int32), ("redundancy", C.c_int32), ("pooling_size", C.c_int32),
        ("continues_pooling", C.c_int32), ("sink_len", C.c_int32), ("decay_factor", C.c_float),
        ("redundancy_lambda", C.c_float), ("redundancy_one_minus_lambda", C.c_float),
        ("redundancy_temperature", C.c_float), ("redundancy_threshold", C.c_float),
        ("softmax_scale", C.c_float),
    ]


_P, _I, _L, _F, _Z = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/zipage_b200.h one to one
SIGNATURES = {
    "zp_last_error": (C.c_char_p, []),
    "zp_version": (_I, []),
    "zp_device_error": (_I, [C.POINTER(C.c_int), _I]),
    "zp_device_error_async": (_I, [_P, _P]),
    "zp_store_kv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _I, _P]),
    "zp_store_query": (_I, [_P, _P, _P, _I, _I, _I, _L, _L, _L, _I, _P, _I, _I, _I, _P]),
    "zp_window_score": (_I, [_P, _P, _P, _P, _P, _P] + [_I] * 8 + [_L] * 4 + [_F, _I, _I, _I, _P]),
    "zp_window_score_workspace_bytes": (_Z, [_I] * 6),
    "zp_window_score_ws": (_I, [_P, _P, _P, _P, _P, _P] + [_I] * 8 + [_L] * 4 + [_F, _I, _I, _I, _P, _Z, _P]),
    "zp_global_score": (_I, [_P, _P, _P, _P] + [_I] * 5 + [_L, _L, _F, _I, _I, _I, _P]),
    "zp_key_norm": (_I, [_P, _P, _P] + [_I] * 6 + [_L, _L, _F, _I, _P]),
    "zp_redundancy_lightning": (_I, [_P, _P, _P] + [_I] * 6 + [_L, _L, _F, _I, _I, _P]),
    "zp_redundancy_exact_workspace_bytes": (_Z, [_I] * 5),
    "zp_redundancy_exact": (_I, [_P, _P, _P] + [_I] * 6 + [_L, _L, _F, _I, _I, _P, _Z, _P]),
    "zp_redundancy_softmax": (_I, [_P, _P] + [_I] * 5 + [_F, _I, _I, _P]),
    "zp_select": (_I, [_P, _P, _P, _P, _P, _P] + [_I] * 5 + [C.POINTER(SelectParams), _I, _P]),
    "zp_compact": (_I, [_P, _P, _P, _P, _P, _P] + [_I] * 7 + [_L] * 4 + [_I, _P]),
    "zp_compress_batch_workspace_bytes": (_Z, [_I] * 7),
    "zp_compress_batch": (_I, [_P] * 11 + [_I] * 9 + [_L] * 6 + [C.POINTER(CompressParams), _I, _I, _P, _Z, _P]),
    "zp_update_tables": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "zp_paged_decode_workspace_bytes": (_Z, [_I] * 4),
    "zp_paged_decode": (_I, [_P] * 6 + [_I] * 6 + [_L, _F, _I, _P, _Z, _P]),
    "zp_paged_decode_noalloc_max_scratch_bytes": (_Z, []),
    "zp_paged_decode_noalloc": (_I, [_P] * 6 + [_I] * 6 + [_L, _F, _I, _P]),
    "zp_varlen_prefill": (_I, [_P] * 7 + [_I] * 7 + [_L, _F, _I, _P]),
    "zp_varlen_prefill_ex": (_I, [_P] * 7 + [_I] * 7 + [_L, _F, _I, _I, _I, _I, _P]),
    "zp_rms_norm": (_I, [_P] * 5 + [_I, _I, _L, _L, _F, _I, _P]),
    "zp_silu_and_mul": (_I, [_P, _P, _I, _I, _I, _P]),
    "zp_qk_norm_rope_store": (_I, [_P] * 5 + [_F] + [_P] * 7 + [_I, _P] + [_I] * 4 + [_L] * 3 + [_I, _P]),
    "zp_sample": (_I, [_P, _P, _P, _P, _I, _I, C.c_uint64, _I, _P]),
    "zp_prepare_decode": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "zp_comm_create": (_I, [_I, _I, _Z, _I, C.POINTER(_P)]),
    "zp_comm_segment": (_I, [_P, C.POINTER(_P), C.POINTER(_Z)]),
    "zp_comm_ipc_handle": (_I, [_P, _P]),
    "zp_comm_open_peer": (_I, [_P, _I, _P]),
    "zp_comm_attach_peer": (_I, [_P, _I, _P]),
    "zp_comm_status": (_I, [_P, C.POINTER(C.c_int)]),
    "zp_comm_destroy": (_I, [_P]),
    "zp_all_reduce": (_I, [_P, _P, _P, _L, _I, _I, _P]),
    "zp_all_reduce_add_rms_norm": (_I, [_P] * 6 + [_L, _I, _F, _I, _I, _P]),
    "zp_all_reduce_emulated": (_I, [_P, _I, _P, _P, _P, _P, _P, _L, _I, _F, _I, _I, _I, _P]),
    "zp_sample_sharded_emulated": (_I, [_P, _I, _P, _P, _P, _P, _I, _I, C.c_uint64, _I, _P]),
    "zp_sample_sharded": (_I, [_P, _P, _P, _P, _P, _I, _I, C.c_uint64, _I, _P]),
}

_lib = None


def load():
    """Load the shared library once; raise (never fall back) when it is missing."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ZipageError(
                f"{LIB_PATH} is missing: build it with `python -m zipage_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int, what: str = ""):
    if rc != 0:
        msg = load().zp_last_error().decode(errors="replace")
        raise ZipageError(f"{what or 'zipage_b200'} failed ({rc}): {msg}")


def device_error(reset=True) -> int:
    """Error word raised by a tcgen05 kernel whose bounded wait ran out (0 = none); synchronises."""
    code = C.c_int(0)
    check(load().zp_device_error(C.byref(code), int(reset)), "zp_device_error")
    return code.value


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return ZP_DTYPE[t.dtype]
    except KeyError:
        raise ZipageError(f"unsupported cache dtype {t.dtype}") from None


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ZipageError("zipage_b200 kernels need CUDA tensors (no CPU path exists)")
