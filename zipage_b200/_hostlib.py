"""ctypes binding of the host control plane (the C ABI declared in include/zipage_b200_host.h).

Same shared library as the kernels, but nothing here needs torch or a GPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libzipage_b200.so"


class SchedulerError(RuntimeError):
    pass


class SchedConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_blocks", "block_size", "max_blocks_per_seq", "enable_prefix_cache", "max_num_seqs",
        "max_num_batched_tokens", "eos", "max_concurrency", "enable_hybrid_engine", "query_cache_len")]


_P, _I, _D = C.c_void_p, C.c_int, C.c_double

# name -> (restype, argtypes); mirrors include/zipage_b200_host.h one to one
SIGNATURES = {
    "zp_sched_last_error": (C.c_char_p, []),
    "zp_sched_create": (_P, [C.POINTER(SchedConfig)]),
    "zp_sched_destroy": (None, [_P]),
    "zp_sched_add": (_I, [_P, _P, _I, C.c_float, _I, _I]),
    "zp_sched_schedule": (_I, [_P, _P, _I, _P]),
    "zp_sched_postprocess": (_I, [_P, _P, _I, _P, _D, _P]),
    "zp_sched_preempt": (_I, [_P, _I]),
    "zp_sched_mark_prefilled": (_I, [_P, _P, _I]),
    "zp_sched_release": (_I, [_P, _I]),
    "zp_sched_counts": (_I, [_P, _P]),
    "zp_sched_seq_info": (_I, [_P, _I, _P]),
    "zp_sched_seq_info_batch": (_I, [_P, _P, _I, _P]),
    "zp_sched_seq_times": (_I, [_P, _I, _P, _P]),
    "zp_sched_seq_set_num_cached": (_I, [_P, _I, _I]),
    "zp_sched_seq_list": (_I, [_P, _I, _I, _P, _I]),
    "zp_sched_queue": (_I, [_P, _I, _P, _I]),
    "zp_sched_block_info": (_I, [_P, _I, _P, _P]),
    "zp_sched_hash_tokens": (C.c_uint64, [_P, _I, _I, C.c_uint64]),
    "zp_sched_decode_inputs": (_I, [_P, _P, _I, _P, _P, _P, _P, _I]),
    "zp_sched_temperatures": (_I, [_P, _P, _I, _P]),
    "zp_sched_prefill_sizes": (_I, [_P, _P, _I, _P]),
    "zp_sched_prefill_inputs": (_I, [_P, _P, _I, _P, _P, _P, _P, _P, _P]),
    "zp_sched_compress_due": (_I, [_P, _P, _I, _P]),
    "zp_sched_compress_inputs": (_I, [_P, _P, _I, _P, _I, _P, _I, _P, _P]),
}

_lib = None


def load():
    """Load the shared library once; raise when it is missing (there is no Python fallback)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise SchedulerError(f"{LIB_PATH} is missing: build it with `python -m zipage_b200.build`")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> int:
    """Negative return codes become exceptions: AssertionError where the reference asserts."""
    if rc < 0:
        msg = load().zp_sched_last_error().decode(errors="replace")
        raise (AssertionError if rc == -2 else SchedulerError)(f"{what} failed ({rc}): {msg}")
    return rc
