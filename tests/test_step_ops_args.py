"""Argument checking of the per-step entry points: every rejection happens before any CUDA call,
so it can be exercised without a GPU (no kernel is launched by these tests)."""
import ctypes as C
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from zipage_b200 import _lib as L  # noqa: E402

INVALID = -1


def _err(lib):
    return lib.zp_last_error().decode()


def test_rms_norm_rejects_bad_arguments():
    lib = L.load()
    assert lib.zp_rms_norm(None, None, None, None, None, 0, 4096, 4096, 4096, 1e-6, 0, None) == 0  # empty batch
    assert lib.zp_rms_norm(None, None, None, None, None, 4, 4096, 4096, 4096, 1e-6, 0, None) == INVALID
    assert "null pointer" in _err(lib)
    p = C.c_void_p(4096)
    assert lib.zp_rms_norm(p, None, p, p, p, 4, 4096, 4096, 4096, 1e-6, 0, None) == INVALID   # residual_out without residual
    assert lib.zp_rms_norm(p, None, p, p, None, 4, 4100, 4100, 4100, 1e-6, 0, None) == INVALID  # not a multiple of 8 elements
    assert lib.zp_rms_norm(C.c_void_p(4098), None, p, p, None, 4, 4096, 4096, 4096, 1e-6, 0, None) == INVALID
    assert "aligned" in _err(lib)
    assert lib.zp_rms_norm(p, None, p, p, None, 4, 1 << 20, 1 << 20, 1 << 20, 1e-6, 0, None) == INVALID
    assert "too large" in _err(lib)
    assert lib.zp_rms_norm(p, None, p, p, None, 4, 4096, 4096, 4096, 1e-6, 7, None) == INVALID   # dtype code


def test_other_step_ops_reject_bad_arguments():
    lib = L.load()
    p = C.c_void_p(4096)
    assert lib.zp_silu_and_mul(None, None, 0, 128, 0, None) == 0
    assert lib.zp_silu_and_mul(None, p, 3, 128, 0, None) == INVALID
    assert lib.zp_silu_and_mul(p, p, 3, 100, 0, None) == INVALID          # 100 bf16 is not whole vectors
    args = lambda **kw: [kw.get("qkv", p), p, p, p, p, 1e-6, kw.get("q_out", p), None, kw.get("kc"), kw.get("vc"),
                         kw.get("slots"), kw.get("qc"), kw.get("trip"), kw.get("ntrip", 0), None, kw.get("n", 5), 8, 2,
                         kw.get("D", 128), 1536, 0, 0, 0, None]
    assert lib.zp_qk_norm_rope_store(*args(n=0)) == 0
    assert lib.zp_qk_norm_rope_store(*args(q_out=None)) == INVALID
    assert lib.zp_qk_norm_rope_store(*args(slots=p)) == INVALID             # slot mapping without caches
    assert lib.zp_qk_norm_rope_store(*args(ntrip=2)) == INVALID             # triples without a window buffer
    assert lib.zp_qk_norm_rope_store(*args(D=96)) == INVALID
    assert "head_dim" in _err(lib)
    assert lib.zp_qk_norm_rope_store(*args(qkv=C.c_void_p(4100))) == INVALID
    assert lib.zp_sample(None, None, None, None, 0, 1000, 0, 0, None) == 0
    assert lib.zp_sample(p, None, None, p, 2, 1000, 0, 0, None) == INVALID
    assert lib.zp_sample(p, p, None, p, 2, 0, 0, 0, None) == INVALID
    assert lib.zp_prepare_decode(p, p, p, 3, 9, 32, 256, p, p, p, p, None, None) == INVALID
    assert lib.zp_prepare_decode(None, p, p, 3, 9, 32, 256, p, p, p, p, p, None) == INVALID
    assert lib.zp_prepare_decode(p, p, p, 3, 9, 300, 256, p, p, p, p, p, None) == INVALID  # window longer than a page
