"""The C-ABI library builds, loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared(header="zipage_b200.h"):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from zipage_b200.build import build
    lib_path = build()
    lib = ctypes.CDLL(str(lib_path))
    names = _declared()
    assert len(names) >= 15
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    lib.zp_version.restype = ctypes.c_int
    assert lib.zp_version() >= 1


def test_binding_table_matches_header():
    from zipage_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    _lib.load()


def test_host_control_plane_header_library_and_binding_agree():
    from zipage_b200 import _hostlib
    from zipage_b200.build import build
    names = _declared("zipage_b200_host.h")
    assert len(names) >= 15 and sorted(_hostlib.SIGNATURES) == names
    lib = ctypes.CDLL(str(build()))
    assert not [n for n in names if not hasattr(lib, n)]
    _hostlib.load()


def test_every_header_is_covered():
    assert sorted(p.name for p in (ROOT / "include").glob("*.h")) == ["zipage_b200.h", "zipage_b200_host.h"]


def test_argument_errors_are_reported_without_a_gpu():
    from zipage_b200 import _lib
    lib = _lib.load()
    rc = lib.zp_store_kv(None, None, None, None, None, 4, 8, 128, 1024, 1024, 0, None)
    assert rc == -1 and b"null" in lib.zp_last_error()
    assert lib.zp_store_kv(None, None, None, None, None, 0, 8, 128, 1024, 1024, 0, None) == 0
