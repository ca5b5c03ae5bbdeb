"""Peer-memory all-reduce: the bounded wait on one GPU, the collective itself on two."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


def _gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def test_wait_for_an_absent_peer_times_out_and_reports():
    """A communicator of world size 2 whose peer never launches: the flag it waits for is never
    set, the wait ends after the 50 ms limit, the status word says so, and the context works on."""
    import ctypes as C
    from zipage_b200 import _lib as L
    from zipage_b200.layers.step_ops import rms_norm
    dev = _gpu()
    lib = L.load()
    h = C.c_void_p()
    L.check(lib.zp_comm_create(0, 2, 1 << 20, 50, C.byref(h)), "create")
    try:
        p, n = C.c_void_p(), C.c_size_t()
        L.check(lib.zp_comm_segment(h, C.byref(p), C.byref(n)), "segment")
        absent = torch.zeros(n.value, dtype=torch.uint8, device=dev)   # stands for the peer's segment
        L.check(lib.zp_comm_attach_peer(h, 1, C.c_void_p(absent.data_ptr())), "attach")
        x = torch.ones(4096, dtype=torch.bfloat16, device=dev)
        code = C.c_int(-1)
        L.check(lib.zp_comm_status(h, C.byref(code)), "status")
        assert code.value == 0
        L.check(lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), x.numel(), L.dtype_code(x), 1, L.stream_ptr()), "all_reduce")
        torch.cuda.synchronize()
        L.check(lib.zp_comm_status(h, C.byref(code)), "status")
        assert code.value == 1   # ZP_COMM_TIMEOUT
        # this rank's flag did reach the peer's segment
        flags = absent[: 2 * 8 * 256 * 4].view(torch.int32)
        assert int(flags[0]) == 1
    finally:
        lib.zp_comm_destroy(h)
    y = rms_norm(torch.ones(4, 256, dtype=torch.bfloat16, device=dev),
                 torch.ones(256, dtype=torch.bfloat16, device=dev), 1e-6)
    assert torch.allclose(y.float(), torch.ones(4, 256, device=dev), atol=1e-2)


def test_argument_checks():
    import ctypes as C
    from zipage_b200 import _lib as L
    _gpu()
    lib = L.load()
    h = C.c_void_p()
    assert lib.zp_comm_create(0, 3, 1 << 20, 50, C.byref(h)) != 0      # world size
    assert lib.zp_comm_create(2, 2, 1 << 20, 50, C.byref(h)) != 0      # rank
    L.check(lib.zp_comm_create(1, 2, 4096, 50, C.byref(h)), "create")
    try:
        x = torch.ones(4096, dtype=torch.bfloat16, device="cuda:0")
        # peer 0 not attached; message larger than the areas; ragged size
        assert lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), 64, L.dtype_code(x), 0, L.stream_ptr()) != 0
        assert b"not attached" in lib.zp_last_error()
        assert lib.zp_comm_attach_peer(h, 1, L.ptr(x)) != 0               # itself
        L.check(lib.zp_comm_attach_peer(h, 0, L.ptr(x)), "attach")       # (never launched)
        assert lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), 4096, L.dtype_code(x), 0, L.stream_ptr()) != 0
        assert lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), 12, L.dtype_code(x), 0, L.stream_ptr()) != 0
    finally:
        lib.zp_comm_destroy(h)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_reduce_across_gpus(world):
    _gpu()
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(29731 + world), str(ROOT / "tests" / "tp_comm_worker.py")],
        capture_output=True, text=True, timeout=420, env=env)
    sys.stdout.write(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert all(f"rank {i} OK" in r.stdout for i in range(world))
    print([ln for ln in r.stdout.splitlines() if ln.startswith("TPCOMM")])
