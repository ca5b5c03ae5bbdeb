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


def _absent_peer_comm(lib, L, C, dev, max_bytes, timeout_ms):
    """A world-2 communicator on one GPU whose peer is a zeroed buffer that nothing ever writes."""
    h = C.c_void_p()
    L.check(lib.zp_comm_create(0, 2, max_bytes, timeout_ms, C.byref(h)), "create")
    p, n = C.c_void_p(), C.c_size_t()
    L.check(lib.zp_comm_segment(h, C.byref(p), C.byref(n)), "segment")
    absent = torch.zeros(n.value, dtype=torch.uint8, device=dev)
    L.check(lib.zp_comm_attach_peer(h, 1, C.c_void_p(absent.data_ptr())), "attach")
    return h, absent


def _status(lib, L, C, h):
    code = C.c_int(-1)
    L.check(lib.zp_comm_status(h, C.byref(code)), "status")
    return code.value


@pytest.mark.parametrize("form", ["flagged_lines", "two_shot", "fused_flagged", "sampler"])
def test_absent_peer_costs_about_one_time_limit(form):
    """Host-injected failure (a peer that never launches), 50 ms limit, for the forms with many
    waits per thread: flagged lines (one wait per 16-byte vector and peer), the two meetings of
    the two-shot form, and the two exchange phases of the sharded sampler.  The first wait that
    runs out makes the failure sticky, so the whole call — and five more calls after it, as a
    replayed decode graph would issue — ends within a small multiple of ONE limit."""
    import ctypes as C
    import time
    from zipage_b200 import _lib as L
    dev = _gpu()
    lib = L.load()
    h, absent = _absent_peer_comm(lib, L, C, dev, 1 << 20, 50)
    try:
        rows, hidden = 64, 4096
        x = torch.ones(rows, hidden, dtype=torch.bfloat16, device=dev)
        res = torch.ones_like(x)
        wgt = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        logits = torch.randn(48, 3000, device=dev).to(torch.bfloat16)
        temps = torch.ones(48, device=dev)
        toks = torch.empty(48, dtype=torch.int64, device=dev)

        def call():
            if form == "flagged_lines":
                L.check(lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), x.numel(), L.dtype_code(x), 3, L.stream_ptr()), form)
            elif form == "two_shot":
                L.check(lib.zp_all_reduce(h, L.ptr(x), L.ptr(x), x.numel(), L.dtype_code(x), 2, L.stream_ptr()), form)
            elif form == "fused_flagged":
                L.check(lib.zp_all_reduce_add_rms_norm(h, L.ptr(x), L.ptr(res), L.ptr(wgt), L.ptr(x), L.ptr(res), rows,
                                                       hidden, 1e-6, L.dtype_code(x), 3, L.stream_ptr()), form)
            else:
                L.check(lib.zp_sample_sharded(h, L.ptr(logits), L.ptr(temps), None, L.ptr(toks), 48, 3000, 7,
                                              L.dtype_code(logits), L.stream_ptr()), form)

        assert _status(lib, L, C, h) == 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        call()
        torch.cuda.synchronize()
        first = time.perf_counter() - t0
        assert _status(lib, L, C, h) == 1          # ZP_COMM_TIMEOUT
        assert 0.04 < first < 0.5, first            # one limit, not one per wait
        t0 = time.perf_counter()
        for _ in range(5):
            call()
        torch.cuda.synchronize()
        later = time.perf_counter() - t0
        assert later < 0.05, later                  # the failure is sticky: no further waiting
        assert _status(lib, L, C, h) == 1
    finally:
        lib.zp_comm_destroy(h)
    y = torch.ones(8, device=dev) * 2              # the context keeps working
    assert float(y.sum()) == 16.0


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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_world_sizes_as_one_cooperative_launch(world):
    """Every rank of the world as blocks of one cooperative launch on one GPU (the per-rank code is
    the multi-GPU kernel's): bit-exact against the fp32 rank-order sum for both algorithms, over
    consecutive calls, and the fused residual + RMSNorm form against the RMSNorm kernel."""
    import ctypes as C
    from zipage_b200 import _lib as L
    from zipage_b200.layers.step_ops import rms_norm
    dev = _gpu()
    lib = L.load()
    comms = []
    try:
        for r in range(world):
            h = C.c_void_p()
            L.check(lib.zp_comm_create(r, world, 1 << 20, 2000, C.byref(h)), "create")
            comms.append(h)
        segs = []
        for h in comms:
            p, n = C.c_void_p(), C.c_size_t()
            L.check(lib.zp_comm_segment(h, C.byref(p), C.byref(n)), "segment")
            segs.append(p)
        for r, h in enumerate(comms):
            for q in range(world):
                if q != r:
                    L.check(lib.zp_comm_attach_peer(h, q, segs[q]), "attach")
        arr = (C.c_void_p * world)(*[h.value for h in comms])
        g = torch.Generator(device=dev).manual_seed(world)

        def ptrs(ts):
            return (C.c_void_p * world)(*[t.data_ptr() for t in ts])

        for dtype in (torch.bfloat16, torch.float32):
            for rows, elems in ((40, 1024), (3, 4096 if dtype == torch.float32 else 8192), (300, 512)):
                for algo in (1, 2, 3):
                    for _ in range(3):      # consecutive calls alternate the areas
                        xs = [torch.randn(rows, elems, device=dev, generator=g).to(dtype) for _ in range(world)]
                        outs = [torch.empty_like(x) for x in xs]
                        L.check(lib.zp_all_reduce_emulated(arr, world, ptrs(xs), ptrs(outs), None, None, None, rows,
                                                           elems, 0.0, L.dtype_code(xs[0]), algo, 0, L.stream_ptr()),
                                "emulated")
                        acc = xs[0].float()
                        for x in xs[1:]:
                            acc = acc + x.float()
                        want = acc.to(dtype)
                        for o in outs:
                            assert torch.equal(o, want), (world, dtype, rows, elems, algo)
                    # fused form
                    res = torch.randn(rows, elems, device=dev, generator=g).to(dtype)
                    w = (1 + 0.1 * torch.randn(elems, device=dev, generator=g)).to(dtype)
                    res_outs = [torch.empty_like(res) for _ in range(world)]
                    L.check(lib.zp_all_reduce_emulated(arr, world, ptrs(xs), ptrs(outs), L.ptr(res), L.ptr(w),
                                                       ptrs(res_outs), rows, elems, 1e-6, L.dtype_code(res), algo, 1,
                                                       L.stream_ptr()), "emulated fused")
                    y0, r0 = rms_norm(want, w, 1e-6, res)
                    for o, ro in zip(outs, res_outs):
                        assert torch.equal(ro, r0)
                        if dtype == torch.float32:
                            assert torch.allclose(o, y0, rtol=3e-6, atol=1e-6)
                        else:
                            d = (o.float() - y0.float()).abs()
                            assert (d <= 2.0 ** -7 * y0.float().abs().clamp_min(1e-3)).all()
                            assert (d > 0).float().mean() < 0.01
        torch.cuda.synchronize()
        for h in comms:
            code = C.c_int(-1)
            L.check(lib.zp_comm_status(h, C.byref(code)), "status")
            assert code.value == 0
    finally:
        for h in comms:
            lib.zp_comm_destroy(h)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_sampler_world_sizes_as_one_cooperative_launch(world):
    """The sharded sampler for every rank of the world in one cooperative launch on one GPU: every
    rank's tokens == the single-GPU sampler on the concatenated logits == the CPU oracle."""
    import ctypes as C
    from oracle import step_ops_oracle as S
    from zipage_b200 import _lib as L
    from zipage_b200.layers.step_ops import sample
    dev = _gpu()
    lib = L.load()
    comms = []
    try:
        for r in range(world):
            h = C.c_void_p()
            L.check(lib.zp_comm_create(r, world, 1 << 16, 2000, C.byref(h)), "create")
            comms.append(h)
        segs = []
        for h in comms:
            p, n = C.c_void_p(), C.c_size_t()
            L.check(lib.zp_comm_segment(h, C.byref(p), C.byref(n)), "segment")
            segs.append(p)
        for r, h in enumerate(comms):
            for q in range(world):
                if q != r:
                    L.check(lib.zp_comm_attach_peer(h, q, segs[q]), "attach")
        arr = (C.c_void_p * world)(*[h.value for h in comms])
        for dtype, B, Vs in ((torch.bfloat16, 37, 2000), (torch.float32, 70, 1001), (torch.float16, 5, 18992)):
            torch.manual_seed(3 + world)
            V = Vs * world
            full = (3 * torch.randn(B, V)).to(dtype).to(dev)
            temps = (0.3 + torch.rand(B)).to(dev)
            draws = torch.empty(B, V).exponential_(1.0).to(dev)
            full[3, 5] = full[3, (world - 1) * Vs + 9] = 40.0     # an exact tie between the first and the last shard
            draws[3, 5] = draws[3, (world - 1) * Vs + 9] = 0.5
            shards = [full[:, r * Vs:(r + 1) * Vs].contiguous() for r in range(world)]
            nshards = [draws[:, r * Vs:(r + 1) * Vs].contiguous() for r in range(world)]
            outs = [torch.empty(B, dtype=torch.int64, device=dev) for _ in range(world)]

            def ptrs(ts):
                return (C.c_void_p * world)(*[t.data_ptr() for t in ts])

            L.check(lib.zp_sample_sharded_emulated(arr, world, ptrs(shards), L.ptr(temps), ptrs(nshards), ptrs(outs), B,
                                                   Vs, 0, L.dtype_code(full), L.stream_ptr()), "emulated sampler")
            want = sample(full, temps, noise=draws)
            assert torch.equal(want.cpu(), S.sample_race(full.cpu(), temps.cpu(), draws.cpu()))
            for o in outs:
                assert torch.equal(o, want), (world, dtype, B, Vs)
            assert int(want[3]) == 5
            L.check(lib.zp_sample_sharded_emulated(arr, world, ptrs(shards), L.ptr(temps), None, ptrs(outs), B, Vs, 11,
                                                   L.dtype_code(full), L.stream_ptr()), "emulated sampler, generator")
            want = sample(full, temps, seed=11)
            for o in outs:
                assert torch.equal(o, want), (world, dtype, B, Vs, "generator")
        for h in comms:
            code = C.c_int(-1)
            L.check(lib.zp_comm_status(h, C.byref(code)), "status")
            assert code.value == 0
    finally:
        for h in comms:
            lib.zp_comm_destroy(h)
