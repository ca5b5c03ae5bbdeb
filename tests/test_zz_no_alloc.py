"""zp_paged_decode_noalloc: the decode entry point for hosts that must not allocate device memory
while decoding (all free memory already belongs to the KV cache; no cudaMalloc stalls allowed).
Its split-KV scratch is an array built into the library instead of a caller workspace.

Checked through the C ABI against zp_paged_decode on the same inputs, twice in a row (the array is
shared between calls and keeps the previous call's contents), and with a batch that is too large
for the built-in array.  Collected last on purpose."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BS = 256


def _case(seed, B, Hq, Hkv, dtype, dev):
    g = torch.Generator().manual_seed(seed)
    P, NBmax, D = 24, 9, 128
    kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    lens = torch.randint(300, NBmax * BS + 1, (B,), generator=g).to(torch.int32)
    table = torch.full((B, NBmax), -1, dtype=torch.int32)
    for b in range(B):
        n = (int(lens[b]) + BS - 1) // BS
        table[b, :n] = torch.randperm(P, generator=g)[:n].to(torch.int32)
    q = torch.randn(B, Hq, D, generator=g).to(dtype).to(dev)
    return q, kc, vc, lens.to(dev), table.to(dev)


def _call(lib, noalloc, q, kc, vc, lens, table, ws=None):
    from zipage_b200 import _lib as L
    B, Hq, D = q.shape
    Hkv = kc.shape[2]
    out = torch.empty_like(q)
    common = (L.ptr(q), L.ptr(kc), L.ptr(vc), L.ptr(lens), L.ptr(table), L.ptr(out), B,
              table.shape[1], Hq, Hkv, D, BS, kc.stride(0), float(D ** -0.5), L.dtype_code(q))
    if noalloc:
        rc = lib.zp_paged_decode_noalloc(*common, L.stream_ptr())
    else:
        rc = lib.zp_paged_decode(*common, L.ptr(ws), ws.numel(), L.stream_ptr())
    return rc, out


def test_noalloc_decode_matches_workspace_decode_twice():
    from zipage_b200 import _lib as L
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = L.load()
    assert lib.zp_paged_decode_noalloc_max_scratch_bytes() == 4 << 20
    ws = torch.empty(lib.zp_paged_decode_workspace_bytes(8, 32, 128, 32), dtype=torch.uint8, device=dev)
    # small batches: the kernel splits each sequence's keys over several blocks, so scratch is used
    cases = [_case(100, 2, 8, 2, torch.bfloat16, dev), _case(101, 3, 32, 8, torch.float32, dev)]
    refs = []
    for c in cases:
        rc, ref = _call(lib, False, *c, ws)
        assert rc == 0, lib.zp_last_error()
        refs.append(ref)
    # two calls in a row on different inputs, then the first again: the shared array still holds
    # the previous call's partials each time
    for idx in (0, 1, 0):
        rc, new = _call(lib, True, *cases[idx])
        torch.cuda.synchronize()
        assert rc == 0, lib.zp_last_error()
        # same kernels and same split choice as the workspace entry point: identical bits
        assert torch.equal(new, refs[idx])
        # and directly against the CPU oracle's softmax attention, within the tolerance the decode
        # tests use (2e-2 of the largest output for bf16, 1e-3 for fp32)
        from oracle import zipage_oracle as O
        q, kc, vc, lens, table = (t.cpu() for t in cases[idx])
        want = O.paged_decode_attention(q.unsqueeze(1), kc, vc, lens, table).squeeze(1).float()
        tol = 1e-3 if q.dtype == torch.float32 else 2e-2
        assert (new.cpu().float() - want).abs().max() <= tol * want.abs().max()


def test_noalloc_decode_rejects_batches_beyond_the_builtin_scratch():
    from zipage_b200 import _lib as L
    dev = torch.device("cuda:0")
    lib = L.load()
    # 591 sequences x 1 kv head x 8 query heads: 2 splits x 8 heads x 130 floats each = 4.9 MB
    c = _case(7, 591, 8, 1, torch.bfloat16, dev)
    rc, _ = _call(lib, True, *c)
    assert rc == -4 and b"built-in" in lib.zp_last_error()
    # 300 such sequences fit (2 splits, 2.5 MB) and agree with the workspace entry point
    c = _case(8, 300, 8, 1, torch.bfloat16, dev)
    ws = torch.empty(lib.zp_paged_decode_workspace_bytes(300, 8, 128, 32), dtype=torch.uint8, device=dev)
    rc_new, new = _call(lib, True, *c)
    rc_ref, ref = _call(lib, False, *c, ws)
    torch.cuda.synchronize()
    assert rc_new == 0 and rc_ref == 0 and torch.equal(new, ref)
