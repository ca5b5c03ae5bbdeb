"""GPU parity of the per-step ops (through the C ABI) against the reference fixtures and the oracle."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))
from step_cases import CASE, DTYPES, build_step_inputs, decode_state, from_np  # noqa: E402

pytestmark = pytest.mark.gpu


def _gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _load(name, dtype):
    z = np.load(ROOT / "tests" / "golden" / f"step_ops_{name}.npz")
    return {k: from_np(z[k], dtype) for k in z.files}


def _close(a, b, dtype, what):
    """fp32: a few ulps (the reductions sum in a different order); 16-bit: identical up to one
    rounding step of T in a small fraction of the elements (the same cause)."""
    a, b = a.float().cpu(), b.float().cpu()
    if dtype == torch.float32:
        assert torch.allclose(a, b, rtol=3e-6, atol=1e-6), what
    else:
        step = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)   # one unit in the last place, at most
        diff = (a - b).abs()
        assert (diff <= step * b.abs().clamp_min(1e-3) * 1.01).all(), what
        assert (diff > 0).float().mean() < 0.01, (what, (diff > 0).float().mean())


@pytest.mark.parametrize("name", list(DTYPES))
def test_elementwise_ops_match_reference_fixtures(name):
    from zipage_b200.layers import step_ops as P
    dev, dt, c = _gpu(), DTYPES[name], CASE
    inp = {k: v.to(dev) for k, v in build_step_inputs(dt).items()}
    ref = _load(name, dt)
    _close(P.rms_norm(inp["x"], inp["w_hidden"], c["eps"]), ref["rms"], dt, "rms_norm")
    y, res = P.rms_norm(inp["x"], inp["w_hidden"], c["eps"], residual=inp["residual"])
    _close(y, ref["add_rms"], dt, "add_rms_norm")
    want_res = (inp["x"].float() + inp["residual"].float()).to(dt).cpu()   # (fp32 fixture: aliased, see the oracle test)
    assert torch.equal(res.cpu(), want_res if dt == torch.float32 else ref["add_rms_residual"])
    _close(P.silu_and_mul(inp["gate_up"]), ref["silu_mul"], dt, "silu_and_mul")
    cache = P.rope_cos_sin_cache(c["D"], c["max_position"], c["rope_base"], dev)
    q, k, v = P.qk_norm_rope_store(inp["qkv"], inp["positions"], cache, inp["w_q"], inp["w_k"], c["eps"],
                                   c["Hq"], c["Hkv"], c["D"])
    _close(q, ref["q_rot"], dt, "q norm+rope")
    _close(k, ref["k_rot"], dt, "k norm+rope")
    tok = P.sample(inp["logits"], inp["temperatures"], noise=ref["noise"].float().to(dev))
    assert torch.equal(tok.cpu(), ref["tokens"].long())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_qk_store_writes_caches_and_window(dtype):
    """The fused launch against the oracle's q/k plus plain copies: K/V rows at their slots
    (slot -1 skipped), window queries at their triples, everything else untouched."""
    from oracle import step_ops_oracle as S
    from zipage_b200.layers import step_ops as P
    dev = _gpu()
    g = torch.Generator().manual_seed(3)
    N, Hq, Hkv, D, QCL, C, pages = 37, 8, 2, 128, 16, 6, 5
    qkv = (torch.randn(N, (Hq + 2 * Hkv) * D, generator=g) * 1.3).to(dtype)
    wq = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    wk = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)
    pos = torch.randint(0, 4096, (N,), generator=g)
    cache = S.rope_cos_sin_cache(D, 4096, 1e6)
    slots = torch.randperm(pages * 256, generator=g)[:N].to(torch.int32)
    slots[5] = -1
    trip = torch.tensor([[2, 1, 0], [9, 4, 15], [30, 0, 7]], dtype=torch.int32)
    qo, ko, vo = S.qk_norm_rope(qkv, pos, cache, wq, wk, 1e-6, Hq, Hkv, D)
    kc = torch.full((pages * 256, Hkv, D), 7.0, dtype=dtype, device=dev)
    vc = torch.full((pages * 256, Hkv, D), 7.0, dtype=dtype, device=dev)
    qc = torch.full((C, QCL, Hq, D), 7.0, dtype=dtype, device=dev)
    q, k, v = P.qk_norm_rope_store(qkv.to(dev), pos.to(dev), cache.to(dev), wq.to(dev), wk.to(dev), 1e-6,
                                   Hq, Hkv, D, k_cache=kc, v_cache=vc, slot_mapping=slots.to(dev),
                                   query_cache=qc, query_slot_mapping=trip.to(dev))
    _close(q, qo, dtype, "q")
    _close(k, ko, dtype, "k")
    assert torch.equal(v.cpu(), vo)
    keep = slots != -1
    assert torch.equal(kc[slots[keep].long()].cpu(), k.cpu()[keep])
    assert torch.equal(vc[slots[keep].long()].cpu(), vo[keep])
    untouched = torch.ones(pages * 256, dtype=torch.bool)
    untouched[slots[keep].long()] = False
    assert (kc.cpu()[untouched] == 7.0).all() and (vc.cpu()[untouched] == 7.0).all()
    for row, qid, idx in trip.tolist():
        assert torch.equal(qc[qid, idx].cpu(), q[row].cpu())
    mask = torch.ones(C, QCL, dtype=torch.bool)
    for _, qid, idx in trip.tolist():
        mask[qid, idx] = False
    assert (qc.cpu()[mask] == 7.0).all()


def test_rms_norm_in_place_and_model_sizes():
    """Qwen3-8B hidden size, in-place residual update (residual_out = the residual buffer) and a
    strided input, against the oracle."""
    from oracle import step_ops_oracle as S
    from zipage_b200 import _lib as L
    dev = _gpu()
    g = torch.Generator().manual_seed(11)
    N, H = 33, 4096
    big = torch.randn(N, H + 64, generator=g).to(torch.bfloat16)
    x = big[:, :H]                      # row stride H + 64
    res = (3 * torch.randn(N, H, generator=g)).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    want, want_res = S.add_rms_norm(x, res, w, 1e-6)
    xd, rd, wd = big.to(dev)[:, :H], res.to(dev), w.to(dev)
    out = torch.empty(N, H, dtype=torch.bfloat16, device=dev)
    L.check(L.load().zp_rms_norm(L.ptr(xd), L.ptr(rd), L.ptr(wd), L.ptr(out), L.ptr(rd), N, H, xd.stride(0),
                                 H, 1e-6, L.dtype_code(xd), L.stream_ptr()))
    assert torch.equal(rd.cpu(), want_res)
    _close(out, want, torch.bfloat16, "add_rms_norm 4096")


def test_sampler_race_properties():
    """Full vocabulary: with the oracle's noise the same tokens; with the built-in generator the
    empirical distribution of many draws follows softmax(logits / T), and greedy-like temperature
    picks the arg-max."""
    from oracle import step_ops_oracle as S
    from zipage_b200.layers import step_ops as P
    dev = _gpu()
    g = torch.Generator().manual_seed(5)
    B, V = 6, 151936
    logits = (2.5 * torch.randn(B, V, generator=g)).to(torch.bfloat16)
    temps = torch.tensor([0.6, 1.0, 0.3, 1.5, 0.6, 1.0])
    noise = torch.empty(B, V).exponential_(1, generator=g)
    want = S.sample_race(logits, temps, noise)
    got = P.sample(logits.to(dev), temps.to(dev), noise=noise.to(dev))
    assert torch.equal(got.cpu(), want)
    # the built-in draws: a small vocabulary, many rows with the same logits
    V2, R = 8, 40000
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -0.5, -1.0, -2.0, 1.5])
    lg = row.repeat(R, 1).to(torch.bfloat16).to(dev)
    tk = P.sample(lg, torch.full((R,), 0.8, device=dev), seed=77)
    freq = torch.bincount(tk.cpu(), minlength=V2).float() / R
    p = torch.softmax(row.to(torch.bfloat16).float() / 0.8, 0)
    assert (freq - p).abs().max() < 0.01
    cold = P.sample(lg[:16], torch.full((16,), 1e-3, device=dev), seed=3)
    assert (cold.cpu() == 0).all()


def test_prepare_decode_matches_reference_fixture():
    from zipage_b200.layers import step_ops as P
    dev = _gpu()
    st = decode_state()
    z = np.load(ROOT / "tests" / "golden" / "prepare_decode.npz")
    tables = torch.from_numpy(z["block_tables"]).to(dev)
    pos, ctx, slot, trip, n = P.prepare_decode(
        torch.tensor(st["num_tokens"], dtype=torch.int32, device=dev), tables,
        torch.tensor(st["query_ids"], dtype=torch.int32, device=dev), st["query_cache_len"])
    assert np.array_equal(pos.cpu().numpy(), z["positions"])
    assert np.array_equal(ctx.cpu().numpy(), z["context_lens"])
    assert np.array_equal(slot.cpu().numpy(), z["slot_mapping"])
    k = int(n.item())
    assert k == len(z["triples"]) and np.array_equal(trip[:k].cpu().numpy(), z["triples"])


def test_prepare_decode_large_batch_against_oracle():
    """More sequences than one pass of the block handles; the triples keep sequence order."""
    from oracle import step_ops_oracle as S
    from zipage_b200.layers import step_ops as P
    dev = _gpu()
    rs = np.random.RandomState(9)
    B = 2500
    lens = rs.randint(1, 12, size=B)
    tables = [list(rs.randint(0, 10000, size=int(n))) for n in lens]
    num_tokens = [int((n - 1) * 256 + rs.randint(1, 257)) + int(rs.randint(0, 3)) * 256 for n in lens]
    qids = [int(q) for q in rs.randint(-1, 64, size=B)]
    pos, ctx, slot, padded, trip = S.prepare_decode(num_tokens, tables, qids, 32)
    gp, gc, gs, gt, gn = P.prepare_decode(torch.tensor(num_tokens, dtype=torch.int32, device=dev),
                                          padded.to(dev), torch.tensor(qids, dtype=torch.int32, device=dev), 32)
    assert torch.equal(gp.cpu(), pos) and torch.equal(gc.cpu(), ctx) and torch.equal(gs.cpu(), slot)
    k = int(gn.item())
    assert k == len(trip) and torch.equal(gt[:k].cpu(), trip)


def test_decode_step_without_host_lists():
    """prepare_decode -> fused q/k kernel with the triple count left on the device: the window
    rows of exactly the sequences inside their observation window are written, nothing else."""
    from oracle import step_ops_oracle as S
    from zipage_b200.layers import step_ops as P
    dev = _gpu()
    st = decode_state()
    B, Hq, Hkv, D, QCL = len(st["num_tokens"]), 4, 2, 128, st["query_cache_len"]
    g = torch.Generator().manual_seed(2)
    width = max(len(t) for t in st["block_tables"])
    tables = torch.tensor([t + [-1] * (width - len(t)) for t in st["block_tables"]], dtype=torch.int32, device=dev)
    pos, ctx, slot, trip, ntrip = P.prepare_decode(
        torch.tensor(st["num_tokens"], dtype=torch.int32, device=dev), tables,
        torch.tensor(st["query_ids"], dtype=torch.int32, device=dev), QCL)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16)
    w = torch.ones(D, dtype=torch.bfloat16)
    cache = S.rope_cos_sin_cache(D, 8192, 1e6)
    pages = int(tables.max()) + 1
    kc = torch.zeros((pages * 256, Hkv, D), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    qc = torch.full((8, QCL, Hq, D), 7.0, dtype=torch.bfloat16, device=dev)
    q, _, _ = P.qk_norm_rope_store(qkv.to(dev), pos, cache.to(dev), w.to(dev), w.to(dev), 1e-6, Hq, Hkv, D,
                                   k_cache=kc, v_cache=vc, slot_mapping=slot, query_cache=qc,
                                   query_slot_mapping=trip, query_slot_count=ntrip, return_k=False)
    _, _, _, _, want = S.prepare_decode(st["num_tokens"], st["block_tables"], st["query_ids"], QCL)
    mask = torch.ones(8, QCL, dtype=torch.bool)
    for row, qid, idx in want.tolist():
        assert torch.equal(qc[qid, idx].cpu(), q[row].cpu())
        mask[qid, idx] = False
    assert (qc.cpu()[mask] == 7.0).all()
    assert (kc[slot.long()].float().abs().sum(dim=(1, 2)) > 0).all()   # every sequence's K row was stored
