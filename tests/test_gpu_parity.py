"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the golden fixtures."""
from pathlib import Path

import numpy as np
import pytest
import torch

from cases import BS, CASES, build_inputs, tensor_sha

pytestmark = pytest.mark.gpu

GOLD = Path(__file__).resolve().parent / "golden"


def _gpu():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    return torch.device("cuda:0")


def _unpack(bits, shape):
    return torch.from_numpy(np.unpackbits(bits, axis=-1)[..., : shape[-1]].astype(bool)).view(shape)


def _cfgs(case):
    from oracle import zipage_oracle as O
    from zipage_b200.compress import CompressConfig
    return O.CompressConfig(**case["cfg"]), CompressConfig(**case["cfg"])


def _run_gpu(case, inp, dtype, impl="auto"):
    from zipage_b200.compress import compress_chunk
    dev = _gpu()
    _, cfg = _cfgs(case)
    k, v, q = (inp[n].to(dtype).to(dev) for n in ("k", "v", "q"))
    sc = inp["score_cache"].to(dtype).to(dev) if cfg.use_global_score else None
    from zipage_b200 import kernel as K
    att = K.attention_score(k, q, inp["query_ids"].to(dev), inp["block_tables"].to(dev), impl=impl)
    dbg = compress_chunk(k, v, q, sc, inp["query_ids"].to(dev), inp["block_tables"].to(dev),
                         inp["targets"].to(dev), inp["compressed"].to(dev), cfg, impl=impl,
                         return_debug=True)
    torch.cuda.synchronize()
    return dict(att=att.cpu(), final=dbg["final"].cpu(), keep=dbg["keep"].cpu(),
                red_logits=None if dbg["red_logits"] is None else dbg["red_logits"].cpu(),
                k=k.cpu(), v=v.cpu(), sc=None if sc is None else sc.cpu())


def _run_oracle(case, inp, dtype):
    from oracle import zipage_oracle as O
    ocfg, _ = _cfgs(case)
    k, v, q = (inp[n].to(dtype).clone() for n in ("k", "v", "q"))
    sc = inp["score_cache"].to(dtype).clone() if ocfg.use_global_score else None
    att = O.attention_score(k, q, inp["query_ids"], inp["block_tables"])
    parts = {}
    final, keep = O.compress(k, v, q, sc, inp["query_ids"], inp["block_tables"], inp["targets"],
                             inp["compressed"], ocfg, parts=parts)
    return dict(att=att, final=final, keep=keep, k=k, v=v, sc=sc, parts=parts)


FP32_CASES = [n for n in CASES if CASES[n]["dtype"] == "float32"]


@pytest.mark.parametrize("name", FP32_CASES)
def test_fp32_matches_reference_fixture(name):
    """fp32: kept sets and compacted caches bit-exact with the reference's own run;
    scores within 1e-3 relative (the tolerance stated for fp32)."""
    case = CASES[name]
    g = np.load(GOLD / f"{name}.npz")
    inp = build_inputs(case)
    out = _run_gpu(case, inp, torch.float32)
    L, B, Hkv = case["L"], len(case["tables"]), case["Hkv"]
    NB = inp["block_tables"].shape[1]
    att_ref = torch.from_numpy(g["attention_score"])
    assert torch.allclose(out["att"], att_ref, rtol=1e-3, atol=1e-9)
    final_ref = torch.from_numpy(g["final_scores"]).view(L, B, Hkv, NB, BS)
    fin = torch.isfinite(final_ref)
    assert torch.equal(out["final"][~fin], final_ref[~fin])
    scale = final_ref[fin].abs().max()
    assert (out["final"][fin] - final_ref[fin]).abs().max() <= 1e-3 * scale
    keep_ref = _unpack(g["keep"], (L, B, Hkv, NB * BS)).view(L, B, Hkv, NB, BS)
    assert torch.equal(out["keep"], keep_ref)
    assert tensor_sha(torch.stack([out["k"], out["v"]])) == str(g["kv_after_sha"])
    if out["sc"] is not None:
        assert torch.allclose(out["sc"], torch.from_numpy(g["score_cache_after"]), rtol=1e-3, atol=1e-9)


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_16bit_matches_oracle(name, dtype):
    """16-bit caches: scores within 2e-2 relative of the oracle run in the same dtype; kept sets
    may differ only where scores sit within a rounding step of the cut."""
    case = CASES[name]
    inp = build_inputs(case)
    ref = _run_oracle(case, inp, dtype)
    out = _run_gpu(case, inp, dtype)
    a, b = out["att"].float(), ref["att"].float()
    assert (a - b).abs().max() <= 2e-2 * b.abs().max()
    fa, fb = out["final"].float(), ref["final"].float()
    fin = torch.isfinite(fb)
    assert torch.equal(fa[~fin], fb[~fin])
    assert (fa[fin] - fb[fin]).abs().max() <= 2e-2 * fb[fin].abs().max()
    # kept sets may differ only on indices whose score sits within one rounding step of the cut
    from oracle.boundary import kept_set_report
    L, B, Hkv = ref["keep"].shape[:3]
    rep = kept_set_report(ref["final"].reshape(L, B, Hkv, -1), ref["keep"].reshape(L, B, Hkv, -1),
                          out["keep"].reshape(L, B, Hkv, -1), BS * case["cfg"]["budget_blocks"], dtype,
                          ref["parts"])
    assert rep["outside"] == 0 and rep["mismatch"] < 1e-2, rep


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selection_and_compaction_are_bit_exact_given_scores(dtype):
    """Integer/index work: fed the oracle's selection scores, the GPU top-k returns the identical
    kept set (lowest index wins ties), and the GPU compaction of that set reproduces the oracle's
    caches bit for bit."""
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    dev = _gpu()
    case = CASES["recipe_lightning_fp32"]
    inp = build_inputs(case)
    ref = _run_oracle(case, inp, dtype)
    L, B, Hkv, NB = ref["final"].shape[:4]
    # coarse scores -> many exact ties, including at the cut
    g = torch.Generator().manual_seed(3)
    coarse = (torch.randint(0, 40, ref["final"].shape, generator=g).float() / 64).to(dtype)
    coarse[~torch.isfinite(ref["final"].float())] = ref["final"][~torch.isfinite(ref["final"].float())]
    k_top = BS * case["cfg"]["budget_blocks"]
    for scores in (ref["final"], coarse):
        want = O.topk_mask(scores.view(L, B, Hkv, -1), k_top)
        got = K.topk_mask(scores.view(L, B, Hkv, -1).to(dev), k_top).cpu()
        assert torch.equal(got, want)
    keep = O.topk_mask(coarse.view(L, B, Hkv, -1), k_top).view(L, B, Hkv, NB, BS)
    k1, v1 = inp["k"].to(dtype).clone(), inp["v"].to(dtype).clone()
    sc1 = inp["score_cache"].to(dtype).clone()
    O.compress_kv(k1, v1, keep, inp["block_tables"], inp["targets"])
    O.compress_score(sc1, keep, inp["block_tables"], inp["targets"])
    k2, v2, sc2 = (t.to(dtype).to(dev) for t in (inp["k"], inp["v"], inp["score_cache"]))
    K.compress_kv(k2, v2, keep.to(dev), inp["block_tables"].to(dev), inp["targets"].to(dev))
    K.compress_score(sc2, keep.to(dev), inp["block_tables"].to(dev), inp["targets"].to(dev))
    assert torch.equal(k2.cpu(), k1) and torch.equal(v2.cpu(), v1) and torch.equal(sc2.cpu(), sc1)


def test_store_kernels():
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    dev = _gpu()
    g = torch.Generator().manual_seed(0)
    P, Hkv, Hq, D, QCL, C, N = 5, 8, 32, 128, 16, 6, 37
    for dtype in (torch.bfloat16, torch.float32):
        key = torch.randn(N, Hkv, D, generator=g).to(dtype)
        val = torch.randn(N, Hkv, D, generator=g).to(dtype)
        kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
        vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
        slots = torch.randperm(P * BS, generator=g)[:N].to(torch.int32)
        slots[3] = -1
        slots[20] = -1
        kc2, vc2 = kc.to(dev), vc.to(dev)
        # strided source rows, as the q/k/v split of a fused projection gives
        packed = torch.cat([key, val], dim=1).to(dev)
        K.store_kvcache(packed[:, :Hkv], packed[:, Hkv:], kc2, vc2, slots.to(dev))
        O.store_kvcache(key, val, kc, vc, slots)
        assert torch.equal(kc2.cpu(), kc) and torch.equal(vc2.cpu(), vc)
        q = torch.randn(N, Hq, D, generator=g).to(dtype)
        qc = torch.zeros(C, QCL, Hq, D).to(dtype)
        triples = torch.tensor([[0, 2, 0], [5, 2, 1], [9, 0, 15], [36, 5, 7]], dtype=torch.int32)
        qc2 = qc.to(dev)
        K.store_query_cache(q.to(dev), qc2, triples.to(dev))
        O.store_query_cache(q, qc, triples)
        assert torch.equal(qc2.cpu(), qc)
        K.store_query_cache(q.to(dev), torch.empty(0, device=dev, dtype=dtype), triples.to(dev))


def test_store_query_ignores_the_unwritten_tail_of_a_device_built_list():
    """A triple buffer of fixed capacity whose valid count lives in a device word (what
    zp_prepare_decode leaves behind): rows past the count hold garbage and must store nothing;
    triples that point outside the query rows or the cache are skipped, not dereferenced."""
    from zipage_b200 import kernel as K
    dev = _gpu()
    g = torch.Generator().manual_seed(4)
    Hq, D, QCL, C, N = 8, 128, 16, 4, 6
    q = torch.randn(N, Hq, D, generator=g).to(torch.bfloat16).to(dev)
    qc = torch.zeros(C, QCL, Hq, D, dtype=torch.bfloat16, device=dev)
    triples = torch.tensor([[0, 2, 0], [5, 1, 15], [3, 0, 7],
                            [1 << 28, 1 << 28, 1 << 28], [-5, -1, 99], [2, 3, 3]],   # garbage tail
                           dtype=torch.int32, device=dev)
    count = torch.tensor([3], dtype=torch.int32, device=dev)
    K.store_query_cache(q, qc, triples, count)
    want = torch.zeros_like(qc)
    want[2, 0], want[1, 15], want[0, 7] = q[0], q[5], q[3]
    assert torch.equal(qc, want)
    # without a count every row is read, and the out-of-range ones are skipped
    qc.zero_()
    K.store_query_cache(q, qc, triples)
    want[3, 3] = q[2]
    torch.cuda.synchronize()
    assert torch.equal(qc, want)


def test_redundancy_functions_match_oracle():
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    dev = _gpu()
    case = CASES["all_stages_exact_fp32"]
    inp = build_inputs(case)
    k, bt = inp["k"], inp["block_tables"]
    for fn_o, fn_k in ((O.raw_redudancy_score, K.raw_redudancy_score),
                       (O.lightning_redudancy_score, K.lightning_redudancy_score)):
        lo, ro = fn_o(k, bt, 0.5, 0.4, return_logits=True)
        lk, rk = fn_k(k.to(dev), bt.to(dev), 0.5, 0.4, return_logits=True)
        lo, lk = lo.reshape(-1), lk.cpu().reshape(-1)
        fin = torch.isfinite(lo)
        assert torch.equal(fin, torch.isfinite(lk))
        assert (lo[fin] - lk[fin]).abs().max() <= 1e-4 * lo[fin].abs().max()
        assert torch.allclose(rk.cpu(), ro, rtol=1e-3, atol=1e-10)
    n_o = O.key_norm(k, bt)
    n_k = K.key_norm(k.to(dev), bt.to(dev)).cpu()
    assert torch.allclose(n_k, n_o, rtol=1e-5)


def test_window_mask_and_logits():
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    dev = _gpu()
    case = CASES["plain_fp32"]
    inp = build_inputs(case)
    so, lo = O.attention_score(inp["k"], inp["q"], inp["query_ids"], inp["block_tables"],
                               return_logits=True)
    sk, lk = K.attention_score(inp["k"].to(dev), inp["q"].to(dev), inp["query_ids"].to(dev),
                               inp["block_tables"].to(dev), return_logits=True)
    fin = torch.isfinite(lo)
    assert torch.equal(fin, torch.isfinite(lk.cpu()))
    assert (lo[fin] - lk.cpu()[fin]).abs().max() < 1e-4
    for red in ("mean", "max"):
        a = O.attention_score(inp["k"], inp["q"], inp["query_ids"], inp["block_tables"], reduced=red)
        b = K.attention_score(inp["k"].to(dev), inp["q"].to(dev), inp["query_ids"].to(dev),
                              inp["block_tables"].to(dev), reduced=red).cpu()
        assert torch.allclose(a, b, rtol=1e-3, atol=1e-9)
    w1 = O.window_mask(so.clone(), inp["block_tables"], 16)
    w2 = K.window_mask(sk.clone(), inp["block_tables"].to(dev), 16).cpu()
    assert torch.equal(torch.isinf(w1), torch.isinf(w2))


def test_compaction_properties_at_scale():
    """Config-2 shaped rows (9 pages -> 8) on many units: the compacted pages hold exactly the
    kept rows in order (checked by gathering), untouched pages stay untouched."""
    from zipage_b200 import kernel as K
    dev = _gpu()
    torch.manual_seed(1)
    Ln, B, Hkv, D, NB, NT = 3, 24, 8, 128, 9, 9
    P = B * NB + 7
    k = torch.randn(Ln, P, BS, Hkv, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn_like(k)
    perm = torch.randperm(P, device=dev)[: B * NB].view(B, NB).to(torch.int32)
    table = perm.clone()
    table[:, -1] = -table[:, -1] - 2
    target = perm.clone()
    fresh = torch.arange(P, device=dev, dtype=torch.int32)
    unused = fresh[~torch.isin(fresh, perm.flatten())]
    target[0, 0] = unused[0]          # first-time compression: a fresh page replaces a shared one
    target[1, 0] = unused[1]
    scores = torch.rand(Ln, B, Hkv, NB * BS, device=dev)
    keep = K.topk_mask(scores, 8 * BS).view(Ln, B, Hkv, NB, BS)
    k0, v0 = k.clone(), v.clone()
    K.compress_kv(k, v, keep, table, target)
    torch.cuda.synchronize()
    for l in range(Ln):
        for b in range(0, B, 5):
            for h in (0, 7):
                idx = keep[l, b, h].flatten().nonzero().flatten()
                assert idx.numel() == 8 * BS
                src = k0[l, perm[b].long()][:, :, h].reshape(NB * BS, D)[idx]
                dst = k[l, target[b, :8].long()][:, :, h].reshape(8 * BS, D)
                assert torch.equal(src, dst)
                srcv = v0[l, perm[b].long()][:, :, h].reshape(NB * BS, D)[idx]
                dstv = v[l, target[b, :8].long()][:, :, h].reshape(8 * BS, D)
                assert torch.equal(srcv, dstv)
    # pages no sequence owns are untouched
    assert torch.equal(k[:, unused[2:].long()], k0[:, unused[2:].long()])


def test_update_tables():
    from zipage_b200 import kernel as K
    dev = _gpu()
    tgt = torch.tensor([[5, 2, 9], [1, 7, 3]], dtype=torch.int32, device=dev)
    nt, ctx, nxt = K.update_tables(tgt, table_width=5)
    assert nt.cpu().tolist() == [[5, 2, 9, -1, -1], [1, 7, 3, -1, -1]]
    assert ctx.cpu().tolist() == [2 * BS + 1] * 2
    assert nxt.cpu().tolist() == [9 * BS, 3 * BS]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("exact", [False, True])
def test_redundancy_tcgen05_matches_simt_and_oracle(dtype, exact):
    """The tensor-core similarity kernels against the SIMT kernels (same dtype) and the oracle."""
    from oracle import zipage_oracle as O
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.synthetic import make_compress_workload
    dev = _gpu()
    w = make_compress_workload(B=5, L=3, Hkv=2, Hq=4, QCL=16, budget=2, pages_per_seq=[3, 4, 3, 5, 3],
                               dtype=dtype, device=dev, seed=21, similar_keys=True, spare_pages=2)
    k, bt = w.kv_cache[0], w.block_tables
    a = K.redundancy_logits(k, bt, 0.5, exact=exact, impl="tcgen05")
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    b = K.redundancy_logits(k, bt, 0.5, exact=exact, impl="simt")
    fn = O.raw_redudancy_score if exact else O.lightning_redudancy_score
    lo, _ = fn(k.cpu(), bt.cpu(), 0.5, 0.4, return_logits=True)
    a, b, lo = a.float().cpu().reshape(-1), b.float().cpu().reshape(-1), lo.float().reshape(-1)
    fin = torch.isfinite(b)
    assert torch.equal(fin, torch.isfinite(a)) and torch.equal(fin, torch.isfinite(lo))
    scale = b[fin].abs().max()
    assert scale > 2.0  # the similar keys make the exemption rule matter
    assert (a[fin] - b[fin]).abs().max() <= 1e-2 * scale
    assert (a[fin] - lo[fin]).abs().max() <= 2e-2 * scale


@pytest.mark.parametrize("exact", [False, True])
def test_redundancy_tcgen05_many_jobs_per_block(exact):
    """Enough (unit, page) jobs that every persistent block walks through dozens of them, with
    ragged tables: the stage rings, page-slot rotation and barrier phases wrap many times.  The
    SIMT kernels are the reference at this size."""
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.synthetic import make_compress_workload
    dev = _gpu()
    lens = [3 + (i * 7) % 8 for i in range(96)]          # 3..10 pages
    w = make_compress_workload(B=96, L=2, Hkv=4, Hq=8, QCL=16, budget=2, pages_per_seq=lens,
                               dtype=torch.bfloat16, device=dev, seed=5, similar_keys=True)
    k, bt = w.kv_cache[0], w.block_tables
    for _ in range(2):   # twice: state left behind by a launch must not matter
        a = K.redundancy_logits(k, bt, 0.5, exact=exact, impl="tcgen05")
        torch.cuda.synchronize()
        assert _lib.device_error() == 0
    b = K.redundancy_logits(k, bt, 0.5, exact=exact, impl="simt")
    a, b = a.float().reshape(-1), b.float().reshape(-1)
    fin = torch.isfinite(b)
    assert torch.equal(fin, torch.isfinite(a))
    scale = b[fin].abs().max()
    assert scale > 2.0
    assert (a[fin] - b[fin]).abs().max() <= 1e-2 * scale


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv,QCL,reduced", [(8, 2, 32, "mean"), (4, 2, 16, "mean"), (2, 2, 16, "max"),
                                                 (16, 2, 16, "mean")])
def test_window_score_tcgen05_matches_simt_and_oracle(dtype, Hq, Hkv, QCL, reduced):
    from oracle import zipage_oracle as O
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.synthetic import make_compress_workload
    dev = _gpu()
    w = make_compress_workload(B=5, L=3, Hkv=Hkv, Hq=Hq, QCL=QCL, budget=2, pages_per_seq=[3, 4, 3, 5, 3],
                               dtype=dtype, device=dev, seed=31, spare_pages=2)
    a = K.attention_score(w.kv_cache[0], w.query_cache, w.query_ids, w.block_tables, reduced=reduced,
                          impl="tcgen05")
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    b = K.attention_score(w.kv_cache[0], w.query_cache, w.query_ids, w.block_tables, reduced=reduced,
                          impl="simt")
    o = O.attention_score(w.kv_cache[0].cpu(), w.query_cache.cpu(), w.query_ids.cpu(),
                          w.block_tables.cpu(), reduced=reduced)
    a, b, o = a.float().cpu(), b.float().cpu(), o.float()
    scale = o.abs().max()
    assert (a - b).abs().max() <= 2e-2 * scale
    assert (a - o).abs().max() <= 2e-2 * scale
    # the bulk agrees to the last bit of T; only isolated roundings differ
    assert (a != o).float().mean() < 0.02


@pytest.mark.parametrize("variant", ["exact", "lightning"])
def test_config1_shapes_fp32_bit_exact_against_oracle(variant):
    """The single-layer CPU config (4 ragged sequences of 9, 9, 10, 10 full pages, 32 query / 8 KV
    heads, window 32, pool 7, lambda 0.5, budget 8 pages) in fp32: identical kept sets and
    identical compacted caches."""
    from oracle import zipage_oracle as O
    from zipage_b200.compress import CompressConfig, compress_chunk
    from zipage_b200.synthetic import make_compress_workload
    dev = _gpu()
    kw = dict(budget_blocks=8, query_cache_len=32, use_redudancy=True,
              lightning_redudancy=variant == "lightning", redudancy_lambda=0.5, redudancy_temperature=0.4,
              enable_pooling=True, continues_pooling=True, pooling_size=7)
    w = make_compress_workload(B=4, L=1, Hkv=8, Hq=32, QCL=32, budget=8, pages_per_seq=[9, 9, 10, 10],
                               dtype=torch.float32, device="cpu", seed=0, compressed_prob=0.0)
    ko, vo = w.kv_cache[0].clone(), w.kv_cache[1].clone()
    _, keep_o = O.compress(ko, vo, w.query_cache, None, w.query_ids, w.block_tables, w.target_tables,
                           w.compressed, O.CompressConfig(**kw))
    kg = w.kv_cache.to(dev)
    dbg = compress_chunk(kg[0], kg[1], w.query_cache.to(dev), None, w.query_ids.to(dev),
                         w.block_tables.to(dev), w.target_tables.to(dev), w.compressed.to(dev),
                         CompressConfig(**kw), return_debug=True)
    torch.cuda.synchronize()
    assert torch.equal(dbg["keep"].cpu(), keep_o)
    assert torch.equal(kg[0].cpu(), ko) and torch.equal(kg[1].cpu(), vo)
    assert (keep_o.flatten(3).sum(-1) == 8 * BS).all()
