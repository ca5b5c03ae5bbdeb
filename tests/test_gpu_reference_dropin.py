"""The drop-in, dropped in: the reference's own ModelRunner.compress on the GPU.

`ModelRunner.compress` (zipage/engine/model_runner.py:424-631, unmodified, from baseline/_ref) is
run twice on the same bf16 caches: once with the reference's Triton kernels, once with
`zipage_b200.kernel` functions bound at its import sites.  Checked:
  * both runs leave `time_record` with the same keys (the engine reads them, zipage_engine.py);
  * stage outputs of the Triton kernels and of this library agree within the bf16 tolerance;
  * the kept sets differ only on indices whose selection score (the reference run's own) lies
    within one rounding step of the cut, and the compacted caches agree row for row elsewhere.
Skipped with the reason when the reference or Triton is not available on the machine.
"""
import pytest
import torch

import ref_binding as RB

pytestmark = pytest.mark.gpu
BS = 256


def _need_reference():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    ok, why = RB.reference_available()
    if not ok:
        pytest.skip(why)
    return RB.import_reference()


def _workload(dtype, seed, global_score):
    from zipage_b200.synthetic import make_compress_workload
    return make_compress_workload(B=6, L=4, Hkv=8, Hq=32, QCL=32, budget=8, dtype=dtype, device="cuda:0",
                                  seed=seed, with_score_cache=global_score, compressed_prob=0.5)


@pytest.mark.parametrize("variant", ["lightning", "exact"])
def test_reference_compress_with_bound_kernels(variant):
    from oracle.boundary import kept_set_report
    mr = _need_reference()
    dtype = torch.bfloat16
    cfg = dict(budget_blocks=8, query_cache_len=32, use_global_score=True, decay_factor=0.8,
               use_redudancy=True, lightning_redudancy=variant == "lightning", redudancy_lambda=0.5,
               redudancy_temperature=0.4, enable_pooling=True)
    w = _workload(dtype, 31, True)
    L = w.kv_cache.shape[1]
    tables = [[int(x) for x in row if x != -1] for row in w.tables_plain.cpu().tolist()]
    seqs = RB.sequences(tables, w.target_tables.cpu().tolist(), w.query_ids.cpu().tolist(),
                        w.compressed.cpu().tolist())
    rec = {}

    def recording(fn, tag):
        def topk(scores, k):
            keep = fn(scores, k)
            rec.setdefault(tag, []).append((scores.clone(), keep.clone()))
            return keep
        return topk

    # run A: the reference's own kernels (layer_stride 2: two chunks, as the engine walks the layers)
    kvA, qA, scA = w.kv_cache.clone(), w.query_cache.clone(), w.score_cache.clone()
    runA = RB.bare_runner(mr, kvA, qA, scA, cfg, L, 2)
    orig_topk = mr.topk_mask
    mr.topk_mask = recording(orig_topk, "ref")
    try:
        mr.ModelRunner.compress(runA, seqs)
    finally:
        mr.topk_mask = orig_topk
    # run B: the same method, zipage_b200.kernel bound in place of zipage.kernel
    kvB, qB, scB = w.kv_cache.clone(), w.query_cache.clone(), w.score_cache.clone()
    runB = RB.bare_runner(mr, kvB, qB, scB, cfg, L, 2)
    with RB.bound_kernels(mr):
        mr.topk_mask = recording(mr.topk_mask, "ours")
        mr.ModelRunner.compress(runB, seqs)
    torch.cuda.synchronize()
    assert set(runA.time_record) == set(runB.time_record), (sorted(runA.time_record), sorted(runB.time_record))
    assert all(runB.time_record[k] > 0 for k in runB.time_record)
    outside = differing = 0
    worst = 0.0
    for (fa, ka), (fb, kb) in zip(rec["ref"], rec["ours"]):
        fin = torch.isfinite(fa.float())
        assert torch.equal(fin, torch.isfinite(fb.float()))
        assert (fa.float()[fin] - fb.float()[fin]).abs().max() <= 2e-2 * fa.float()[fin].abs().max()
        rep = kept_set_report(fa.cpu(), ka.cpu(), kb.cpu(), 8 * BS, dtype,
                              parts=dict(score_term=fa.cpu().float().abs() + 1e-4, red_term=None))
        outside += rep["outside"]; differing += rep["differing"]; worst = max(worst, rep["worst"])
    total = sum(k.numel() for _, k in rec["ref"])
    print(f"reference compress() [{variant}]: Triton kernels vs zipage_b200 bound: {differing} of {total} keep "
          f"flags differ, {outside} outside one step of the cut (worst {worst:.2f} steps); "
          f"stage keys {sorted(k for k in runB.time_record if not k.endswith('_sum'))}")
    assert outside == 0
    assert differing <= 2e-3 * total
    # compacted caches: bit-identical for every (layer, sequence, head) whose kept sets agree (one
    # differing flag shifts every later row of that unit, so the others are not comparable row by row)
    keepA = torch.cat([k for _, k in rec["ref"]], dim=0)      # [L, B, Hkv, NB*BS], chunks in layer order
    keepB = torch.cat([k for _, k in rec["ours"]], dim=0)
    agree = (keepA == keepB).all(dim=-1)                       # [L, B, Hkv]
    assert agree.float().mean() > 0.8
    tgt = w.target_tables[:, :8].long()                        # the pages that receive the kept rows
    checked = 0
    for b in range(tgt.shape[0]):
        a = kvA[:, :, tgt[b]]                                  # [2, L, 8, BS, Hkv, D]
        c = kvB[:, :, tgt[b]]
        same = (a == c).all(dim=-1).all(dim=3).all(dim=2).all(dim=0)   # [L, Hkv]
        assert bool(same[agree[:, b]].all()), (b, same, agree[:, b])
        checked += int(agree[:, b].sum())
    print(f"compacted K/V bit-identical on all {checked} units whose kept sets agree")


def test_reference_stage_kernels_against_this_library():
    """Kernel by kernel on bf16 inputs: the reference's Triton kernels run natively on this GPU
    (no interpreter), this library beside them."""
    _need_reference()
    from zipage.kernel.attention_score import attention_score as r_att
    from zipage.kernel.global_score import global_score as r_glob
    from zipage.kernel.lightning_redudancy_score import lightning_redudancy_score as r_light
    from zipage.kernel.raw_redudancy_score import raw_redudancy_score as r_raw
    from zipage.kernel.compress_kv import compress_kv as r_ckv
    from zipage.kernel.utils import topk_mask as r_topk
    from zipage_b200 import kernel as K
    w = _workload(torch.bfloat16, 32, True)
    k = w.kv_cache[0]
    pairs = [
        ("attention_score", r_att(k, w.query_cache, w.query_ids, w.block_tables),
         K.attention_score(k, w.query_cache, w.query_ids, w.block_tables)),
        ("lightning_redudancy_score", r_light(k, w.block_tables, temperature=0.4),
         K.lightning_redudancy_score(k, w.block_tables, temperature=0.4)),
        ("raw_redudancy_score", r_raw(k, w.block_tables, temperature=0.4),
         K.raw_redudancy_score(k, w.block_tables, temperature=0.4)),
    ]
    for name, a, b in pairs:
        a, b = a.float(), b.float()
        rel = (a - b).abs().max().item() / a.abs().max().item()
        print(f"{name}: max rel err {rel:.2e}, differing elements {(a != b).float().mean().item():.2e}")
        assert rel <= 2e-2, name
    s1 = K.attention_score(k, w.query_cache, w.query_ids, w.block_tables)
    s2 = s1.clone()
    c1, c2 = w.score_cache.clone(), w.score_cache.clone()
    r_glob(s1, c1, w.block_tables, w.compressed, 0.8)
    K.global_score(s2, c2, w.block_tables, w.compressed, 0.8)
    assert torch.equal(s1, s2) and torch.equal(c1, c2)
    # compaction given the same flags: bit-identical caches
    flat = s1.view(*s1.shape[:3], -1)
    keep = r_topk(flat, 8 * BS).view(s1.shape)
    ka, va, kb, vb = w.kv_cache[0].clone(), w.kv_cache[1].clone(), w.kv_cache[0].clone(), w.kv_cache[1].clone()
    r_ckv(ka, va, keep, w.block_tables, w.target_tables)
    K.compress_kv(kb, vb, keep, w.block_tables, w.target_tables)
    torch.cuda.synchronize()
    assert torch.equal(ka, kb) and torch.equal(va, vb)
