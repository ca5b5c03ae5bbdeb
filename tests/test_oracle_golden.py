"""The oracle against fixtures produced by the unmodified reference
(tests/golden/make_golden.py).  CPU only."""
from pathlib import Path

import numpy as np
import pytest
import torch

from cases import BS, CASES, build_inputs, tensor_sha
from oracle import zipage_oracle as O

GOLD = Path(__file__).resolve().parent / "golden"


def _unpack(bits, shape):
    return torch.from_numpy(np.unpackbits(bits, axis=-1)[..., : shape[-1]].astype(bool)).view(shape)


def _run_oracle(case):
    inp = build_inputs(case)
    cfg = O.CompressConfig(**case["cfg"])
    k, v, q = inp["k"].clone(), inp["v"].clone(), inp["q"].clone()
    sc = inp["score_cache"].clone() if cfg.use_global_score else None
    att = O.attention_score(k, q, inp["query_ids"], inp["block_tables"])
    red_logits = None
    if cfg.use_redudancy:
        fn = O.lightning_redudancy_score if cfg.lightning_redudancy else O.raw_redudancy_score
        red_logits, _ = fn(k, inp["block_tables"], temperature=cfg.redudancy_temperature,
                           return_logits=True)
    final, keep = O.compress(k, v, q, sc, inp["query_ids"], inp["block_tables"], inp["targets"],
                             inp["compressed"], cfg)
    return inp, dict(att=att, red_logits=red_logits, final=final, keep=keep, k=k, v=v, sc=sc)


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference(name):
    case = CASES[name]
    g = np.load(GOLD / f"{name}.npz")
    inp, o = _run_oracle(case)
    assert tensor_sha(inp["k"], inp["v"], inp["q"], inp["score_cache"]) == str(g["inputs_sha"])
    fp32 = case["dtype"] == "float32"
    L, B, Hkv = case["L"], len(case["tables"]), case["Hkv"]
    NB = inp["block_tables"].shape[1]

    att_ref = torch.from_numpy(g["attention_score"])
    tol = 1e-6 if fp32 else 2e-3
    assert torch.allclose(o["att"].float(), att_ref, rtol=tol, atol=1e-9 if fp32 else 1e-7)

    if o["red_logits"] is not None:
        ref = torch.from_numpy(g["redudancy_logits"]).view(L, B, Hkv, -1)
        got = o["red_logits"].float().view(L, B, Hkv, -1)
        fin = torch.isfinite(ref)
        assert torch.equal(fin, torch.isfinite(got))
        scale = ref[fin].abs().max()
        err = (got[fin] - ref[fin]).abs().max()
        assert err <= (2e-5 if fp32 else 8e-3) * scale, (err, scale)

    final_ref = torch.from_numpy(g["final_scores"]).view(L, B, Hkv, NB * BS)
    final = o["final"].float().view(L, B, Hkv, NB * BS)
    fin = torch.isfinite(final_ref)
    assert torch.equal(final[~fin], final_ref[~fin])  # the +inf / -inf masks are exact
    scale = final_ref[fin].abs().max()
    err = (final[fin] - final_ref[fin]).abs().max()
    assert err <= (1e-5 if fp32 else 4e-3) * scale, (err, scale)

    keep_ref = _unpack(g["keep"], (L, B, Hkv, NB * BS))
    lit = _unpack(g["keep_literal"], (L, B, Hkv, NB * BS))
    k_top = BS * case["cfg"]["budget_blocks"]
    # the pinned tie rule is one valid answer of the reference's unordered top-k
    assert O.topk_mask_agrees_with_unordered(final_ref, k_top, keep_ref)
    assert O.topk_mask_agrees_with_unordered(final_ref, k_top, lit)
    # canonical selection from the reference's own scores reproduces the fixture bit-exactly
    assert torch.equal(O.topk_mask(final_ref, k_top), keep_ref)
    if fp32:
        # end to end: identical kept sets and identical caches after compaction
        assert torch.equal(o["keep"].view(L, B, Hkv, NB * BS), keep_ref)
        assert tensor_sha(torch.stack([o["k"], o["v"]])) == str(g["kv_after_sha"])
        if o["sc"] is not None:
            assert torch.allclose(o["sc"].float(), torch.from_numpy(g["score_cache_after"]),
                                  rtol=1e-5, atol=1e-9)
    else:
        # 16-bit: kept sets may differ only among scores within one rounding step of the cut
        diff = o["keep"].view(L, B, Hkv, NB * BS) ^ keep_ref
        frac = diff.float().mean().item()
        assert frac < 5e-3, frac


def test_compaction_serial_equals_gather():
    case = CASES["plain_fp32"]
    inp = build_inputs(case)
    L, Hkv = case["L"], case["Hkv"]
    B, NB = inp["block_tables"].shape
    g = torch.Generator().manual_seed(5)
    flag = torch.rand(L, B, Hkv, NB, BS, generator=g) < 0.6
    # no more kept rows than the target pages can hold
    for idx in np.ndindex(L, B, Hkv):
        f = flag[idx].view(-1)
        on = torch.nonzero(f).flatten()
        f[on[2 * BS:]] = False
    flag &= (inp["block_tables"] != -1)[None, :, None, :, None]
    k1, v1 = inp["k"].clone(), inp["v"].clone()
    k2, v2 = inp["k"].clone(), inp["v"].clone()
    O.compress_kv(k1, v1, flag, inp["block_tables"], inp["targets"])
    O.compress_kv_serial(k2, v2, flag, inp["block_tables"], inp["targets"])
    assert torch.equal(k1, k2) and torch.equal(v1, v2)


def test_topk_ties_lowest_index():
    s = torch.tensor([[1.0, 2.0, 2.0, 2.0, 0.0, 2.0, float("inf"), float("inf"), float("-inf")]])
    m = O.topk_mask(s, 4)
    assert m.tolist() == [[False, True, True, False, False, False, True, True, False]]
