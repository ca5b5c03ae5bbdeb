"""The CPU restatement of the per-step ops against fixtures produced by the unmodified reference
(tests/golden/make_step_golden.py).  Bit-exact: same library, same rounding points."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests" / "golden"))
from step_cases import CASE, DTYPES, build_step_inputs, decode_state, from_np  # noqa: E402

from oracle import step_ops_oracle as S  # noqa: E402


def _load(name, dtype):
    z = np.load(ROOT / "tests" / "golden" / f"step_ops_{name}.npz")
    return {k: from_np(z[k], dtype) for k in z.files}


@pytest.mark.parametrize("name", list(DTYPES))
def test_elementwise_ops_match_reference(name):
    dt = DTYPES[name]
    inp, ref, c = build_step_inputs(dt), _load(name, dt), CASE
    assert torch.equal(S.rms_norm(inp["x"], inp["w_hidden"], c["eps"]), ref["rms"])
    y, res = S.add_rms_norm(inp["x"], inp["residual"], inp["w_hidden"], c["eps"])
    assert torch.equal(y, ref["add_rms"])
    if dt == torch.float32:
        # In fp32 every `.float()` / `.to(orig_dtype)` of layernorm.py:34-39 is a no-op, so the
        # reference's in-place ops leave `residual` aliased to the normalised output.  That alias
        # is recorded here and not reproduced: the restatement returns the sum, as the 16-bit
        # path (the only one the engine runs) does.
        assert torch.equal(ref["add_rms_residual"], ref["add_rms"])
        assert torch.equal(res, inp["x"] + inp["residual"])
    else:
        assert torch.equal(res, ref["add_rms_residual"])
    assert torch.equal(S.silu_and_mul(inp["gate_up"]), ref["silu_mul"])
    cache = S.rope_cos_sin_cache(c["D"], c["max_position"], c["rope_base"])
    assert torch.equal(cache[inp["positions"]], ref["cos_sin_rows"].float())
    q, k, v = S.qk_norm_rope(inp["qkv"], inp["positions"], cache, inp["w_q"], inp["w_k"], c["eps"],
                             c["Hq"], c["Hkv"], c["D"])
    assert torch.equal(q, ref["q_rot"]) and torch.equal(k, ref["k_rot"])
    tok = S.sample_race(inp["logits"], inp["temperatures"], ref["noise"].float())
    assert torch.equal(tok, ref["tokens"].long())


def test_prepare_decode_matches_reference():
    st = decode_state()
    z = np.load(ROOT / "tests" / "golden" / "prepare_decode.npz")
    pos, ctx, slot, tables, trip = S.prepare_decode(st["num_tokens"], st["block_tables"], st["query_ids"],
                                                    st["query_cache_len"])
    assert np.array_equal(pos.numpy(), z["positions"])
    assert np.array_equal(ctx.numpy(), z["context_lens"])
    assert np.array_equal(slot.numpy(), z["slot_mapping"])
    assert np.array_equal(tables.numpy(), z["block_tables"])
    assert np.array_equal(trip.numpy(), z["triples"]) and len(trip) == 3
