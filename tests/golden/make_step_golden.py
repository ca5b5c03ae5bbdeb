"""Generate the fixtures of the per-step ops by running the UNMODIFIED reference on CPU.

    python tests/golden/make_step_golden.py /path/to/reference

What runs is the reference's own code, eagerly (TorchDynamo disabled, so every `@torch.compile`
method executes exactly as its Python source reads):

* `RMSNorm.forward` with and without a residual (third_party/nanovllm/layers/layernorm.py:42-50),
* `SiluAndMul.forward` (third_party/nanovllm/layers/activation.py:12-14),
* the q/k normalisation and rotation of `Qwen3Attention.forward`
  (third_party/nanovllm/models/qwen3.py:75-79) composed from the reference's `RMSNorm` and
  `RotaryEmbedding` modules,
* `Sampler.calculate_probs` + `Sampler.sample` (zipage/layers/sampler.py:18-31) — the Exp(1) draws
  `sample` makes in place are reproduced with the same seed and stored,
* `ModelRunner.prepare_decode` (zipage/engine/model_runner.py:633-675) on `Sequence` objects, with
  `Tensor.cuda` / `pin_memory=` shimmed to CPU no-ops and `set_context` read back.

Inputs come from `step_cases.py` (seeded); the fixtures `step_ops_<dtype>.npz` hold the outputs.
"""
from __future__ import annotations

import os
import sys
import types
from pathlib import Path

os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from step_cases import CASE, DTYPES, build_step_inputs, decode_state, to_np  # noqa: E402


def main():
    ref_root = Path(sys.argv[1])
    sys.path[:0] = [str(ref_root), str(ref_root / "third_party")]
    from nanovllm.layers.activation import SiluAndMul
    from nanovllm.layers.layernorm import RMSNorm
    from nanovllm.layers.rotary_embedding import RotaryEmbedding
    from zipage.layers.sampler import Sampler

    for name, dt in DTYPES.items():
        inp = build_step_inputs(dt)
        c = CASE
        out = {}
        norm = RMSNorm(c["hidden"], eps=c["eps"])
        norm.weight.data = inp["w_hidden"].clone()
        out["rms"] = norm(inp["x"].clone())
        y, res = norm(inp["x"].clone(), inp["residual"].clone())
        out["add_rms"], out["add_rms_residual"] = y, res
        out["silu_mul"] = SiluAndMul()(inp["gate_up"].clone())

        qn, kn = RMSNorm(c["D"], eps=c["eps"]), RMSNorm(c["D"], eps=c["eps"])
        qn.weight.data, kn.weight.data = inp["w_q"].clone(), inp["w_k"].clone()
        rope = RotaryEmbedding(c["D"], c["D"], c["max_position"], c["rope_base"])
        q, k, v = inp["qkv"].split([c["Hq"] * c["D"], c["Hkv"] * c["D"], c["Hkv"] * c["D"]], dim=-1)
        q = qn(q.view(-1, c["Hq"], c["D"]))
        k = kn(k.view(-1, c["Hkv"], c["D"]))
        q, k = rope(inp["positions"], q, k)
        out["q_rot"], out["k_rot"] = q, k
        out["cos_sin_rows"] = rope.cos_sin_cache.squeeze(1)[inp["positions"]]   # the rows used

        sampler = Sampler()
        probs = sampler.calculate_probs(inp["logits"].clone(), inp["temperatures"])
        torch.manual_seed(c["sample_seed"])
        noise = torch.empty_like(probs).exponential_(1)
        torch.manual_seed(c["sample_seed"])
        out["tokens"] = sampler.sample(probs.clone())
        out["noise"] = noise
        np.savez_compressed(HERE / f"step_ops_{name}.npz", **{k_: to_np(v_) for k_, v_ in out.items()})
        print(name, {k_: tuple(v_.shape) for k_, v_ in out.items()})

    # prepare_decode: the reference method on reference Sequence objects
    import zipage.engine.model_runner as mr
    from zipage.engine.sequence import Sequence
    real_tensor = torch.tensor

    def tensor_no_pin(*a, **kw):
        kw.pop("pin_memory", None)
        return real_tensor(*a, **kw)

    torch.tensor = tensor_no_pin
    torch.Tensor.cuda = lambda self, *a, **kw: self
    captured = {}
    mr.set_context = lambda is_prefill, **kw: captured.update(kw)
    st = decode_state()
    seqs = []
    for n, table, qid in zip(st["num_tokens"], st["block_tables"], st["query_ids"]):
        s = Sequence([1] * n)
        s.block_table = list(table)
        s.query_id = qid
        seqs.append(s)
    runner = types.SimpleNamespace(block_size=256, query_cache_len=st["query_cache_len"])
    runner.get_query_slot_mapping = types.MethodType(mr.ModelRunner.get_query_slot_mapping, runner)
    runner.prepare_block_tables = types.MethodType(mr.ModelRunner.prepare_block_tables, runner)
    _, positions = mr.ModelRunner.prepare_decode(runner, seqs)
    trip = captured["query_slot_mapping"]
    np.savez_compressed(
        HERE / "prepare_decode.npz", positions=positions.numpy(),
        context_lens=captured["context_lens"].numpy(), slot_mapping=captured["slot_mapping"].numpy(),
        block_tables=captured["block_tables"].numpy(),
        triples=(trip.numpy() if trip is not None else np.zeros((0, 3), np.int32)))
    print("prepare_decode", positions.shape, None if trip is None else tuple(trip.shape))


if __name__ == "__main__":
    with torch.inference_mode():   # as the reference's runner does (model_runner.py: run)
        main()
