"""Generate the golden fixtures by running the UNMODIFIED reference on CPU.

Usage (only where the reference tree is available; the fixtures are committed):

    python tests/golden/make_golden.py /path/to/reference [case ...]

What runs is the reference's own code: `ModelRunner.compress`
(zipage/engine/model_runner.py:424-631) with every Triton kernel of
zipage/kernel executed by the Triton CPU interpreter (TRITON_INTERPRET=1).
Because this container has no GPU the script shims exactly the CUDA plumbing
that method touches — `torch.cuda.stream`, `torch.cuda.Event`, `Tensor.cuda`,
`pin_memory=` — with CPU no-ops, and builds the runner object without calling
its constructor (which would load a model).  Nothing of the arithmetic is
replaced, with one stated exception: the reference's `topk_mask`
(zipage/kernel/utils.py:21-36) uses `torch.topk`, whose choice among equal
scores is unspecified.  Its literal answer is recorded (`keep_literal`), and
the compaction that follows is run with the lowest-index-wins answer
(`keep`), which is the rule this repository pins.

Each fixture `<case>.npz` holds: the final selection scores, both keep masks
(bit-packed), the attention scores, redundancy logits where used, SHA-256 of
the inputs and of the caches after compaction, and a few compacted rows.
"""
from __future__ import annotations

import contextlib
import os
import sys
import time
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from cases import BS, CASES, build_inputs, tensor_sha  # noqa: E402


def install_shims():
    real_tensor = torch.tensor

    def tensor_no_pin(*a, **kw):
        kw.pop("pin_memory", None)
        return real_tensor(*a, **kw)

    class FakeEvent:
        def __init__(self, enable_timing=False):
            self.t = 0.0

        def record(self, stream=None):
            self.t = time.perf_counter()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    torch.tensor = tensor_no_pin
    torch.Tensor.cuda = lambda self, *a, **kw: self
    torch.cuda.stream = lambda s: contextlib.nullcontext()
    torch.cuda.Event = FakeEvent


def run_case(name, ref_root):
    case = CASES[name]
    inp = build_inputs(case)
    cfg = dict(
        budget_blocks=8, query_cache_len=16, use_global_score=False, decay_factor=0.8,
        max_norm=False, use_redudancy=False, lightning_redudancy=False, redudancy_lambda=0.2,
        redudancy_temperature=0.4, enable_pooling=False, continues_pooling=False,
        use_attention_sink=False, sink_len=4,
    )
    cfg.update(case["cfg"])

    import zipage.engine.model_runner as mr
    from zipage.kernel.attention_score import attention_score
    from zipage.kernel.lightning_redudancy_score import lightning_redudancy_score
    from zipage.kernel.raw_redudancy_score import raw_redudancy_score

    rec = {}

    def topk_recording(scores, k):
        literal = rec["orig_topk"](scores, k)
        order = torch.sort(scores.float(), dim=-1, descending=True, stable=True).indices
        canon = torch.zeros_like(scores, dtype=torch.bool)
        canon.scatter_(-1, order[..., :k], True)
        rec.setdefault("final", []).append(scores.clone())
        rec.setdefault("keep_literal", []).append(literal.clone())
        rec.setdefault("keep", []).append(canon.clone())
        return canon

    rec["orig_topk"] = mr.topk_mask
    mr.topk_mask = topk_recording

    L = case["L"]
    runner = object.__new__(mr.ModelRunner)
    runner.compress_stream = types.SimpleNamespace(synchronize=lambda: None)
    runner.model = types.SimpleNamespace(model=types.SimpleNamespace(layers=[None] * L))
    runner.layer_stride = L
    runner.block_size = BS
    runner.max_blocks_per_seq = cfg["budget_blocks"] + 1
    runner.query_cache_len = cfg["query_cache_len"]
    runner.use_global_score = cfg["use_global_score"]
    runner.max_norm = cfg["max_norm"]
    runner.decay_factor = cfg["decay_factor"]
    runner.use_redudancy = cfg["use_redudancy"]
    runner.lightning_redudancy = cfg["lightning_redudancy"]
    runner.redudancy_lambda = cfg["redudancy_lambda"]
    runner.redudancy_temperature = cfg["redudancy_temperature"]
    runner.enable_pooling = cfg["enable_pooling"]
    runner.continues_pooling = cfg["continues_pooling"]
    runner.use_attention_sink = cfg["use_attention_sink"]
    runner.sink_len = cfg["sink_len"]
    runner.pooling_size = 5  # zipage/engine/model_runner.py:71
    from collections import defaultdict

    runner.time_record = defaultdict(int)
    runner.kv_cache = torch.stack([inp["k"], inp["v"]]).clone()
    runner.query_cache = inp["q"].clone()
    runner.score_cache = inp["score_cache"].clone() if cfg["use_global_score"] else None

    # stage outputs taken before the op mutates the caches
    att = attention_score(runner.kv_cache[0], runner.query_cache, inp["query_ids"],
                          inp["block_tables"])
    red_logits = None
    if cfg["use_redudancy"]:
        fn = lightning_redudancy_score if cfg["lightning_redudancy"] else raw_redudancy_score
        red_logits, _ = fn(runner.kv_cache[0], inp["block_tables"],
                           temperature=cfg["redudancy_temperature"], return_logits=True)

    seqs = [
        types.SimpleNamespace(query_id=qid, block_table=list(t), new_block_table=list(tt),
                              compressed=c)
        for qid, t, tt, c in zip(case["query_ids"], case["tables"], case["targets"],
                                 case["compressed"])
    ]
    t0 = time.time()
    mr.ModelRunner.compress(runner, seqs)
    mr.topk_mask = rec["orig_topk"]
    print(f"{name}: reference compress() took {time.time() - t0:.1f}s")

    final = rec["final"][0].float().numpy()
    out = dict(
        inputs_sha=np.array(tensor_sha(inp["k"], inp["v"], inp["q"], inp["score_cache"])),
        attention_score=att.float().numpy(),
        final_scores=final,
        keep=np.packbits(rec["keep"][0].numpy().astype(np.uint8), axis=-1),
        keep_literal=np.packbits(rec["keep_literal"][0].numpy().astype(np.uint8), axis=-1),
        kv_after_sha=np.array(tensor_sha(runner.kv_cache)),
        k_sample=runner.kv_cache[0][:, case["targets"][0][0], :4].float().numpy(),
    )
    if red_logits is not None:
        out["redudancy_logits"] = red_logits.float().numpy()
    if runner.score_cache is not None:
        out["score_cache_after"] = runner.score_cache.float().numpy()
    np.savez_compressed(HERE / f"{name}.npz", **out)


def main():
    ref_root = sys.argv[1]
    sys.path[:0] = [ref_root, os.path.join(ref_root, "third_party")]
    install_shims()
    names = sys.argv[2:] or list(CASES)
    for n in names:
        run_case(n, ref_root)


if __name__ == "__main__":
    main()
