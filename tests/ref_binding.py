"""Test support: the unmodified reference (installed under baseline/_ref) with this library's
functions bound at the reference's own call sites, as INTEGRATION.md prescribes.

Nothing here computes; it only locates the reference, builds a `ModelRunner` object without its
constructor (which loads a model) and swaps module-level names.
"""
from __future__ import annotations

import contextlib
import sys
import types
from collections import defaultdict
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

KERNEL_NAMES = ["compress_kv", "compress_score", "attention_score", "raw_redudancy_score",
                "lightning_redudancy_score", "global_score", "window_mask", "topk_mask"]


def reference_available():
    """(ok, reason).  The reference needs its installed copy, Triton and a GPU."""
    if not (REF / "zipage" / "engine" / "model_runner.py").is_file():
        return False, "the reference is not installed under baseline/_ref (baseline/install_reference.py)"
    try:
        import triton  # noqa: F401
    except Exception as e:
        return False, f"Triton cannot be imported: {type(e).__name__}: {e}"
    return True, ""


def import_reference():
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import zipage.engine.model_runner as mr
    return mr


@contextlib.contextmanager
def bound_kernels(mr):
    """zipage/engine/model_runner.py:19-27 with the imports switched to zipage_b200.kernel."""
    from zipage_b200 import kernel as K
    saved = {n: getattr(mr, n) for n in KERNEL_NAMES}
    try:
        for n in KERNEL_NAMES:
            setattr(mr, n, getattr(K, n))
        yield
    finally:
        for n, f in saved.items():
            setattr(mr, n, f)


def bare_runner(mr, kv_cache, query_cache, score_cache, cfg, num_layers, layer_stride):
    """A ModelRunner that has exactly the attributes `compress` reads (model_runner.py:32-110)."""
    import torch
    r = object.__new__(mr.ModelRunner)
    r.compress_stream = torch.cuda.Stream()
    r.model = types.SimpleNamespace(model=types.SimpleNamespace(layers=[None] * num_layers))
    r.layer_stride = layer_stride
    r.block_size = kv_cache.shape[3]
    r.max_blocks_per_seq = cfg["budget_blocks"] + 1
    r.query_cache_len = cfg["query_cache_len"]
    r.use_global_score = cfg.get("use_global_score", False)
    r.max_norm = cfg.get("max_norm", False)
    r.decay_factor = cfg.get("decay_factor", 0.8)
    r.use_redudancy = cfg.get("use_redudancy", False)
    r.lightning_redudancy = cfg.get("lightning_redudancy", False)
    r.redudancy_lambda = cfg.get("redudancy_lambda", 0.2)
    r.redudancy_temperature = cfg.get("redudancy_temperature", 0.4)
    r.enable_pooling = cfg.get("enable_pooling", False)
    r.continues_pooling = cfg.get("continues_pooling", False)
    r.use_attention_sink = cfg.get("use_attention_sink", False)
    r.sink_len = cfg.get("sink_len", 4)
    r.pooling_size = 5  # zipage/engine/model_runner.py:71
    r.time_record = defaultdict(int)
    r.kv_cache, r.query_cache, r.score_cache = kv_cache, query_cache, score_cache
    return r


def sequences(tables, targets, query_ids, compressed):
    return [types.SimpleNamespace(query_id=int(q), block_table=list(t), new_block_table=list(g),
                                  compressed=bool(c))
            for q, t, g, c in zip(query_ids, tables, targets, compressed)]
