"""Seeded inputs of the golden cases (shared by the generator and the tests).

Inputs are not stored: they are rebuilt from `numpy.random.RandomState`, whose
stream is frozen by numpy's compatibility policy, and each fixture carries a
SHA-256 of the inputs it was made from so that a drift would be noticed.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch

BS = 256  # page size (zipage/engine/sequence.py:15)

# name -> parameters.  `tables` are the sequences' page lists (decoded ids, in
# table order); `targets` the host-chosen destination pages (budget+1 each);
# flags follow zipage/config.py:22-46.
CASES = {
    # attention score only, two ragged sequences (4 and 3 pages), G = 4
    "plain_fp32": dict(
        seed=11, dtype="float32", L=2, P=10, Hkv=2, Hq=8, D=128, QCL=16, C=4,
        tables=[[7, 2, 9, 4], [1, 5, 3]], targets=[[7, 2, 9], [1, 5, 3]],
        query_ids=[3, 1], compressed=[False, False], cfg=dict(budget_blocks=2, query_cache_len=16),
    ),
    # the README recipe: global score + pooling + lightning redundancy;
    # one first-time compression with a fresh target page, one repeat
    "recipe_lightning_fp32": dict(
        seed=12, dtype="float32", L=2, P=10, Hkv=2, Hq=4, D=128, QCL=16, C=3,
        tables=[[0, 4, 6, 8], [2, 9, 5]], targets=[[1, 4, 6], [2, 9, 5]],
        query_ids=[0, 2], compressed=[False, True],
        cfg=dict(budget_blocks=2, query_cache_len=16, use_global_score=True, decay_factor=0.8,
                 use_redudancy=True, lightning_redudancy=True, redudancy_lambda=0.2,
                 redudancy_temperature=0.4, enable_pooling=True),
    ),
    # exact redundancy with every optional stage on
    "all_stages_exact_fp32": dict(
        seed=13, dtype="float32", L=1, P=8, Hkv=2, Hq=4, D=128, QCL=32, C=2,
        tables=[[3, 1, 6, 0], [5, 2, 7]], targets=[[3, 1, 6], [5, 2, 7]],
        query_ids=[1, 0], compressed=[True, False],
        cfg=dict(budget_blocks=2, query_cache_len=32, use_global_score=True, decay_factor=0.7,
                 max_norm=True, use_redudancy=True, lightning_redudancy=False,
                 redudancy_lambda=0.5, redudancy_temperature=0.4, enable_pooling=True,
                 continues_pooling=True, use_attention_sink=True, sink_len=4),
    ),
    # 16-bit rounding points (bf16 does not work under the Triton interpreter; fp16 does)
    "recipe_exact_fp16": dict(
        seed=14, dtype="float16", L=1, P=6, Hkv=2, Hq=4, D=128, QCL=16, C=2,
        tables=[[4, 0, 2], [1, 5, 3]], targets=[[4, 0, 2], [1, 5, 3]],
        query_ids=[0, 1], compressed=[True, False],
        cfg=dict(budget_blocks=2, query_cache_len=16, use_global_score=True, decay_factor=0.8,
                 use_redudancy=True, lightning_redudancy=False, redudancy_lambda=0.2,
                 redudancy_temperature=0.4, enable_pooling=True),
    ),
    "recipe_lightning_fp16": dict(
        seed=15, dtype="float16", L=1, P=6, Hkv=2, Hq=4, D=128, QCL=16, C=2,
        tables=[[4, 0, 2], [1, 5, 3]], targets=[[4, 0, 2], [1, 5, 3]],
        query_ids=[0, 1], compressed=[True, False],
        cfg=dict(budget_blocks=2, query_cache_len=16, use_global_score=True, decay_factor=0.8,
                 use_redudancy=True, lightning_redudancy=True, redudancy_lambda=0.2,
                 redudancy_temperature=0.4, enable_pooling=True),
    ),
}


def encode_tables(tables):
    """Pad with -1 and mark each sequence's last page as -(id)-2
    (zipage/engine/model_runner.py:440-441, :457-463)."""
    nb = max(len(t) for t in tables)
    rows = [t[:-1] + [-t[-1] - 2] + [-1] * (nb - len(t)) for t in tables]
    return torch.tensor(rows, dtype=torch.int32)


def build_inputs(case):
    """Returns dict(k, v, q, score_cache, block_tables, targets, query_ids, compressed)."""
    rs = np.random.RandomState(case["seed"])
    L, P, Hkv, Hq, D, QCL, C = (case[x] for x in ("L", "P", "Hkv", "Hq", "D", "QCL", "C"))
    dt = getattr(torch, case["dtype"])
    k = rs.standard_normal((L, P, BS, Hkv, D)).astype(np.float32)
    v = rs.standard_normal((L, P, BS, Hkv, D)).astype(np.float32)
    q = rs.standard_normal((L, C, QCL, Hq, D)).astype(np.float32)
    # near-duplicate keys so that the similarity threshold (0.5) is exceeded:
    # inside a page, across pages of a sequence, and clusters of three
    for t in case["tables"]:
        a, b = t[0], t[1]
        k[:, b, 16:48] = k[:, a, 64:96] + 0.35 * rs.standard_normal((L, 32, Hkv, D))
        k[:, a, 200:216] = k[:, a, 100:116] + 0.25 * rs.standard_normal((L, 16, Hkv, D))
        k[:, t[-1], 5:13] = k[:, a, 100:108] + 0.30 * rs.standard_normal((L, 8, Hkv, D))
        k[:, t[-1], 120:128] = 1.7 * k[:, t[-1], 60:68]  # exact direction duplicates
    sc = rs.uniform(0.0, 2.0 / (BS * 3), size=(L, P, BS, Hkv)).astype(np.float32)
    out = dict(
        k=torch.from_numpy(k).to(dt), v=torch.from_numpy(v).to(dt), q=torch.from_numpy(q).to(dt),
        score_cache=torch.from_numpy(sc).to(dt),
        block_tables=encode_tables(case["tables"]),
        targets=torch.tensor(case["targets"], dtype=torch.int32),
        query_ids=torch.tensor(case["query_ids"], dtype=torch.int32),
        compressed=torch.tensor(case["compressed"], dtype=torch.bool),
    )
    return out


def tensor_sha(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()
