"""Seeded inputs of the per-step-op fixtures (shared by the generator and the tests)."""
from __future__ import annotations

import numpy as np
import torch

CASE = dict(N=7, hidden=512, inter=384, Hq=8, Hkv=2, D=128, eps=1e-6, max_position=4096,
            rope_base=1000000.0, B=5, vocab=1031, sample_seed=1234)
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _randn(rs, *shape, scale=1.0):
    return torch.from_numpy((rs.standard_normal(shape) * scale).astype(np.float32))


def build_step_inputs(dtype):
    c = CASE
    rs = np.random.RandomState(20240607)
    inp = {
        "x": _randn(rs, c["N"], c["hidden"]).to(dtype),
        "residual": _randn(rs, c["N"], c["hidden"], scale=3.0).to(dtype),
        "w_hidden": (1.0 + 0.1 * _randn(rs, c["hidden"])).to(dtype),
        "gate_up": _randn(rs, c["N"], 2 * c["inter"], scale=2.0).to(dtype),
        "qkv": _randn(rs, c["N"], (c["Hq"] + 2 * c["Hkv"]) * c["D"], scale=1.5).to(dtype),
        "w_q": (1.0 + 0.2 * _randn(rs, c["D"])).to(dtype),
        "w_k": (1.0 + 0.2 * _randn(rs, c["D"])).to(dtype),
        "positions": torch.from_numpy(rs.randint(0, c["max_position"], size=c["N"]).astype(np.int64)),
        "logits": _randn(rs, c["B"], c["vocab"], scale=4.0).to(dtype),
        "temperatures": torch.tensor([0.6, 1.0, 0.3, 1.5, 0.6], dtype=torch.float32),
    }
    return inp


def decode_state():
    """Running sequences of a decode step: true token counts, (compacted) block tables, window
    ids.  Covers: a token inside and outside the observation window, the first and the last slot
    of a page, a sequence without a window buffer, tables of different length."""
    return dict(
        query_cache_len=32,
        num_tokens=[2049, 2305 + 230, 256 * 3, 256 * 12 + 225, 700, 256 * 5 + 224, 256 * 2 + 256],
        block_tables=[[3, 9, 4, 1, 7, 8, 2, 6, 11], [20, 21, 22, 23, 24, 25, 26, 27, 28],
                      [30, 31, 32], [40, 41, 42, 43, 44, 45, 46, 47, 48], [50, 51, 52],
                      [60, 61, 62, 63, 64, 65], [70, 71, 72]],
        query_ids=[0, 3, 1, -1, 2, 4, 5],
    )


def to_np(t: torch.Tensor):
    """bf16 has no numpy dtype: store its bit pattern as uint16."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def from_np(a, dtype):
    if dtype == torch.bfloat16 and a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())
