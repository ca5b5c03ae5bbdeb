"""Kept-set boundary rule for 16-bit caches (test infrastructure, like the rest of oracle/).

In fp32 the kept sets of the CUDA path and of the oracle are compared bit for bit.  In bf16 /
fp16 two correct implementations of the reference's formulas can differ in the last place of a
score (accumulation order of the dot products, exp / division rounding), and the top-k cut of
zipage/kernel/utils.py:21-36 turns a last-place difference of a score that sits AT the cut into
a different kept index.  The rule checked here is the only difference that is accepted:

    every index that one side keeps and the other drops has an oracle selection score within
    ONE rounding step (of the cache dtype) of the oracle's k-th largest score of that row.

The selection score is `score*lambda - redundancy*(1-lambda)` (model_runner.py:559-561): a
difference of two rounded terms, so its own last place can be far finer than the last place of
the terms it was made from.  "One rounding step" is therefore the step of the larger of the two
terms at that index (or at the cut element, whichever is larger) — the amount by which the
selection score moves when one of its inputs moves by one unit in the last place.
"""
from __future__ import annotations

import torch

_MANT = {torch.bfloat16: 7, torch.float16: 10, torch.float32: 23}


def rounding_step(x: torch.Tensor, dtype) -> torch.Tensor:
    """Spacing of `dtype` values at the magnitude of x (fp32 tensor in, fp32 out)."""
    a = x.float().abs().clamp_min(torch.finfo(dtype).tiny)
    return torch.exp2(torch.floor(torch.log2(a)) - _MANT[dtype])


def kept_set_report(final, keep_ref, keep_got, k, dtype, parts=None):
    """Compare two keep masks row by row against the oracle's selection scores.

    final [..., N] oracle selection scores (cache dtype, +/-inf allowed); keep_ref / keep_got
    bool [..., N]; k = number kept per row; parts = the dict filled by
    zipage_oracle.compress_scores (terms of the combination) or None.
    Returns dict(mismatch = fraction of differing flags, differing = count, outside = count of
    differing indices farther than one step from the cut, worst = largest gap in steps).
    """
    N = final.shape[-1]
    f = final.reshape(-1, N).float()
    kr = keep_ref.reshape(-1, N)
    kg = keep_got.reshape(-1, N)
    mag = f.abs()
    if parts is not None and parts.get("score_term") is not None:
        mag = torch.maximum(mag, parts["score_term"].reshape(-1, N).float().abs())
        if parts.get("red_term") is not None:
            mag = torch.maximum(mag, parts["red_term"].reshape(-1, N).float().abs())
    mag = torch.where(torch.isfinite(mag), mag, torch.zeros_like(mag))
    differing = outside = 0
    worst = 0.0
    for r in range(f.shape[0]):
        d = torch.nonzero(kr[r] ^ kg[r]).flatten()
        if d.numel() == 0:
            continue
        differing += int(d.numel())
        row = f[r]
        kk = min(k, N)
        order = torch.sort(row, descending=True, stable=True).indices
        cut = order[kk - 1]
        t = row[cut]
        step = torch.maximum(rounding_step(mag[r][d], dtype), rounding_step(mag[r][cut], dtype))
        gap = (row[d] - t).abs() / step
        gap = torch.where(torch.isfinite(gap), gap, torch.full_like(gap, float("inf")))
        outside += int((gap > 1.0).sum())
        worst = max(worst, float(gap.max()))
    return dict(mismatch=float((kr ^ kg).float().mean()), differing=differing, outside=outside,
                worst=worst)
