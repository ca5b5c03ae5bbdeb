"""CPU restatement of the small per-step ops around the attention path (test infrastructure only).

These are the "next" rows after the compression path: the element-wise ops of one decoder layer
step and the host-side decode bookkeeping, restated in plain PyTorch with the reference's rounding
points *as the Python source executes them eagerly* (the reference wraps most of them in
`torch.compile`; a compiler may keep fp32 intermediates where the eager code rounds to the model
dtype, so bit-parity is pinned against eager execution of the unmodified reference:
tests/golden/make_step_golden.py runs it with TorchDynamo disabled).

Only tests/, the smoke test and bench.py's CPU-baseline leg may import this module; the product
never does.
"""
from __future__ import annotations

import torch

BLOCK_SIZE = 256


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """third_party/nanovllm/layers/layernorm.py:17-26 — fp32 mean of squares, x * rsqrt(var + eps)
    rounded to the input dtype, then multiplied by the weight in that dtype."""
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * weight


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """layernorm.py:29-40 — the sum x + residual is formed in fp32; the new residual is that sum
    rounded to the input dtype, while the normalisation uses the UNROUNDED fp32 sum."""
    dt = x.dtype
    xf = x.float() + residual.float()
    new_residual = xf.to(dt)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * weight, new_residual


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """third_party/nanovllm/layers/activation.py:12-14 — silu(gate) in the input dtype (computed in
    fp32, rounded), times up, rounded again."""
    a, b = x.chunk(2, -1)
    return torch.nn.functional.silu(a) * b


def rope_cos_sin_cache(head_dim: int, max_position: int, base: float) -> torch.Tensor:
    """rotary_embedding.py:19-22, :84-89 (default rope type): [max_position, head_dim] fp32,
    cos in the first half of a row, sin in the second."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """rotary_embedding.py:8-16 — rotate the two halves of the head dim in fp32, round once."""
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def qk_norm_rope(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                 q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, Hq: int, Hkv: int,
                 D: int):
    """third_party/nanovllm/models/qwen3.py:75-79 — split the fused projection, RMS-normalise
    every q and k head over the head dim, rotate both.  Returns q [N,Hq,D], k [N,Hkv,D],
    v [N,Hkv,D]."""
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    q = rms_norm(q.reshape(-1, Hq, D), q_weight, eps)
    k = rms_norm(k.reshape(-1, Hkv, D), k_weight, eps)
    v = v.reshape(-1, Hkv, D)
    cs = cos_sin[positions].unsqueeze(1)      # [N,1,D]
    cos, sin = cs.chunk(2, dim=-1)
    return apply_rotary_emb(q, cos, sin), apply_rotary_emb(k, cos, sin), v


def sample_race(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """zipage/layers/sampler.py:18-31 — probs = softmax(fp32 logits / T); token = argmax of
    probs / max(noise, 1e-10) with `noise` the Exp(1) draws the reference makes in place (passed
    in so that both sides race on the same draws)."""
    lg = logits.float() / temperatures.unsqueeze(1)
    probs = torch.softmax(lg, dim=-1)
    return (probs / noise.clamp_min(1e-10)).argmax(dim=-1)


def prepare_decode(num_tokens, block_tables, query_ids, query_cache_len, block_size=BLOCK_SIZE):
    """zipage/engine/model_runner.py:633-675 with :306-317 and :319-350 — per running sequence the
    position of the token being fed, the context length, the cache slot its K/V go to and, when the
    token lies in the observation window of its page, the (row, query_id, window index) triple.
    num_tokens: list of len(seq); block_tables: list of lists; query_ids: list (-1 = no window).
    Returns positions [B] i64, context_lens [B] i32, slot_mapping [B] i32, padded tables
    [B, max_len] i32 (-1 padded), triples [n,3] i32."""
    pos, ctx, slot, trip = [], [], [], []
    for i, (n, table, qid) in enumerate(zip(num_tokens, block_tables, query_ids)):
        if n <= 0 or len(table) == 0:
            # padding row of a fixed-size graph batch, filled as the replay branch fills it
            # (model_runner.py:716-719: slot -1, context length 0)
            pos.append(0); ctx.append(0); slot.append(-1)
            continue
        nblocks = (n + block_size - 1) // block_size
        last = n - (nblocks - 1) * block_size
        pos.append(n - 1)
        ctx.append((len(table) - 1) * block_size + last)
        slot.append(table[-1] * block_size + last - 1)
        if qid != -1 and last > block_size - query_cache_len:
            trip.append((i, qid, last - (block_size - query_cache_len) - 1))
    width = max(1, max(len(t) for t in block_tables))
    padded = [list(t) + [-1] * (width - len(t)) for t in block_tables]
    return (torch.tensor(pos, dtype=torch.int64), torch.tensor(ctx, dtype=torch.int32),
            torch.tensor(slot, dtype=torch.int32), torch.tensor(padded, dtype=torch.int32),
            torch.tensor(trip, dtype=torch.int32).reshape(-1, 3))


# ---- the sampler over a vocabulary sharded across ranks -----------------------------------------
# The reference gathers the shards' logits to rank 0 (zipage/layers/embed_head.py:27-34) and
# samples there (zipage/layers/sampler.py:17-31).  The three functions below restate the same race
# shard by shard: softmax statistics per shard, the shard's winner against the global statistics,
# the best of the winners.  Their composition must give sample_race() of the concatenated logits.

def shard_softmax_stats(logits_shard: torch.Tensor, temperatures: torch.Tensor):
    """Per row: the shard's maximum of logits / T and the sum of exp(logits / T - maximum)."""
    lg = logits_shard.float() / temperatures.unsqueeze(1)
    m = lg.max(dim=-1).values
    return m, torch.exp(lg - m.unsqueeze(1)).sum(dim=-1)


def shard_race_winner(logits_shard, temperatures, noise_shard, m_all, z_all, index_base):
    """m_all, z_all [world, B] in rank order.  Returns the shard's best value of
    (exp(l / T - M) / Z) / max(noise, 1e-10) per row and its global index (first on ties)."""
    M = m_all.max(dim=0).values
    Z = torch.zeros_like(M)
    for r in range(m_all.shape[0]):                       # rank order, as every rank sums it
        Z = Z + z_all[r] * torch.exp(m_all[r] - M)
    lg = logits_shard.float() / temperatures.unsqueeze(1)
    val = torch.exp(lg - M.unsqueeze(1)) / Z.unsqueeze(1) / noise_shard.clamp_min(1e-10)
    best, idx = val.max(dim=-1)
    return best, idx + index_base


def combine_winners(vals: torch.Tensor, idxs: torch.Tensor) -> torch.Tensor:
    """vals, idxs [world, B]: the larger value wins, then the lower global index."""
    best, besti = vals[0].clone(), idxs[0].clone()
    for r in range(1, vals.shape[0]):
        take = (vals[r] > best) | ((vals[r] == best) & (idxs[r] < besti))
        best, besti = torch.where(take, vals[r], best), torch.where(take, idxs[r], besti)
    return besti


def all_reduce_rank_order(parts, dtype):
    """dist.all_reduce(y) of RowParallelLinear.forward (third_party/nanovllm/layers/linear.py:149-153)
    with the summation order pinned: fp32, rank 0 first, one rounding to the tensor dtype."""
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    return acc.to(dtype)
