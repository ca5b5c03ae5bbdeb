"""CPU oracle for the compressed-PagedAttention hot path (TEST INFRASTRUCTURE).

This module is the checker, never the product: only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import it.  It is a
PyTorch-on-CPU restatement of what the reference computes, one function per
reference function, keeping the reference's argument order and tensor layouts.
Where the reference stores an intermediate in the model dtype ``T`` the oracle
rounds at the same place, so that bf16 and fp32 runs follow the same rounding
points as the reference's kernels.

Parity pins: the functions of the compression op are pinned against golden
vectors produced by running the unmodified reference (its Triton kernels under
the Triton CPU interpreter, and its ``ModelRunner.compress`` glue) in fp32; the
generator is ``tests/golden/make_golden.py``.  The two attention functions
(`flash_attn_with_kvcache`, `flash_attn_varlen_func`) live in the third-party
flash-attn package, which cannot execute without a GPU: for those two the
oracle restates the published softmax-attention formula and their
parity is UNPINNED.

Block-table encoding used by every function of the compression op
(reference: zipage/engine/model_runner.py:440-441): ``-1`` is padding, an id
``>= 0`` is an ordinary page, ``-(id) - 2`` marks the last page of the sequence
(the page that holds the observation window).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

NEG_INF = float("-inf")
POS_INF = float("inf")


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def decode_block_table(block_table: torch.Tensor):
    """Split an encoded table into (page ids, valid mask, last-page mask).

    Padding entries get page id 0 (never dereferenced by callers that honour
    the valid mask).  Encoding: zipage/kernel/attention_score.py:81-86.
    """
    bt = block_table.to(torch.int64)
    valid = bt != -1
    last = bt < -1
    ids = torch.where(last, -bt - 2, bt)
    ids = torch.where(valid, ids, torch.zeros_like(ids))
    return ids, valid, last


def _gather_keys(k_cache: torch.Tensor, ids_row: torch.Tensor) -> torch.Tensor:
    """k_cache [L,P,BS,Hkv,D], ids_row [NB] -> [L,Hkv,NB*BS,D] (no dtype change)."""
    L, _, BS, Hkv, D = k_cache.shape
    pages = k_cache[:, ids_row]  # [L,NB,BS,Hkv,D]
    return pages.permute(0, 3, 1, 2, 4).reshape(L, Hkv, -1, D)


# --------------------------------------------------------------------------
# a1 / a2: cache writes
# --------------------------------------------------------------------------
def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """Scatter this step's K/V rows into the paged cache.

    Follows zipage/layers/attention.py:12-50: row i goes to flat slot
    ``slot_mapping[i]`` (= page*block_size + position in page); slot -1 is
    skipped.  Caches are [P, BS, Hkv, D] and are modified in place.
    """
    N, H, D = key.shape
    kc = k_cache.view(-1, H, D)
    vc = v_cache.view(-1, H, D)
    sm = slot_mapping.to(torch.int64)
    for i in range(N):  # later rows win on duplicate slots, as a serial scatter would
        s = int(sm[i])
        if s == -1:
            continue
        kc[s] = key[i]
        vc[s] = value[i]


def store_query_cache(query, query_cache, slot_mapping):
    """Observation-window buffer write.

    Follows zipage/kernel/store_query_cache.py:7-68: for every triple
    (row, query_id, idx) copy query[row] ([Hq, D]) to query_cache[query_id, idx].
    query_cache is [C, QCL, Hq, D]; an empty cache makes the call a no-op.
    """
    if query_cache.numel() == 0:
        return
    for row, qid, idx in slot_mapping.tolist():
        query_cache[qid, idx] = query[row]


# --------------------------------------------------------------------------
# a3: window-masked attention scoring
# --------------------------------------------------------------------------
def attention_logits(k_cache, query_cache, seq_idx, block_table, softmax_scale=None):
    """Logits buffer [L,B,Hq,QCL,NB*BS] in the cache dtype, -inf where masked.

    Follows zipage/kernel/attention_score.py:44-130 (and the PyTorch statement
    of the same thing in tests/test_attention_score.py:248-296): fp32 dot
    product, times the scale, causal mask inside the last page
    (column > BS - QCL + row is masked), rounded to the cache dtype; padded
    pages stay at the buffer's -inf fill.
    """
    L, _, BS, Hkv, D = k_cache.shape
    _, _, QCL, Hq, _ = query_cache.shape
    B, NB = block_table.shape
    G = Hq // Hkv
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    ids, valid, last = decode_block_table(block_table)
    out = torch.full((L, B, Hq, QCL, NB * BS), NEG_INF, dtype=k_cache.dtype)
    col = torch.arange(BS)[None, :]
    row = torch.arange(BS - QCL, BS)[:, None]
    causal = col > row  # [QCL, BS]
    for b in range(B):
        keys = _gather_keys(k_cache, ids[b]).float()  # [L,Hkv,N,D]
        q = query_cache[:, int(seq_idx[b])].float()  # [L,QCL,Hq,D]
        q = q.permute(0, 2, 1, 3).reshape(L, Hkv, G * QCL, D)
        qk = torch.matmul(q, keys.transpose(-1, -2)) * softmax_scale  # [L,Hkv,G*QCL,N]
        qk = qk.view(L, Hkv, G, QCL, NB, BS)
        pad = ~valid[b]
        qk = qk.masked_fill(pad[None, None, None, None, :, None], NEG_INF)
        lastm = last[b][None, None, None, None, :, None] & causal[None, None, None, :, None, :]
        qk = qk.masked_fill(lastm, NEG_INF)
        out[:, b] = qk.reshape(L, Hq, QCL, NB * BS).to(k_cache.dtype)
    return out


def attention_score(
    k_cache,
    query_cache,
    seq_idx,
    block_table,
    softmax_scale=None,
    reduced="mean",
    return_logits=False,
):
    """Per-token importance score [L,B,Hkv,NB,BS] in the cache dtype.

    Follows zipage/kernel/attention_score.py:133-250: softmax over the whole
    sequence (in the cache dtype), max over the query heads of a KV group,
    then mean (or max) over the window rows.
    """
    L, _, BS, Hkv, D = k_cache.shape
    _, _, QCL, Hq, _ = query_cache.shape
    B, NB = block_table.shape
    G = Hq // Hkv
    logits = attention_logits(k_cache, query_cache, seq_idx, block_table, softmax_scale)
    x = logits - logits.max(dim=-1, keepdim=True).values
    p = torch.softmax(x, dim=-1)
    if G > 1:
        p = p.view(L, B, Hkv, G, QCL, -1).max(dim=3).values
    p = p.reshape(L, B, Hkv, QCL, NB, BS)
    if reduced == "mean":
        # one rounding, as the CUDA mean reduction the reference runs does
        s = (p.float().sum(dim=3) / QCL).to(p.dtype)
    elif reduced == "max":
        s = p.max(dim=3).values
    else:
        raise ValueError(f"Invalid reduction method: {reduced}")
    if return_logits:
        return s, logits.view(L, B, Hq, QCL, NB, BS)
    return s


# --------------------------------------------------------------------------
# a4: global score
# --------------------------------------------------------------------------
def global_score(
    reduced_scores,
    score_cache,
    block_table,
    compressed,
    decay_factor=0.9,
    activate_method="max",
):
    """Merge new scores with the persisted ones; both tensors change in place.

    Follows zipage/kernel/global_score.py:8-120.  For a sequence that was
    compressed before, every page except its last one merges
    ``max(new, cache*decay)`` (or the sum); everything else takes the new
    score.  The result is written to the score tensor and to score_cache
    [L,P,BS,Hkv].  In a 16-bit dtype the decay scalar and the product are
    rounded to that dtype, as a Triton scalar*tensor multiply does.
    """
    assert 0 <= decay_factor <= 1 and activate_method in ("max", "sum")
    L, B, Hkv, NB, BS = reduced_scores.shape
    T = reduced_scores.dtype
    ids, valid, last = decode_block_table(block_table)
    decay_t = torch.tensor(decay_factor, dtype=T)
    for b in range(B):
        for m in range(NB):
            if not bool(valid[b, m]):
                continue
            pid = int(ids[b, m])
            new = reduced_scores[:, b, :, m, :]  # [L,Hkv,BS]
            if bool(compressed[b]) and not bool(last[b, m]):
                cache = score_cache[:, pid].permute(0, 2, 1)  # [L,Hkv,BS]
                decayed = cache * decay_t
                if activate_method == "max":
                    out = torch.maximum(new, decayed)
                else:
                    out = (new.float() + decayed.float()).to(T)
            else:
                out = new
            out = out.clone()
            reduced_scores[:, b, :, m, :] = out
            score_cache[:, pid] = out.permute(0, 2, 1)
    return reduced_scores


def max_norm_(x4):
    """In-place divide by the per-(layer, seq, head) maximum over the sequence.

    Follows zipage/engine/model_runner.py:482-487 and :551-558; x4 is
    [L,B,Hkv,NB,BS] (viewed flat over the last two axes).
    """
    L, B, Hkv, NB, BS = x4.shape
    flat = x4.view(L, B, Hkv, -1)
    flat.div_(flat.max(dim=-1, keepdim=True).values)
    return x4


# --------------------------------------------------------------------------
# a5: pooling along tokens
# --------------------------------------------------------------------------
def pool_scores(scores, compressed, pooling_size=5, continues_pooling=False):
    """Max-pool along the concatenated token axis.

    Follows zipage/engine/model_runner.py:499-530: kernel ``pooling_size``
    (the reference hard-codes 5), stride 1, -inf padding; sequences that were
    compressed before keep their un-pooled scores unless continues_pooling;
    when every sequence was compressed before the stage is skipped.
    """
    L, B, Hkv, NB, BS = scores.shape
    if not continues_pooling and bool(torch.all(compressed)):
        return scores
    flat = scores.reshape(L * B, Hkv, NB * BS)
    pooled = F.max_pool1d(
        flat.float(), kernel_size=pooling_size, stride=1, padding=pooling_size // 2
    ).to(scores.dtype)
    if not continues_pooling:
        cm = compressed.view(1, B).expand(L, B).reshape(L * B, 1, 1)
        flat = torch.where(cm, flat, pooled)
    else:
        flat = pooled
    return flat.view(L, B, Hkv, NB, BS)


# --------------------------------------------------------------------------
# a6: key norm
# --------------------------------------------------------------------------
def key_norm(key_cache, block_table, norm_epsilon=1e-6):
    """L2 norm of every key, [L,B,Hkv,NB,BS] in the cache dtype, floor 1e-6.

    Follows zipage/kernel/key_norm.py:8-113: fp32 accumulate, rounded to the
    cache dtype, padded pages 0 before the clamp.
    """
    L, _, BS, Hkv, D = key_cache.shape
    B, NB = block_table.shape
    ids, valid, _ = decode_block_table(block_table)
    out = torch.zeros((L, B, Hkv, NB, BS), dtype=key_cache.dtype)
    for b in range(B):
        keys = _gather_keys(key_cache, ids[b]).float()  # [L,Hkv,N,D]
        n = torch.sqrt((keys * keys).sum(dim=-1)).to(key_cache.dtype)
        n = n.view(L, Hkv, NB, BS)
        n = n * valid[b][None, None, :, None].to(n.dtype)
        out[:, b] = n
    return torch.clamp(out, min=norm_epsilon)


def _exempt_latest_similar(S, threshold):
    """Zero, in every column, the entry of the LARGEST row whose value exceeds
    the threshold (zipage/kernel/raw_redudancy_score.py:83-142: rows are
    visited in descending order and a column is exempted once)."""
    above = S > threshold
    n_rows = S.shape[-2]
    ridx = torch.arange(n_rows).view(-1, 1).expand_as(S)
    latest = torch.where(above, ridx, torch.full_like(ridx, -1)).max(dim=-2, keepdim=True).values
    hit = ridx == latest
    return torch.where(hit, torch.zeros_like(S), S)


# --------------------------------------------------------------------------
# a7: exact key-similarity redundancy
# --------------------------------------------------------------------------
def raw_redudancy_score(
    key_cache, block_table, threshold=0.5, temperature=1.0, return_logits=False
):
    """Exact redundancy [L,B,Hkv,NB,BS] in the cache dtype.

    Follows zipage/kernel/raw_redudancy_score.py:10-238 (PyTorch statement of
    the same maths: tests/test_redudancy_paged.py:17-94).  Cosine similarity
    of every key pair of the sequence, diagonal zeroed, the latest similar key
    of every column exempted, row sums, divide by temperature*length, softmax
    over the sequence.  Rounding points kept: the norm is stored in the cache
    dtype; normalised keys and the dot product are fp32; the running row sum
    of each (row, column page) is stored in the cache dtype after each
    16-column tile (:143-155); the column pages are then summed (:218).
    """
    L, _, BS, Hkv, D = key_cache.shape
    B, NB = block_table.shape
    T = key_cache.dtype
    TILE_N = 16
    ids, valid, _ = decode_block_table(block_table)
    norm = key_norm(key_cache, block_table)  # [L,B,Hkv,NB,BS] T
    red = torch.zeros((L, B, Hkv, NB, NB * BS), dtype=T)  # [.., col page, row token]
    for b in range(B):
        vidx = torch.nonzero(valid[b]).flatten()  # table positions of real pages
        nv = int(vidx.numel())
        if nv == 0:
            continue
        keys = _gather_keys(key_cache, ids[b][vidx]).float()  # [L,Hkv,nv*BS,D]
        nrm = norm[:, b][:, :, vidx].reshape(L, Hkv, nv * BS, 1).float()
        kh = keys / nrm
        for l in range(L):
            for h in range(Hkv):
                S = kh[l, h] @ kh[l, h].t()  # [n, n] rows m, cols n
                S.fill_diagonal_(0.0)
                S = _exempt_latest_similar(S, threshold)
                tiles = S.view(nv * BS, nv, BS // TILE_N, TILE_N).sum(dim=-1)
                acc = torch.zeros((nv * BS, nv), dtype=T)
                for t in range(BS // TILE_N):
                    acc = (acc.float() + tiles[:, :, t]).to(T)
                # acc[m_token, n_page] -> red[n_page(table pos), m_token(table pos)]
                rows = (vidx[:, None] * BS + torch.arange(BS)[None, :]).flatten()
                for j in range(nv):
                    red[l, b, h, int(vidx[j]), rows] = acc[:, j]
    red = red.view(L, B, Hkv, NB, NB, BS).sum(dim=-3)  # [L,B,Hkv,NB,BS]
    pad = (block_table == -1)[None, :, None, :, None]
    red = red.masked_fill(pad, NEG_INF)
    red = red.view(L, B, Hkv, -1)
    logits = red.clone() if return_logits else None
    seq_length = (block_table != -1).sum(dim=-1) * BS
    red = red.div_(temperature * seq_length.view(1, B, 1, 1))
    red = red - red.max(dim=-1, keepdim=True).values
    red = red.softmax(dim=-1).reshape(L, B, Hkv, NB, BS)
    if return_logits:
        return logits, red
    return red


# --------------------------------------------------------------------------
# a8: "lightning" (per-page) key-similarity redundancy
# --------------------------------------------------------------------------
def lightning_redudancy_score(
    key_cache, block_table, threshold=0.5, temperature=1.0, return_logits=False
):
    """Per-page redundancy [L,B,Hkv,NB,BS] in the cache dtype.

    Follows zipage/kernel/lightning_redudancy_score.py:10-261 (PyTorch
    statement: tests/test_lightning_redudancy.py:16-91): the same maths as the
    exact form restricted to key pairs of the same page; the fp32 row sum is
    rounded once to the cache dtype (:169); divide by temperature*block_size;
    softmax over the whole sequence, padded pages at -inf.
    """
    L, _, BS, Hkv, D = key_cache.shape
    B, NB = block_table.shape
    T = key_cache.dtype
    ids, valid, _ = decode_block_table(block_table)
    norm = key_norm(key_cache, block_table)
    red = torch.full((L, B, Hkv, NB, BS), NEG_INF, dtype=T)
    for b in range(B):
        for m in range(NB):
            if not bool(valid[b, m]):
                continue
            keys = key_cache[:, int(ids[b, m])].permute(0, 2, 1, 3).float()  # [L,Hkv,BS,D]
            kh = keys / norm[:, b, :, m, :, None].float()
            S = kh @ kh.transpose(-1, -2)  # [L,Hkv,BS,BS]
            eye = torch.eye(BS, dtype=torch.bool)
            S = S.masked_fill(eye, 0.0)
            S = _exempt_latest_similar(S, threshold)
            red[:, b, :, m, :] = S.sum(dim=-1).to(T)
    logits = red.clone() if return_logits else None
    red = red.view(L, B, Hkv, -1)
    red = red.div_(temperature * BS)
    red = red - red.max(dim=-1, keepdim=True).values
    red = red.softmax(dim=-1).reshape(L, B, Hkv, NB, BS)
    if return_logits:
        return logits, red
    return red


# --------------------------------------------------------------------------
# a9: combine / sink / window / pad masks
# --------------------------------------------------------------------------
def combine_scores(scores, redudancy, redudancy_lambda):
    """score*lambda - redundancy*(1-lambda), each product and the difference
    rounded to the cache dtype (zipage/engine/model_runner.py:559-561)."""
    return scores * redudancy_lambda - redudancy * (1 - redudancy_lambda)


def attention_sink_(scores, sink_len):
    """First sink_len tokens of the table order <- +inf
    (zipage/engine/model_runner.py:566-578)."""
    L, B, Hkv, NB, BS = scores.shape
    flat = scores.view(L, B, Hkv, -1)
    flat[..., :sink_len] = POS_INF
    return scores


def window_mask(scores, block_table, query_cache_len):
    """Last query_cache_len slots of the last page <- +inf
    (zipage/kernel/window_mask.py:8-72); in place."""
    _, _, last = decode_block_table(block_table)
    B, NB = block_table.shape
    BS = scores.shape[-1]
    for b in range(B):
        for m in range(NB):
            if bool(last[b, m]):
                scores[:, b, :, m, BS - query_cache_len :] = POS_INF
    return scores


def pad_mask_(scores, block_table):
    """Padded pages <- -inf (zipage/engine/model_runner.py:592-593)."""
    pad = (block_table == -1)[None, :, None, :, None]
    return scores.masked_fill_(pad, NEG_INF)


# --------------------------------------------------------------------------
# a10: top-k keep flags
# --------------------------------------------------------------------------
def topk_mask(scores, k):
    """Keep flags of the k largest entries of the last axis.

    Follows zipage/kernel/utils.py:21-36 with one thing made definite: the
    reference's torch.topk leaves the order of equal values unspecified; here
    ties go to the LOWEST index (stable descending sort).
    """
    order = torch.sort(scores.float(), dim=-1, descending=True, stable=True).indices
    mask = torch.zeros_like(scores, dtype=torch.bool)
    mask.scatter_(-1, order[..., :k], True)
    return mask


def topk_mask_agrees_with_unordered(scores, k, mask):
    """True when `mask` is a valid answer of an order-unspecified top-k: every
    entry strictly above the k-th value is kept, nothing strictly below it is,
    and exactly k are kept.  Used to compare against the literal reference."""
    kth = torch.sort(scores.float(), dim=-1, descending=True).values[..., k - 1 : k]
    above = scores.float() > kth
    below = scores.float() < kth
    ok = (mask | ~above).all() and (~(mask & below)).all()
    return bool(ok) and bool((mask.sum(-1) == k).all())


# --------------------------------------------------------------------------
# a11 / a12: in-place compaction
# --------------------------------------------------------------------------
def _compaction_plan(flag_row, ids_row, valid_row, target_row, BS):
    """(src page, src slot, dst page, dst slot) lists for one (layer, seq, head)."""
    NB = ids_row.numel()
    src_p, src_s = [], []
    fl = flag_row.view(NB, BS)
    for m in range(NB):
        if not bool(valid_row[m]):
            continue
        slots = torch.nonzero(fl[m]).flatten()
        src_p.append(torch.full_like(slots, int(ids_row[m])))
        src_s.append(slots)
    src_p = torch.cat(src_p) if src_p else torch.zeros(0, dtype=torch.int64)
    src_s = torch.cat(src_s) if src_s else torch.zeros(0, dtype=torch.int64)
    n = src_p.numel()
    pos = torch.arange(n)
    dst_p = target_row.to(torch.int64)[pos // BS] if n else src_p
    dst_s = pos % BS
    return src_p, src_s, dst_p, dst_s


def compress_kv(key, value, flag, block_table, target_block_table):
    """Stable forward compaction of the kept K and V rows, in place.

    Follows zipage/kernel/compress_kv.py:8-141: for every (layer, seq, kv
    head), walk the table in order, and copy each kept row to the next free
    slot of the pages listed in target_block_table.  The reference does this
    serially in place; it is only well defined when every destination lies at
    or before the row being read, which the engine guarantees
    (zipage/engine/block_manager.py:129-169).  Under that guarantee the serial
    walk equals "gather all kept rows, then write them", which is what is done
    here; `compress_kv_serial` is the literal walk.
    key/value: [L,P,BS,Hkv,D]; flag: [L,B,Hkv,NB,BS] bool.
    """
    L, _, BS, Hkv, D = key.shape
    B = flag.shape[1]
    ids, valid, _ = decode_block_table(block_table)
    for l in range(L):
        for b in range(B):
            for h in range(Hkv):
                sp, ss, dp, ds = _compaction_plan(
                    flag[l, b, h], ids[b], valid[b], target_block_table[b], BS
                )
                if sp.numel() == 0:
                    continue
                krows = key[l, sp, ss, h].clone()
                vrows = value[l, sp, ss, h].clone()
                key[l, dp, ds, h] = krows
                value[l, dp, ds, h] = vrows


def compress_kv_serial(key, value, flag, block_table, target_block_table):
    """The literal slot-by-slot walk of zipage/kernel/compress_kv.py:50-100
    (slow; used on small cases to check `compress_kv`)."""
    L, _, BS, Hkv, D = key.shape
    B, NB = block_table.shape
    ids, valid, _ = decode_block_table(block_table)
    tgt = target_block_table.to(torch.int64)
    for l in range(L):
        for b in range(B):
            for h in range(Hkv):
                pos = 0
                for m in range(NB):
                    if not bool(valid[b, m]):
                        continue
                    pid = int(ids[b, m])
                    for s in torch.nonzero(flag[l, b, h, m]).flatten().tolist():
                        dp = int(tgt[b, pos // BS])
                        key[l, dp, pos % BS, h] = key[l, pid, s, h]
                        value[l, dp, pos % BS, h] = value[l, pid, s, h]
                        pos += 1


def compress_score(score_cache, flag, block_table, target_block_table):
    """The same compaction for score_cache [L,P,BS,Hkv]
    (zipage/kernel/compress_score.py:8-99)."""
    L, _, BS, Hkv = score_cache.shape
    B = flag.shape[1]
    ids, valid, _ = decode_block_table(block_table)
    for l in range(L):
        for b in range(B):
            for h in range(Hkv):
                sp, ss, dp, ds = _compaction_plan(
                    flag[l, b, h], ids[b], valid[b], target_block_table[b], BS
                )
                if sp.numel() == 0:
                    continue
                vals = score_cache[l, sp, ss, h].clone()
                score_cache[l, dp, ds, h] = vals
    return score_cache


# --------------------------------------------------------------------------
# a15: the whole compression op for one chunk of layers
# --------------------------------------------------------------------------
class CompressConfig:
    """The switches `ModelRunner.compress` reads (zipage/config.py:22-46,
    zipage/engine/model_runner.py:51-71)."""

    def __init__(
        self,
        budget_blocks=8,
        query_cache_len=16,
        use_global_score=False,
        decay_factor=0.8,
        max_norm=False,
        use_redudancy=False,
        lightning_redudancy=False,
        redudancy_lambda=0.2,
        redudancy_temperature=0.4,
        enable_pooling=False,
        continues_pooling=False,
        pooling_size=5,
        use_attention_sink=False,
        sink_len=4,
    ):
        self.__dict__.update(locals())
        del self.__dict__["self"]


def compress_scores(k_cache, query_cache, score_cache, query_ids, block_tables, compressed, cfg,
                    parts=None):
    """Stages attention_score .. pad mask of zipage/engine/model_runner.py:471-593.

    Returns the final selection scores [L,B,Hkv,NB,BS] (cache dtype) and
    updates score_cache in place when the global score is on.  `parts`, if a
    dict, receives the two terms of the combination (`score_term`, `red_term`;
    model_runner.py:559-561) for the kept-set boundary check.
    """
    scores = attention_score(k_cache, query_cache, query_ids, block_tables)
    if cfg.use_global_score:
        if cfg.max_norm:
            scores = max_norm_(scores.contiguous())
        scores = global_score(scores, score_cache, block_tables, compressed, cfg.decay_factor)
    if cfg.enable_pooling:
        scores = pool_scores(scores, compressed, cfg.pooling_size, cfg.continues_pooling)
    if cfg.use_redudancy:
        fn = lightning_redudancy_score if cfg.lightning_redudancy else raw_redudancy_score
        red = fn(k_cache, block_tables, temperature=cfg.redudancy_temperature)
        if cfg.use_global_score and cfg.max_norm:
            red = max_norm_(red.contiguous())
        if parts is not None:
            parts["score_term"] = (scores * cfg.redudancy_lambda).clone()
            parts["red_term"] = (red * (1 - cfg.redudancy_lambda)).clone()
        scores = combine_scores(scores, red, cfg.redudancy_lambda)
    elif parts is not None:
        parts["score_term"] = scores.clone()
        parts["red_term"] = None
    scores = scores.contiguous()
    if cfg.use_attention_sink:
        attention_sink_(scores, cfg.sink_len)
    window_mask(scores, block_tables, cfg.query_cache_len)
    pad_mask_(scores, block_tables)
    return scores


def compress(k_cache, v_cache, query_cache, score_cache, query_ids, block_tables,
             target_block_tables, compressed, cfg, parts=None):
    """One chunk of `ModelRunner.compress` (zipage/engine/model_runner.py:466-622).

    k_cache/v_cache [L,P,BS,Hkv,D], query_cache [L,C,QCL,Hq,D], score_cache
    [L,P,BS,Hkv] or None.  Caches change in place.  Returns (final scores,
    keep flags) for inspection.
    """
    L, _, BS, Hkv, D = k_cache.shape
    B, NB = block_tables.shape
    scores = compress_scores(k_cache, query_cache, score_cache, query_ids, block_tables,
                             compressed, cfg, parts=parts)
    keep = topk_mask(scores.view(L, B, Hkv, -1), BS * cfg.budget_blocks).view(L, B, Hkv, NB, BS)
    compress_kv(k_cache, v_cache, keep, block_tables, target_block_tables)
    if cfg.use_global_score:
        compress_score(score_cache, keep, block_tables, target_block_tables)
    return scores, keep


# --------------------------------------------------------------------------
# a13 / a14: attention over the paged cache  (parity UNPINNED: flash-attn is a
# third-party dependency whose code is not part of the reference tree)
# --------------------------------------------------------------------------
def paged_decode_attention(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale=None):
    """One query token per sequence against its paged K/V.

    Call site: zipage/layers/attention.py:95-103 (`flash_attn_with_kvcache`,
    causal, one query = attends to all `cache_seqlens[b]` cached tokens).
    q [B,1,Hq,D]; caches [P,BS,Hkv,D]; block_table [B,NBmax] (-1 padded).
    fp32 maths, output in q's dtype.
    """
    B, _, Hq, D = q.shape
    _, BS, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    out = torch.empty_like(q)
    for b in range(B):
        n = int(cache_seqlens[b])
        npg = (n + BS - 1) // BS
        pages = block_table[b, :npg].to(torch.int64)
        k = k_cache[pages].reshape(npg * BS, Hkv, D)[:n].float()
        v = v_cache[pages].reshape(npg * BS, Hkv, D)[:n].float()
        qb = q[b, 0].float().view(Hkv, G, D)
        s = torch.einsum("hgd,nhd->hgn", qb, k) * softmax_scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgn,nhd->hgd", p, v)
        out[b, 0] = o.reshape(Hq, D).to(q.dtype)
    return out


def varlen_prefill_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale=None,
                             block_table=None):
    """Causal variable-length attention, bottom-right aligned.

    Call site: zipage/layers/attention.py:79-93 (`flash_attn_varlen_func`).
    q [sum_q,Hq,D].  Without block_table k/v are dense [sum_k,Hkv,D]; with it
    they are the paged caches [P,BS,Hkv,D] and sequence b's keys are the first
    len_k tokens of its pages.  Query i of a sequence (0-based, len_q queries,
    len_k keys) sees keys j <= i + len_k - len_q.
    """
    Hq, D = q.shape[1:]
    Hkv = k.shape[-2]
    G = Hq // Hkv
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    out = torch.empty_like(q)
    B = cu_seqlens_q.numel() - 1
    for b in range(B):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        k0, k1 = int(cu_seqlens_k[b]), int(cu_seqlens_k[b + 1])
        lq, lk = q1 - q0, k1 - k0
        if lq == 0:
            continue
        if block_table is None:
            kb, vb = k[k0:k1].float(), v[k0:k1].float()
        else:
            BS = k.shape[1]
            npg = (lk + BS - 1) // BS
            pages = block_table[b, :npg].to(torch.int64)
            kb = k[pages].reshape(npg * BS, Hkv, D)[:lk].float()
            vb = v[pages].reshape(npg * BS, Hkv, D)[:lk].float()
        qb = q[q0:q1].float().view(lq, Hkv, G, D)
        s = torch.einsum("qhgd,nhd->hgqn", qb, kb) * softmax_scale
        qi = torch.arange(lq)[:, None]
        kj = torch.arange(lk)[None, :]
        s = s.masked_fill((kj > qi + (lk - lq))[None, None], NEG_INF)
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgqn,nhd->qhgd", p, vb)
        out[q0:q1] = o.reshape(lq, Hq, D).to(q.dtype)
    return out
