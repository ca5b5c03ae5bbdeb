"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

They stand in for the math / LongBench workloads the reference was measured on (datasets and
checkpoints are not available offline): K, V ~ N(0,1) and window queries ~ N(0,1) in fp32 then
cast; page ids are a seeded permutation of the pool so tables are non-contiguous.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

BS = 256


@dataclass
class CompressWorkload:
    kv_cache: torch.Tensor       # [2, L, P, BS, Hkv, D]
    query_cache: torch.Tensor    # [L, C, QCL, Hq, D]
    score_cache: torch.Tensor | None  # [L, P, BS, Hkv]
    query_ids: torch.Tensor      # [B] int32
    block_tables: torch.Tensor   # [B, NB] int32, encoded
    target_tables: torch.Tensor  # [B, budget+1] int32
    compressed: torch.Tensor     # [B] bool
    tables_plain: torch.Tensor   # [B, NB] int32 decoded ids (-1 padded)

    @property
    def units(self):
        L, B, Hkv = self.kv_cache.shape[1], self.block_tables.shape[0], self.kv_cache.shape[4]
        return L * B * Hkv


def bytes_per_sequence(L, NB, Hkv, Hq, D, QCL, itemsize, with_score_cache):
    page = L * BS * Hkv * (2 * D + (1 if with_score_cache else 0)) * itemsize
    return NB * page + L * QCL * Hq * D * itemsize


def make_compress_workload(B, L, Hkv, Hq, D=128, QCL=32, budget=8, pages_per_seq=None,
                           dtype=torch.bfloat16, device="cuda", seed=0, with_score_cache=False,
                           compressed_prob=1.0, spare_pages=0, fresh_target_prob=0.0,
                           similar_keys=False):
    """`pages_per_seq`: int or list of table lengths (>= budget+1).  Sequences flagged compressed
    get target == their own first budget+1 pages (repeat compression); with probability
    `fresh_target_prob` an un-compressed sequence gets 1-3 fresh pages at the head of its target
    (first compression with shared prefix pages)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    if pages_per_seq is None:
        pages_per_seq = budget + 1
    lens = [pages_per_seq] * B if isinstance(pages_per_seq, int) else list(pages_per_seq)
    NB = max(lens)
    NT = budget + 1
    n_pages = sum(lens)
    P = n_pages + spare_pages + 3 * B * (1 if fresh_target_prob > 0 else 0)
    perm = torch.randperm(P, generator=gen)
    tables = torch.full((B, NB), -1, dtype=torch.int32)
    pos = 0
    for b, n in enumerate(lens):
        tables[b, :n] = perm[pos:pos + n].to(torch.int32)
        pos += n
    free = perm[pos:].tolist()
    compressed = torch.rand(B, generator=gen) < compressed_prob
    targets = torch.empty((B, NT), dtype=torch.int32)
    for b, n in enumerate(lens):
        if n > NT:
            compressed[b] = False  # a table longer than budget+1 is a first compression
        row = tables[b, :n].tolist()
        if (not bool(compressed[b])) and fresh_target_prob > 0 and \
                float(torch.rand(1, generator=gen)) < fresh_target_prob:
            nfresh = int(torch.randint(1, 4, (1,), generator=gen))
            fresh = [free.pop() for _ in range(nfresh)]
            tgt = fresh + row[nfresh:NT]
        else:
            tgt = row[:NT]
        targets[b] = torch.tensor(tgt, dtype=torch.int32)
    enc = tables.clone()
    for b, n in enumerate(lens):
        enc[b, n - 1] = -enc[b, n - 1] - 2
    dev = torch.device(device)
    kv = torch.empty((2, L, P, BS, Hkv, D), dtype=dtype, device=dev)
    dgen = torch.Generator(device=dev).manual_seed(seed + 1)
    for l in range(L):  # per layer, in place: no temporaries the size of the cache
        kv[0, l].normal_(generator=dgen)
        kv[1, l].normal_(generator=dgen)
    if similar_keys:  # near-duplicate keys so that the similarity threshold is exercised
        for b, n in enumerate(lens):
            a, c = int(tables[b, 0]), int(tables[b, n - 1])
            kv[0, :, c, 16:48] = kv[0, :, a, 64:96] + 0.3 * torch.randn(
                (L, 32, Hkv, D), generator=dgen, device=dev, dtype=torch.float32).to(dtype)
            kv[0, :, a, 200:216] = kv[0, :, a, 100:116] * 1.5
    qc = torch.empty((L, B, QCL, Hq, D), dtype=dtype, device=dev).normal_(generator=dgen)
    sc = None
    if with_score_cache:
        sc = (torch.rand((L, P, BS, Hkv), generator=dgen, device=dev) / (NB * BS)).to(dtype)
    qids = torch.randperm(B, generator=gen).to(torch.int32)
    return CompressWorkload(kv, qc, sc, qids.to(dev), enc.to(dev), targets.to(dev),
                            compressed.to(dev), tables.to(dev))


def algorithmic_bytes_per_unit(NB, D, QCL, G, itemsize, redundancy, global_score, moved_rows):
    """Bytes the op has to move per (layer, sequence, kv head) unit, stage by stage: K read once
    for scoring, the window queries, the score row; K once more for the lightning/exact similarity
    (separate kernel); scores + redundancy read, flags written; compaction reads and writes the
    moved K and V rows (and score scalars)."""
    N = NB * BS
    e = itemsize
    stages = {
        "window_score": N * D * e + G * QCL * D * e + N * e + (2 * N * e if global_score else 0),
        "redundancy": (N * D * e + N * e) if redundancy else 0,
        "select": N * e + (N * e if redundancy else 0) + N,
        "compact": moved_rows * D * e * 2 * 2 + N + (moved_rows * e * 2 if global_score else 0),
    }
    return stages


def shard_kv_heads(w: CompressWorkload, rank: int, world: int) -> CompressWorkload:
    """The slice of a workload that tensor-parallel rank `rank` of `world` owns: KV heads
    [rank*Hkv/world, (rank+1)*Hkv/world) and their query heads (contiguous groups, as the
    reference shards them: third_party/nanovllm/layers/linear.py:106-128).  Tables, targets and
    query ids are replicated.  Units are independent, so no exchange is needed afterwards."""
    Hkv, Hq = w.kv_cache.shape[4], w.query_cache.shape[3]
    assert Hkv % world == 0 and Hq % world == 0
    hk, hq = Hkv // world, Hq // world
    kv = w.kv_cache[:, :, :, :, rank * hk:(rank + 1) * hk].contiguous()
    qc = w.query_cache[:, :, :, rank * hq:(rank + 1) * hq].contiguous()
    sc = None if w.score_cache is None else w.score_cache[..., rank * hk:(rank + 1) * hk].contiguous()
    return CompressWorkload(kv, qc, sc, w.query_ids, w.block_tables, w.target_tables, w.compressed,
                            w.tables_plain)
