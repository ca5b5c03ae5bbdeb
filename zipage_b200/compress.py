"""The compression op of `ModelRunner.compress` on the B200 kernels.

`compress_chunk` runs, for one chunk of layers, the stage sequence of the
reference (zipage/engine/model_runner.py:466-622): window scoring -> global
score -> (pooling, redundancy combine, sink/window/pad masks, top-k) ->
in-place compaction of K/V and the score cache.  The reference's ~20 launches
and its [L,B,Hq,QCL,NB,BS] logits buffer become 4-6 kernel launches with
O(L*B*Hkv*NB*BS) scratch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import kernel as K


@dataclass
class CompressConfig:
    """The switches `ModelRunner.compress` reads; names and defaults follow
    zipage/config.py:22-46 (`budget_blocks` is `max_cache_blocks_per_seq`)."""
    budget_blocks: int = 8
    query_cache_len: int = 16
    use_global_score: bool = False
    decay_factor: float = 0.8
    max_norm: bool = False
    use_redudancy: bool = False
    lightning_redudancy: bool = False
    redudancy_lambda: float = 0.2
    redudancy_temperature: float = 0.4
    enable_pooling: bool = False
    continues_pooling: bool = False
    pooling_size: int = 5
    use_attention_sink: bool = False
    sink_len: int = 4
    redudancy_threshold: float = 0.5  # the kernels' default (raw_redudancy_score.py:161)


def compress_chunk(k_cache, v_cache, query_cache, score_cache, query_ids, block_tables,
                   target_block_tables, compressed, cfg: CompressConfig, impl="auto",
                   workspace=None, return_debug=False, timers=None, return_keep=False):
    """Compress B sequences over the L layers of the given cache views, in place.

    k_cache/v_cache [L,P,BS,Hkv,D]; query_cache [L,C,QCL,Hq,D]; score_cache [L,P,BS,Hkv] or None;
    query_ids [B] int32; block_tables [B,NB] int32 (encoded: -1 pad, -(id)-2 last page);
    target_block_tables [B,budget+1] int32; compressed [B] bool.
    `timers`, if given, is a callable name -> context manager used to time the stages under the
    reference's stage names (model_runner.py:425-430).  `return_keep` returns the keep flags
    [L,B,Hkv,NB,BS] the compaction ran with (for accounting; nothing extra is computed).
    """
    BS = k_cache.shape[2]
    stage = timers if timers is not None else (lambda name: _NULL)
    with stage("attention_score"):
        scores = K.attention_score(k_cache, query_cache, query_ids, block_tables, impl=impl)
    if cfg.use_global_score:
        with stage("global_score"):
            K.global_score(scores, score_cache, block_tables, compressed, cfg.decay_factor,
                           max_norm=cfg.max_norm)
    red_logits, mode = None, "none"
    if cfg.use_redudancy:
        with stage("redudancy_score"):
            mode = "lightning" if cfg.lightning_redudancy else "exact"
            red_logits = K.redundancy_logits(k_cache, block_tables, cfg.redudancy_threshold,
                                             exact=not cfg.lightning_redudancy, impl=impl,
                                             workspace=workspace)
    with stage("topk_mask"):
        out = K.select_keep(
            scores, block_tables, compressed, BS * cfg.budget_blocks, cfg.query_cache_len,
            red_logits=red_logits, redundancy=mode, redudancy_lambda=cfg.redudancy_lambda,
            redudancy_temperature=cfg.redudancy_temperature,
            redundancy_max_norm=cfg.use_global_score and cfg.max_norm,
            pooling_size=cfg.pooling_size if cfg.enable_pooling else 0,
            continues_pooling=cfg.continues_pooling,
            sink_len=cfg.sink_len if cfg.use_attention_sink else 0, return_final=return_debug)
    keep, final = out if return_debug else (out, None)
    with stage("compress_kv"):
        K.compress_kv_and_score(k_cache, v_cache, score_cache if cfg.use_global_score else None,
                                keep, block_tables, target_block_tables)
    if return_debug:
        return dict(scores=scores, red_logits=red_logits, final=final, keep=keep)
    return keep if return_keep else None


def compress_batch(k_cache, v_cache, query_cache, score_cache, query_ids, block_tables,
                   target_block_tables, compressed, cfg: CompressConfig, impl="auto", workspace=None,
                   update_tables=False, return_workspace=False):
    """The same op as `compress_chunk` through the single C entry point `zp_compress_batch`
    (one host call, scratch from one workspace tensor).  Returns (new_table, context_len, next_slot)
    device tensors when update_tables is set, else None.  `return_workspace` returns the (possibly
    newly grown) workspace tensor instead, for callers that keep it between calls."""
    import ctypes

    from . import _lib as L
    Ln, _, BS, Hkv, D = k_cache.shape
    _, _, QCL, Hq, _ = query_cache.shape
    B, NB = block_tables.shape
    NT = target_block_tables.shape[1]
    lib = L.load()
    pr = L.CompressParams()
    pr.budget_blocks, pr.query_cache_len = cfg.budget_blocks, cfg.query_cache_len
    pr.use_global_score, pr.max_norm = int(cfg.use_global_score), int(cfg.max_norm)
    pr.redundancy = 0 if not cfg.use_redudancy else (1 if cfg.lightning_redudancy else 2)
    pr.pooling_size = cfg.pooling_size if cfg.enable_pooling else 0
    pr.continues_pooling = int(cfg.continues_pooling)
    pr.sink_len = cfg.sink_len if cfg.use_attention_sink else 0
    pr.decay_factor = cfg.decay_factor
    pr.redundancy_lambda = cfg.redudancy_lambda
    pr.redundancy_one_minus_lambda = 1 - cfg.redudancy_lambda
    pr.redundancy_temperature = cfg.redudancy_temperature
    pr.redundancy_threshold = cfg.redudancy_threshold
    pr.softmax_scale = 0.0
    code = L.dtype_code(k_cache)
    need = lib.zp_compress_batch_workspace_bytes(Ln, B, NB, Hkv, BS, code, pr.redundancy)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=k_cache.device)
    outs = (None, None, None)
    if update_tables:
        dev = k_cache.device
        outs = (torch.empty((B, NT), dtype=torch.int32, device=dev),
                torch.empty(B, dtype=torch.int32, device=dev), torch.empty(B, dtype=torch.int32, device=dev))
    comp = compressed.to(torch.uint8) if compressed.dtype != torch.uint8 else compressed
    sc = score_cache if cfg.use_global_score else None
    L.check(lib.zp_compress_batch(
        L.ptr(k_cache), L.ptr(v_cache), L.ptr(query_cache), L.ptr(sc), L.ptr(query_ids),
        L.ptr(block_tables), L.ptr(target_block_tables), L.ptr(comp), L.ptr(outs[0]), L.ptr(outs[1]),
        L.ptr(outs[2]), Ln, B, NB, NT, Hq, Hkv, D, QCL, BS, k_cache.stride(0), k_cache.stride(1),
        query_cache.stride(0), query_cache.stride(1), sc.stride(0) if sc is not None else 0,
        sc.stride(1) if sc is not None else 0, ctypes.byref(pr), code, L.IMPL[impl], L.ptr(workspace),
        workspace.numel() * workspace.element_size(), L.stream_ptr()), "compress_batch")
    K._count(4 + int(cfg.use_global_score) + int(update_tables))
    if return_workspace:
        return workspace
    return outs if update_tables else None


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL = _Null()
