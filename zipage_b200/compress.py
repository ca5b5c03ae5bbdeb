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
                   workspace=None, return_debug=False, timers=None):
    """Compress B sequences over the L layers of the given cache views, in place.

    k_cache/v_cache [L,P,BS,Hkv,D]; query_cache [L,C,QCL,Hq,D]; score_cache [L,P,BS,Hkv] or None;
    query_ids [B] int32; block_tables [B,NB] int32 (encoded: -1 pad, -(id)-2 last page);
    target_block_tables [B,budget+1] int32; compressed [B] bool.
    `timers`, if given, is a callable name -> context manager used to time the stages under the
    reference's stage names (model_runner.py:425-430).
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
    return None


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NULL = _Null()
