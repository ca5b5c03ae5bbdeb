"""Drop-in replacements of the reference's `zipage.kernel` functions.

Same names, argument order and tensor layouts as the reference
(zipage/kernel/*.py and zipage/layers/attention.py:35-50); each call goes
through the C ABI of libzipage_b200.so on the current CUDA stream.  Tensors
must live on the GPU; nothing here computes on the CPU.
"""
from __future__ import annotations

import torch

from .. import _lib as L
from .._lib import SelectParams, ZipageError

__all__ = [
    "store_kvcache", "store_query_cache", "attention_score", "global_score", "key_norm",
    "raw_redudancy_score", "lightning_redudancy_score", "window_mask", "topk_mask",
    "compress_kv", "compress_score", "select_keep", "update_tables",
]


# kernels launched through this module since it was last reset (a plain counter for benchmarks)
LAUNCHES = 0


def _count(n=1):
    global LAUNCHES
    LAUNCHES += n


def _i32(t):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise ZipageError("index tensors must be contiguous int32")
    return t


def _cache5(t, name):
    """[L,P,BS,Hkv,D] view whose three inner dims are contiguous."""
    if t.dim() != 5 or t.stride(-1) != 1 or t.stride(-2) != t.shape[-1] or \
            t.stride(-3) != t.shape[-1] * t.shape[-2]:
        raise ZipageError(f"{name} must be [L,P,BS,Hkv,D] with contiguous (BS,Hkv,D)")
    return t


def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """zipage/layers/attention.py:35-50."""
    L.require_cuda(key, value, k_cache, v_cache, slot_mapping)
    N, H, D = key.shape
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == D and value.stride(1) == D
    assert k_cache.stride(1) == H * D and v_cache.stride(1) == H * D
    assert slot_mapping.numel() == N
    L.check(L.load().zp_store_kv(L.ptr(key), L.ptr(value), L.ptr(k_cache), L.ptr(v_cache),
                                 L.ptr(_i32(slot_mapping)), N, H, D, key.stride(0), value.stride(0),
                                 L.dtype_code(k_cache), L.stream_ptr()), "store_kvcache")
    _count()


def store_query_cache(query, query_cache, slot_mapping, valid_count=None):
    """zipage/kernel/store_query_cache.py:35-68.  `valid_count`: optional device int32 [1] with the
    number of leading rows of `slot_mapping` that are valid (a device-built list of fixed
    capacity); rows past it are not read."""
    if query_cache.numel() == 0:  # warm-up
        return
    L.require_cuda(query, query_cache, slot_mapping, valid_count)
    N, H, D = query.shape
    assert query.stride(-1) == 1 and query.stride(1) == D
    assert query_cache.stride(1) == H * D
    L.check(L.load().zp_store_query(L.ptr(query), L.ptr(query_cache), L.ptr(_i32(slot_mapping)),
                                    slot_mapping.shape[0], H, D, query.stride(0),
                                    query_cache.stride(0), query_cache.stride(1),
                                    L.dtype_code(query_cache), L.ptr(valid_count), N,
                                    query_cache.shape[0], query_cache.shape[1], L.stream_ptr()),
            "store_query_cache")
    _count()


def attention_score(k_cache, query_cache, seq_idx, block_table, softmax_scale=None,
                    reduced="mean", return_logits=False, impl="auto"):
    """zipage/kernel/attention_score.py:133-250 -> [L,B,Hkv,NB,BS]."""
    L.require_cuda(k_cache, query_cache, seq_idx, block_table)
    _cache5(k_cache, "k_cache")
    assert query_cache.is_contiguous() or (query_cache.stride(-1) == 1)
    Ln, _, BS, Hkv, D = k_cache.shape
    _, _, QCL, Hq, _ = query_cache.shape
    B, NB = block_table.shape
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    if reduced not in ("mean", "max"):
        raise ValueError(f"Invalid reduction method: {reduced}")
    scores = torch.empty((Ln, B, Hkv, NB, BS), dtype=k_cache.dtype, device=k_cache.device)
    logits = None
    if return_logits:
        logits = torch.empty((Ln, B, Hq, QCL, NB, BS), dtype=k_cache.dtype, device=k_cache.device)
    lib = L.load()
    need = lib.zp_window_score_workspace_bytes(Ln, B, NB, Hq, Hkv, QCL)
    ws = None
    if need and impl != "simt" and k_cache.dtype != torch.float32 and not return_logits:
        ws = torch.empty(need + 256, dtype=torch.uint8, device=k_cache.device)
    L.check(lib.zp_window_score_ws(
        L.ptr(k_cache), L.ptr(query_cache), L.ptr(_i32(seq_idx)), L.ptr(_i32(block_table)),
        L.ptr(scores), L.ptr(logits), Ln, B, NB, Hq, Hkv, D, QCL, BS, k_cache.stride(0),
        k_cache.stride(1), query_cache.stride(0), query_cache.stride(1), float(softmax_scale),
        0 if reduced == "mean" else 1, L.dtype_code(k_cache), L.IMPL[impl], L.ptr(ws),
        0 if ws is None else ws.numel(), L.stream_ptr()), "attention_score")
    _count()
    if return_logits:
        return scores, logits
    return scores


def global_score(reduced_scores, score_cache, block_table, compressed, decay_factor=0.9,
                 activate_method="max", max_norm=False):
    """zipage/kernel/global_score.py:77-120 (in place); `max_norm` folds in the division by the
    row maximum that model_runner.py:482-487 performs first."""
    L.require_cuda(reduced_scores, score_cache, block_table, compressed)
    assert 0 <= decay_factor <= 1 and activate_method in ("max", "sum")
    Ln, B, Hkv, NB, BS = reduced_scores.shape
    assert reduced_scores.is_contiguous() and score_cache.stride(-1) == 1
    comp = compressed.to(torch.uint8) if compressed.dtype != torch.uint8 else compressed
    L.check(L.load().zp_global_score(
        L.ptr(reduced_scores), L.ptr(score_cache), L.ptr(_i32(block_table)), L.ptr(comp), Ln, B, NB,
        Hkv, BS, score_cache.stride(0), score_cache.stride(1), float(decay_factor),
        0 if activate_method == "max" else 1, int(max_norm), L.dtype_code(reduced_scores),
        L.stream_ptr()), "global_score")
    _count(2 if max_norm else 1)
    return reduced_scores


def key_norm(key_cache, block_table, norm_epsilon=1e-6):
    """zipage/kernel/key_norm.py:72-113 -> [L,B,Hkv,NB,BS]."""
    L.require_cuda(key_cache, block_table)
    _cache5(key_cache, "key_cache")
    Ln, _, BS, Hkv, D = key_cache.shape
    B, NB = block_table.shape
    out = torch.empty((Ln, B, Hkv, NB, BS), dtype=key_cache.dtype, device=key_cache.device)
    L.check(L.load().zp_key_norm(L.ptr(key_cache), L.ptr(_i32(block_table)), L.ptr(out), Ln, B, NB,
                                 Hkv, D, BS, key_cache.stride(0), key_cache.stride(1),
                                 float(norm_epsilon), L.dtype_code(key_cache), L.stream_ptr()),
            "key_norm")
    _count()
    return out


def redundancy_logits(key_cache, block_table, threshold=0.5, exact=True, impl="auto", workspace=None):
    """Row sums of the exempted similarity matrix, [L,B,Hkv,NB,BS] (padded pages -inf)."""
    L.require_cuda(key_cache, block_table)
    _cache5(key_cache, "key_cache")
    Ln, _, BS, Hkv, D = key_cache.shape
    B, NB = block_table.shape
    lib = L.load()
    out = torch.empty((Ln, B, Hkv, NB, BS), dtype=key_cache.dtype, device=key_cache.device)
    common = (L.ptr(key_cache), L.ptr(_i32(block_table)), L.ptr(out), Ln, B, NB, Hkv, D, BS,
              key_cache.stride(0), key_cache.stride(1), float(threshold), L.dtype_code(key_cache),
              L.IMPL[impl])
    if exact:
        need = lib.zp_redundancy_exact_workspace_bytes(Ln, B, NB, Hkv, BS)
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=key_cache.device)
        L.check(lib.zp_redundancy_exact(*common, L.ptr(workspace),
                                        workspace.numel() * workspace.element_size(),
                                        L.stream_ptr()), "raw_redudancy_score")
        _count(2)
    else:
        L.check(lib.zp_redundancy_lightning(*common, L.stream_ptr()), "lightning_redudancy_score")
        _count()
    return out


def _redundancy(key_cache, block_table, threshold, temperature, return_logits, exact, impl):
    logits = redundancy_logits(key_cache, block_table, threshold, exact, impl)
    Ln, B, Hkv, NB, BS = logits.shape
    red = logits.clone() if return_logits else logits
    L.check(L.load().zp_redundancy_softmax(L.ptr(red), L.ptr(block_table), Ln, B, NB, Hkv, BS,
                                           float(temperature), int(exact), L.dtype_code(red),
                                           L.stream_ptr()), "redundancy softmax")
    _count()
    if return_logits:
        return (logits.view(Ln, B, Hkv, -1), red) if exact else (logits, red)
    return red


def raw_redudancy_score(key_cache, block_table, threshold=0.5, temperature=1.0,
                        return_logits=False, impl="auto"):
    """zipage/kernel/raw_redudancy_score.py:158-238."""
    return _redundancy(key_cache, block_table, threshold, temperature, return_logits, True, impl)


def lightning_redudancy_score(key_cache, block_table, threshold=0.5, temperature=1.0,
                              return_logits=False, impl="auto"):
    """zipage/kernel/lightning_redudancy_score.py:172-261."""
    return _redundancy(key_cache, block_table, threshold, temperature, return_logits, False, impl)


def select_keep(scores, block_table, compressed, top_k, query_cache_len, red_logits=None,
                redundancy="none", redudancy_lambda=0.2, redudancy_temperature=0.4,
                redundancy_max_norm=False, pooling_size=0, continues_pooling=False, sink_len=0,
                pad_mask=True, return_final=False):
    """Fused pooling / combine / sink / window / pad masks and top-k of
    zipage/engine/model_runner.py:499-602 -> keep flags [L,B,Hkv,NB,BS] (bool).
    Ties go to the lowest index."""
    L.require_cuda(scores, block_table, compressed, red_logits)
    Ln, B, Hkv, NB, BS = scores.shape
    assert scores.is_contiguous()
    sp = SelectParams()
    sp.top_k, sp.query_cache_len = int(top_k), int(query_cache_len)
    sp.pooling_size, sp.continues_pooling = int(pooling_size), int(continues_pooling)
    sp.use_redundancy = {"none": 0, "lightning": 1, "exact": 2}[redundancy]
    sp.redundancy_max_norm, sp.sink_len, sp.pad_mask = int(redundancy_max_norm), int(sink_len), int(pad_mask)
    sp.redundancy_lambda = float(redudancy_lambda)
    sp.redundancy_one_minus_lambda = float(1 - redudancy_lambda)
    sp.redundancy_temperature = float(redudancy_temperature)
    keep = torch.empty((Ln, B, Hkv, NB, BS), dtype=torch.uint8, device=scores.device)
    final = torch.empty_like(scores) if return_final else None
    comp = compressed.to(torch.uint8) if compressed.dtype != torch.uint8 else compressed
    import ctypes
    L.check(L.load().zp_select(L.ptr(scores), L.ptr(red_logits), L.ptr(_i32(block_table)),
                               L.ptr(comp), L.ptr(keep), L.ptr(final), Ln, B, NB, Hkv, BS,
                               ctypes.byref(sp), L.dtype_code(scores), L.stream_ptr()), "select")
    _count()
    keep = keep.view(torch.bool)
    return (keep, final) if return_final else keep


def window_mask(scores, block_table, query_cache_len):
    """zipage/kernel/window_mask.py:47-72 (in place): last QCL slots of the last page <- +inf."""
    L.require_cuda(scores, block_table)
    Ln, B, Hkv, NB, BS = scores.shape
    sp = SelectParams()
    sp.top_k, sp.query_cache_len = 0, int(query_cache_len)
    comp = torch.zeros(B, dtype=torch.uint8, device=scores.device)
    keep = torch.empty((Ln, B, Hkv, NB, BS), dtype=torch.uint8, device=scores.device)
    import ctypes
    L.check(L.load().zp_select(L.ptr(scores), None, L.ptr(_i32(block_table)), L.ptr(comp),
                               L.ptr(keep), L.ptr(scores), Ln, B, NB, Hkv, BS, ctypes.byref(sp),
                               L.dtype_code(scores), L.stream_ptr()), "window_mask")
    _count()
    return scores


def topk_mask(scores, k):
    """zipage/kernel/utils.py:21-36 with ties resolved to the lowest index.
    scores [L,B,Hkv,N] -> bool mask of the same shape."""
    L.require_cuda(scores)
    Ln, B, Hkv, N = scores.shape
    s5 = scores.contiguous().view(Ln, B, Hkv, 1, N)
    table = torch.zeros((B, 1), dtype=torch.int32, device=scores.device)
    comp = torch.zeros(B, dtype=torch.uint8, device=scores.device)
    keep = select_keep(s5, table, comp, k, 0, pad_mask=False)
    return keep.view(Ln, B, Hkv, N)


def _compact(k, v, sc, flag, block_table, target_block_table, what):
    L.require_cuda(k, v, sc, flag, block_table, target_block_table)
    Ln, B, Hkv, NB, BS = flag.shape
    NT = target_block_table.shape[1]
    f = flag.view(torch.uint8) if flag.dtype == torch.bool else flag
    assert f.is_contiguous()
    ref = k if k is not None else sc
    D = k.shape[-1] if k is not None else 0
    if k is not None:
        _cache5(k, "key"), _cache5(v, "value")
        assert k.stride(0) == v.stride(0) and k.stride(1) == v.stride(1)
    L.check(L.load().zp_compact(
        L.ptr(k), L.ptr(v), L.ptr(sc), L.ptr(f), L.ptr(_i32(block_table)),
        L.ptr(_i32(target_block_table)), Ln, B, NB, NT, Hkv, D, BS,
        k.stride(0) if k is not None else 0, k.stride(1) if k is not None else 0,
        sc.stride(0) if sc is not None else 0, sc.stride(1) if sc is not None else 0,
        L.dtype_code(ref), L.stream_ptr()), what)
    _count()


def compress_kv(key, value, flag, block_table, target_block_table):
    """zipage/kernel/compress_kv.py:103-141 (in place)."""
    _compact(key, value, None, flag, block_table, target_block_table, "compress_kv")


def compress_score(score_cache, flag, block_table, target_block_table):
    """zipage/kernel/compress_score.py:66-99 (in place)."""
    _compact(None, None, score_cache, flag, block_table, target_block_table, "compress_score")
    return score_cache


def compress_kv_and_score(key, value, score_cache, flag, block_table, target_block_table):
    """Both compactions in one launch (same kept rows, same plan)."""
    _compact(key, value, score_cache, flag, block_table, target_block_table, "compress_kv+score")


def update_tables(target_block_table, table_width=None, block_size=256):
    """Device-side table update after a compaction: returns (new_table [B,width] padded with -1,
    context_len [B] = block_size*(NT-1)+1, next_slot [B] = page*block_size); host counterpart:
    zipage/engine/scheduler.py:150-156.  `block_size` is the cache's page size (any multiple of
    256 in the reference, zipage/config.py:48)."""
    B, NT = target_block_table.shape
    width = table_width or NT
    dev = target_block_table.device
    new_table = torch.empty((B, width), dtype=torch.int32, device=dev)
    ctx = torch.empty(B, dtype=torch.int32, device=dev)
    nxt = torch.empty(B, dtype=torch.int32, device=dev)
    L.check(L.load().zp_update_tables(L.ptr(_i32(target_block_table)), L.ptr(new_table), L.ptr(ctx),
                                      L.ptr(nxt), B, NT, width, int(block_size), L.stream_ptr()),
            "update_tables")
    _count()
    return new_table, ctx, nxt
