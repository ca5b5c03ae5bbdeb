"""Attention over the paged (compressed) KV cache.

`Attention` keeps the reference layer's contract (zipage/layers/attention.py:53-104): store this
step's K/V, store the window queries, then varlen causal attention (prefill; paged when a prefix
was cached) or paged decode attention — with the two flash-attn calls and both Triton store
kernels replaced by libzipage_b200 kernels.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _lib as L
from ..kernel import _count, store_kvcache, store_query_cache
from ..utils.context import get_context

_ws_cache: dict = {}


def _workspace(device, nbytes):
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def paged_decode_attention(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale=None):
    """Replaces flash_attn_with_kvcache(q[B,1,Hq,D], k_cache, v_cache, cache_seqlens=...,
    block_table=..., causal=True) as called at zipage/layers/attention.py:95-103."""
    L.require_cuda(q, k_cache, v_cache, cache_seqlens, block_table)
    B, one, Hq, D = q.shape
    assert one == 1 and q.is_contiguous()
    _, BS, Hkv, _ = k_cache.shape
    assert k_cache.stride(2) == D and k_cache.stride(1) == Hkv * D and v_cache.stride() == k_cache.stride()
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    out = torch.empty_like(q)
    lib = L.load()
    ws = _workspace(q.device, lib.zp_paged_decode_workspace_bytes(B, Hq, D, 32))
    L.check(lib.zp_paged_decode(L.ptr(q), L.ptr(k_cache), L.ptr(v_cache), L.ptr(cache_seqlens),
                                L.ptr(block_table), L.ptr(out), B, block_table.shape[1], Hq, Hkv, D,
                                BS, k_cache.stride(0), float(softmax_scale), L.dtype_code(q),
                                L.ptr(ws), ws.numel(), L.stream_ptr()), "paged_decode_attention")
    _count(1)
    return out


def varlen_prefill_attention(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k,
                             softmax_scale=None, block_table=None, impl="auto"):
    """Replaces flash_attn_varlen_func(..., causal=True, block_table=...) as called at
    zipage/layers/attention.py:82-93.  q [sum_q,Hq,D]; k,v dense [sum_k,Hkv,D] or, with
    block_table, the paged caches [P,BS,Hkv,D]."""
    L.require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, block_table)
    _, Hq, D = q.shape
    Hkv = k.shape[-2]
    assert q.is_contiguous()
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    if block_table is None:
        assert k.is_contiguous() and v.is_contiguous()
        BS, stride_page, nbmax = 0, 0, 0
    else:
        BS = k.shape[1]
        assert k.stride(2) == D and k.stride(1) == Hkv * D and v.stride() == k.stride()
        stride_page, nbmax = k.stride(0), block_table.shape[1]
    out = torch.empty_like(q)
    B = cu_seqlens_q.numel() - 1
    total_k = 0 if block_table is not None else k.shape[0]
    L.check(L.load().zp_varlen_prefill_ex(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(cu_seqlens_q),
                                          L.ptr(cu_seqlens_k), L.ptr(block_table), L.ptr(out), B,
                                          int(max_seqlen_q), nbmax, Hq, Hkv, D, BS, stride_page,
                                          float(softmax_scale), q.shape[0], total_k, L.IMPL[impl],
                                          L.dtype_code(q), L.stream_ptr()),
            "varlen_prefill_attention")
    _count(1)
    return out


class Attention(nn.Module):
    """Drop-in for zipage.layers.attention.Attention (same constructor, same cache attributes)."""

    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])
        self.q_cache = torch.tensor([])

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        context = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if k_cache.numel() and v_cache.numel():
            store_kvcache(k, v, k_cache, v_cache, context.slot_mapping)
        if context.query_slot_mapping is not None:
            # a device-built triple list has fixed capacity; only its first query_slot_count rows count
            store_query_cache(q, self.q_cache, context.query_slot_mapping,
                              getattr(context, "query_slot_count", None))
        return self.attend(q, k, v)

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
        """The attention call alone, for callers that wrote the caches already (the fused
        q/k normalisation + rotation + store launch)."""
        context = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if context.is_prefill:
            if context.block_tables is not None:  # prefix cache: keys come from the pages
                k, v = k_cache, v_cache
            return varlen_prefill_attention(
                q.contiguous(), k if context.block_tables is not None else k.contiguous(),
                v if context.block_tables is not None else v.contiguous(),
                context.max_seqlen_q, context.cu_seqlens_q, context.max_seqlen_k,
                context.cu_seqlens_k, self.scale, context.block_tables)
        return paged_decode_attention(q.contiguous().unsqueeze(1), k_cache, v_cache,
                                      context.context_lens, context.block_tables, self.scale)
