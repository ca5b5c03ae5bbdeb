"""The per-step ops around the attention path on libzipage_b200 kernels.

Same names and call contracts as the reference modules they replace:
`RMSNorm` (third_party/nanovllm/layers/layernorm.py), `SiluAndMul`
(third_party/nanovllm/layers/activation.py), `Sampler` (zipage/layers/sampler.py);
`qk_norm_rope_store` replaces the q/k normalisation + rotation of `Qwen3Attention.forward`
(third_party/nanovllm/models/qwen3.py:75-79) together with the two cache writes at the head of
`Attention.forward` (zipage/layers/attention.py:72-77); `prepare_decode` replaces the host loop of
`ModelRunner.prepare_decode` (zipage/engine/model_runner.py:633-675) from device-resident state.
There is no CPU path: non-CUDA tensors are rejected.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _lib as L
from ..kernel import _count


def rms_norm(x, weight, eps, residual=None):
    """x [..., H]; returns out, or (out, new_residual) when a residual is given."""
    L.require_cuda(x, weight, residual)
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    assert x2.stride(-1) == 1 and weight.is_contiguous() and weight.dtype == x.dtype
    out = torch.empty((x2.shape[0], H), dtype=x.dtype, device=x.device)
    res_out = None
    if residual is not None:
        residual = residual.reshape(-1, H)
        assert residual.is_contiguous() and residual.dtype == x.dtype
        res_out = torch.empty_like(residual)
    L.check(L.load().zp_rms_norm(L.ptr(x2), L.ptr(residual), L.ptr(weight), L.ptr(out), L.ptr(res_out),
                                 x2.shape[0], H, x2.stride(0), out.stride(0), float(eps),
                                 L.dtype_code(x), L.stream_ptr()), "rms_norm")
    _count(1)
    out = out.view(x.shape)
    return out if residual is None else (out, res_out.view(x.shape))


class RMSNorm(nn.Module):
    """layernorm.py:5-50."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x, residual=None):
        return rms_norm(x, self.weight, self.eps, residual)


def silu_and_mul(x):
    L.require_cuda(x)
    two_i = x.shape[-1]
    x2 = x.reshape(-1, two_i)
    assert x2.is_contiguous() and two_i % 2 == 0
    out = torch.empty((x2.shape[0], two_i // 2), dtype=x.dtype, device=x.device)
    L.check(L.load().zp_silu_and_mul(L.ptr(x2), L.ptr(out), x2.shape[0], two_i // 2, L.dtype_code(x),
                                     L.stream_ptr()), "silu_and_mul")
    _count(1)
    return out.view(*x.shape[:-1], two_i // 2)


class SiluAndMul(nn.Module):
    """activation.py:6-14."""

    def forward(self, x):
        return silu_and_mul(x)


def rope_cos_sin_cache(head_dim, max_position, base, device):
    """RotaryEmbedding.cos_sin_cache (rotary_embedding.py:84-89, default rope type) as
    [max_position, head_dim] fp32."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_position, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(device)


def qk_norm_rope_store(qkv, positions, cos_sin, q_weight, k_weight, eps, num_heads, num_kv_heads,
                       head_dim, k_cache=None, v_cache=None, slot_mapping=None, query_cache=None,
                       query_slot_mapping=None, return_k=True, query_slot_count=None):
    """qkv [N, (Hq+2Hkv)*D] -> q [N,Hq,D] (normalised, rotated), k [N,Hkv,D] (or None), and, when
    given, K/V rows written to the paged caches at slot_mapping and window queries written to
    query_cache at the (row, query_id, index) triples — one launch.  `query_slot_count`: a device
    int32 tensor with the number of valid rows of `query_slot_mapping` (as `prepare_decode` returns
    it); without it every row is taken."""
    L.require_cuda(qkv, positions, cos_sin, q_weight, k_weight, k_cache, v_cache, slot_mapping,
                   query_cache, query_slot_mapping, query_slot_count)
    N = qkv.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    assert qkv.shape[1] == (Hq + 2 * Hkv) * D and qkv.stride(1) == 1
    assert positions.dtype == torch.int64 and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    q = torch.empty((N, Hq, D), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((N, Hkv, D), dtype=qkv.dtype, device=qkv.device) if return_k else None
    ntrip = 0 if query_slot_mapping is None else query_slot_mapping.shape[0]
    cs_seq = query_cache.stride(0) if query_cache is not None else 0
    cs_slot = query_cache.stride(1) if query_cache is not None else 0
    if k_cache is not None:
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
    L.check(L.load().zp_qk_norm_rope_store(
        L.ptr(qkv), L.ptr(positions), L.ptr(cos_sin), L.ptr(q_weight), L.ptr(k_weight), float(eps),
        L.ptr(q), L.ptr(k), L.ptr(k_cache), L.ptr(v_cache), L.ptr(slot_mapping), L.ptr(query_cache),
        L.ptr(query_slot_mapping), ntrip, L.ptr(query_slot_count), N, Hq, Hkv, D, qkv.stride(0), cs_seq, cs_slot,
        L.dtype_code(qkv), L.stream_ptr()), "qk_norm_rope_store")
    _count(1)
    v = qkv[:, (Hq + Hkv) * D:].view(N, Hkv, D)
    return q, k, v


def sample(logits, temperatures, noise=None, seed=0):
    """tokens [B] int64; `noise` = the Exp(1) draws ([B, V] fp32) or None for the built-in
    counter-based generator keyed by `seed`."""
    L.require_cuda(logits, temperatures, noise)
    B, V = logits.shape
    assert logits.is_contiguous() and temperatures.dtype == torch.float32
    if noise is not None:
        assert noise.dtype == torch.float32 and noise.is_contiguous() and noise.shape == logits.shape
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    L.check(L.load().zp_sample(L.ptr(logits), L.ptr(temperatures), L.ptr(noise), L.ptr(out), B, V,
                               int(seed), L.dtype_code(logits), L.stream_ptr()), "sample")
    _count(1)
    return out


class Sampler(nn.Module):
    """zipage/layers/sampler.py:6-48 without the repetition penalty (a transformers logits
    processor the reference applies before this op).  Each call advances the seed."""

    def __init__(self, seed: int = 0):
        super().__init__()
        self.seed = seed

    def forward(self, logits, temperatures, noise=None):
        self.seed += 1
        return sample(logits, temperatures, noise, self.seed)


def prepare_decode(num_tokens, block_tables, query_ids, query_cache_len, block_size=256):
    """Device tensors in, device tensors out: positions [B] i64, context_lens [B] i32,
    slot_mapping [B] i32, triples [B,3] i32 with n_triples [1] i32 valid rows."""
    L.require_cuda(num_tokens, block_tables, query_ids)
    B, W = block_tables.shape
    dev = block_tables.device
    pos = torch.empty(B, dtype=torch.int64, device=dev)
    ctx = torch.empty(B, dtype=torch.int32, device=dev)
    slot = torch.empty(B, dtype=torch.int32, device=dev)
    trip = torch.empty((B, 3), dtype=torch.int32, device=dev)
    ntrip = torch.empty(1, dtype=torch.int32, device=dev)
    assert num_tokens.dtype == torch.int32 and block_tables.dtype == torch.int32 and block_tables.is_contiguous()
    L.check(L.load().zp_prepare_decode(L.ptr(num_tokens), L.ptr(block_tables), L.ptr(query_ids), B, W,
                                       query_cache_len, block_size, L.ptr(pos), L.ptr(ctx), L.ptr(slot),
                                       L.ptr(trip), L.ptr(ntrip), L.stream_ptr()), "prepare_decode")
    _count(1)
    return pos, ctx, slot, trip, ntrip
