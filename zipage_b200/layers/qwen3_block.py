"""Qwen3 decoder blocks on libzipage_b200 kernels, one GPU per replica or tensor-parallel.

Same module tree and forward contracts as third_party/nanovllm/models/qwen3.py:14-170
(`Qwen3Attention`, `Qwen3MLP`, `Qwen3DecoderLayer`, `Qwen3Model`): the projections are plain
`nn.Linear` (cuBLAS), everything between them is one of this library's kernels.  In
`Qwen3Attention.forward` the q/k head normalisation, the rotation and the two cache writes
(qwen3.py:75-79 and zipage/layers/attention.py:72-77) are one launch, so `Attention.attend` is
called instead of `Attention.forward`.

With a `TPCommunicator` the heads and the MLP's intermediate columns are split across the ranks as
in third_party/nanovllm/layers/linear.py:54-153 (QKV / merged-column / row parallel).  The
row-parallel projections (o_proj, down_proj) return their partial sums; the all-reduce happens
inside the RMSNorm that consumes them (post_attention_layernorm, the next block's input_layernorm,
the final norm) as one fused launch over peer memory.  The embedding is replicated.
"""
from __future__ import annotations

import torch
from torch import nn

from ..utils.context import get_context
from .attention import Attention
from .step_ops import RMSNorm, SiluAndMul, qk_norm_rope_store, rope_cos_sin_cache


def reduce_add_norm(comm, norm, partial, residual):
    """RMSNorm(all_reduce(partial) + residual): one fused launch with a communicator."""
    if comm is None:
        return norm(partial, residual)
    return comm.all_reduce_add_rms_norm(partial, residual, norm.weight, norm.eps)


class Qwen3Attention(nn.Module):
    def __init__(self, hidden_size, num_heads, num_kv_heads, max_position=4096 * 32, head_dim=None,
                 rms_norm_eps=1e-06, qkv_bias=False, rope_theta=10000, comm=None):
        super().__init__()
        tp = comm.world if comm is not None else 1
        assert num_heads % tp == 0 and num_kv_heads % tp == 0
        self.head_dim = head_dim or hidden_size // num_heads
        self.total_num_heads, self.total_num_kv_heads = num_heads, num_kv_heads
        num_heads, num_kv_heads = num_heads // tp, num_kv_heads // tp   # this rank's heads
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.scaling = self.head_dim ** -0.5
        self.eps = rms_norm_eps
        self.qkv_proj = nn.Linear(hidden_size, (num_heads + 2 * num_kv_heads) * self.head_dim, bias=qkv_bias)
        self.o_proj = nn.Linear(num_heads * self.head_dim, hidden_size, bias=False)
        self.max_position, self.rope_theta = max_position, rope_theta
        self._cos_sin = None  # fp32 table, built on the first call's device (never cast with the module)
        self.attn = Attention(num_heads, self.head_dim, self.scaling, num_kv_heads)
        self.q_norm = RMSNorm(self.head_dim, eps=rms_norm_eps)
        self.k_norm = RMSNorm(self.head_dim, eps=rms_norm_eps)

    def forward(self, positions, hidden_states):
        qkv = self.qkv_proj(hidden_states)
        if self._cos_sin is None or self._cos_sin.device != qkv.device:
            self._cos_sin = rope_cos_sin_cache(self.head_dim, self.max_position, self.rope_theta, qkv.device)
        context = get_context()
        attn = self.attn
        have_kv = attn.k_cache.numel() > 0 and attn.v_cache.numel() > 0
        have_q = context.query_slot_mapping is not None and attn.q_cache.numel() > 0
        q, k, v = qk_norm_rope_store(
            qkv, positions, self._cos_sin, self.q_norm.weight, self.k_norm.weight, self.eps,
            self.num_heads, self.num_kv_heads, self.head_dim,
            k_cache=attn.k_cache if have_kv else None, v_cache=attn.v_cache if have_kv else None,
            slot_mapping=context.slot_mapping if have_kv else None,
            query_cache=attn.q_cache if have_q else None,
            query_slot_mapping=context.query_slot_mapping if have_q else None,
            return_k=context.is_prefill and context.block_tables is None,
            query_slot_count=context.query_slot_count if have_q else None)
        o = attn.attend(q, k, v)
        return self.o_proj(o.flatten(1, -1))


class Qwen3MLP(nn.Module):
    def __init__(self, hidden_size, intermediate_size, hidden_act="silu", comm=None):
        super().__init__()
        assert hidden_act == "silu"
        tp = comm.world if comm is not None else 1
        assert intermediate_size % tp == 0
        intermediate_size //= tp
        self.gate_up_proj = nn.Linear(hidden_size, 2 * intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self.act_fn = SiluAndMul()

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


class Qwen3DecoderLayer(nn.Module):
    """`config`: any object with the Qwen3Config fields read below."""

    def __init__(self, config, comm=None):
        super().__init__()
        self.comm = comm
        # The reference hands config.rope_scaling to its rope initialiser, which changes the
        # frequencies and the attention scaling (zipage/layers/rotary_embedding.py:67-83).  Only
        # the unscaled table is built here: a scaled configuration is refused rather than rotated
        # with the wrong table.
        rs = getattr(config, "rope_scaling", None)
        if rs and rs.get("rope_type", rs.get("type", "default")) != "default":
            raise NotImplementedError(f"rope_scaling {rs!r} is not supported (default rope only)")
        self.self_attn = Qwen3Attention(
            hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
            num_kv_heads=config.num_key_value_heads, max_position=config.max_position_embeddings,
            rms_norm_eps=config.rms_norm_eps, qkv_bias=getattr(config, "attention_bias", False),
            head_dim=getattr(config, "head_dim", None), rope_theta=getattr(config, "rope_theta", 1000000), comm=comm)
        self.mlp = Qwen3MLP(config.hidden_size, config.intermediate_size, config.hidden_act, comm=comm)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, positions, hidden_states, residual):
        """With a communicator, `hidden_states` (when a residual comes with it) and the return
        value are partial sums over the ranks; the norms reduce them."""
        if residual is None:
            hidden_states, residual = self.input_layernorm(hidden_states), hidden_states
        else:
            hidden_states, residual = reduce_add_norm(self.comm, self.input_layernorm, hidden_states, residual)
        hidden_states = self.self_attn(positions, hidden_states)
        hidden_states, residual = reduce_add_norm(self.comm, self.post_attention_layernorm, hidden_states, residual)
        hidden_states = self.mlp(hidden_states)
        return hidden_states, residual


class Qwen3Model(nn.Module):
    def __init__(self, config, comm=None):
        super().__init__()
        self.comm = comm
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([Qwen3DecoderLayer(config, comm) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids, positions):
        hidden_states = self.embed_tokens(input_ids)
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(positions, hidden_states, residual)
        hidden_states, _ = reduce_add_norm(self.comm, self.norm, hidden_states, residual)
        return hidden_states

    @torch.no_grad()
    def load_full_state(self, full_state, rank=0, world=1):
        """Copy this rank's shards out of an unsharded state dict (the slicing of
        third_party/nanovllm/layers/linear.py:85-153 weight loaders)."""
        for name, p in self.state_dict().items():
            w = full_state[name]
            if name.endswith("qkv_proj.weight") or name.endswith("qkv_proj.bias"):
                a = self.layers[0].self_attn
                D, Hq, Hkv = a.head_dim, a.total_num_heads, a.total_num_kv_heads
                q, k, v = w.split([Hq * D, Hkv * D, Hkv * D], dim=0)
                w = torch.cat([t.chunk(world, 0)[rank] for t in (q, k, v)], 0)
            elif name.endswith("gate_up_proj.weight"):
                w = torch.cat([t.chunk(world, 0)[rank] for t in w.chunk(2, 0)], 0)
            elif name.endswith("o_proj.weight") or name.endswith("down_proj.weight"):
                w = w.chunk(world, 1)[rank]
            p.copy_(w)

    def bind_caches(self, kv_cache, query_cache):
        """kv_cache [2, L, P, BS, Hkv, D], query_cache [L, C, QCL, Hq, D]: the per-layer views the
        reference assigns in ModelRunner.allocate_kv_cache (zipage/engine/model_runner.py:299-306)."""
        for i, layer in enumerate(self.layers):
            layer.self_attn.attn.k_cache = kv_cache[0, i]
            layer.self_attn.attn.v_cache = kv_cache[1, i]
            layer.self_attn.attn.q_cache = query_cache[i]
