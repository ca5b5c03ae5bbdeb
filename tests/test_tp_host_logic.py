"""The tensor-parallel rows on CPU: the sharded sampler's algorithm over two gloo ranks against the
full-vocabulary oracle, the pinned all-reduce order, and the weight sharding of the blocks."""
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _sampler_rank(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import step_ops_oracle as S
    torch.manual_seed(4)                                   # replicated inputs
    B, Vs = 40, 777
    full = 3 * torch.randn(B, Vs * world)
    full[3, 5] = full[3, Vs + 9] = 40.0                    # equal logits in two shards
    temps = 0.3 + torch.rand(B)
    draws = torch.empty(B, Vs * world).exponential_(1.0)
    draws[3, 5] = draws[3, Vs + 9] = 0.5                   # ... and equal draws: an exact tie
    sl = slice(rank * Vs, (rank + 1) * Vs)
    m, z = S.shard_softmax_stats(full[:, sl], temps)
    ms, zs = [torch.empty_like(m) for _ in range(world)], [torch.empty_like(z) for _ in range(world)]
    dist.all_gather(ms, m); dist.all_gather(zs, z)         # 8 bytes per row and rank
    val, idx = S.shard_race_winner(full[:, sl], temps, draws[:, sl], torch.stack(ms), torch.stack(zs), rank * Vs)
    vals, idxs = [torch.empty_like(val) for _ in range(world)], [torch.empty_like(idx) for _ in range(world)]
    dist.all_gather(vals, val); dist.all_gather(idxs, idx)  # 8 more
    tok = S.combine_winners(torch.stack(vals), torch.stack(idxs))
    want = S.sample_race(full, temps, draws)
    ok = torch.equal(tok, want) and int(tok[3]) == 5
    # all-reduce with the pinned order: every rank computes the same bits from the gathered parts
    x = torch.randn(1000, generator=torch.Generator().manual_seed(rank)).to(torch.bfloat16)
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    mine = S.all_reduce_rank_order(parts, torch.bfloat16)
    theirs = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(theirs, mine)
    ok = ok and all(torch.equal(t, mine) for t in theirs)
    if rank == 0:
        Path(tmp).write_text("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_sampler_two_ranks_gloo(tmp_path):
    port = 31500 + os.getpid() % 2000
    res = tmp_path / "result.txt"
    mp.spawn(_sampler_rank, args=(2, port, str(res)), nprocs=2, join=True)
    assert res.read_text() == "ok"


def test_block_weight_sharding_recombines():
    """Column shards of qkv / gate_up concatenate back to the full projections (per head group and
    per gate/up half), row shards of o_proj / down_proj sum back to the full product."""
    from zipage_b200.layers.qwen3_block import Qwen3Model
    cfg = SimpleNamespace(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                          intermediate_size=96, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=50,
                          num_hidden_layers=2, max_position_embeddings=128, rope_theta=1e4, attention_bias=True)
    torch.manual_seed(0)
    full = Qwen3Model(cfg)
    world = 2
    shards = []
    for rank in range(world):
        m = Qwen3Model(cfg, SimpleNamespace(world=world, rank=rank))
        m.load_full_state(full.state_dict(), rank, world)
        shards.append(m)
    x = torch.randn(5, 64)
    a_full, a = full.layers[1].self_attn, [s.layers[1].self_attn for s in shards]
    D, Hq, Hkv = 16, 4, 2
    qkv = a_full.qkv_proj(x)
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], -1)
    parts = [s.qkv_proj(x).split([Hq // world * D, Hkv // world * D, Hkv // world * D], -1) for s in a]
    for full_t, i in ((q, 0), (k, 1), (v, 2)):
        assert torch.allclose(torch.cat([p[i] for p in parts], -1), full_t, atol=1e-6)
    o_in = torch.randn(5, Hq * D)
    got = sum(s.o_proj(o_in.chunk(world, -1)[r]) for r, s in enumerate(a))
    assert torch.allclose(got, a_full.o_proj(o_in), atol=1e-5)
    m_full, m = full.layers[0].mlp, [s.layers[0].mlp for s in shards]
    g_full, u_full = m_full.gate_up_proj(x).chunk(2, -1)
    gs = [s.gate_up_proj(x).chunk(2, -1) for s in m]
    assert torch.allclose(torch.cat([g[0] for g in gs], -1), g_full, atol=1e-6)
    assert torch.allclose(torch.cat([g[1] for g in gs], -1), u_full, atol=1e-6)
    h = torch.randn(5, 96)
    got = sum(s.down_proj(h.chunk(world, -1)[r]) for r, s in enumerate(m))
    assert torch.allclose(got, m_full.down_proj(h), atol=1e-5)
    # replicated parts
    assert torch.equal(shards[1].embed_tokens.weight, full.embed_tokens.weight)
    assert torch.equal(shards[1].layers[0].input_layernorm.weight, full.layers[0].input_layernorm.weight)
