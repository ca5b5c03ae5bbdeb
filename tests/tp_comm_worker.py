"""One rank of the two-GPU all-reduce test (run by test_gpu_tp_comm.py under torch.distributed.run).

Checks the peer-memory all-reduce bit for bit against the fp32 rank-order sum of the gathered
inputs, the fused residual + RMSNorm form against all-reduce followed by the RMSNorm kernel, and
the area hand-over between consecutive calls without any host synchronisation in between.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def expected(x, dtype):
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, x)
    acc = parts[0].float()
    for p in parts[1:]:
        acc = acc + p.float()
    return acc.to(dtype)


def tensor_parallel_decode_step(comm, dev, rank, world):
    """Decoder blocks split over the ranks (heads, MLP columns), the all-reduces fused into the
    norms: the hidden states agree with the unsharded model's on one GPU (bf16 tolerance: the
    partial sums are rounded per rank), are the same bits on every rank, and a CUDA-graph replay of
    the step equals the launch-by-launch step bit for bit, caches included."""
    from types import SimpleNamespace
    from zipage_b200.engine.decode_graph import DecodeGraphRunner
    from zipage_b200.layers.qwen3_block import Qwen3Model
    cfg = SimpleNamespace(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                          intermediate_size=2048, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=1000,
                          num_hidden_layers=3, max_position_embeddings=4096, rope_theta=1e6)
    QCL, BS, pages, B = 32, 256, 24, 6
    torch.manual_seed(5)                                    # replicated weights and state
    full = Qwen3Model(cfg)
    for p in full.parameters():
        if p.dim() == 1:
            p.data = 1.0 + 0.1 * torch.randn_like(p)
    full = full.to(torch.bfloat16).to(dev).eval()
    sharded = Qwen3Model(cfg, comm).to(torch.bfloat16).to(dev).eval()
    sharded.load_full_state(full.state_dict(), rank, world)
    Hq, Hkv, D, Ln = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_hidden_layers
    kv_full = (0.5 * torch.randn(2, Ln, pages, BS, Hkv, D)).to(torch.bfloat16).to(dev)
    qc_full = torch.zeros(Ln, 8, QCL, Hq, D, dtype=torch.bfloat16, device=dev)
    hk, hq = Hkv // world, Hq // world
    kv = kv_full[:, :, :, :, rank * hk:(rank + 1) * hk].contiguous()
    qc = qc_full[:, :, :, rank * hq:(rank + 1) * hq].contiguous()
    full.bind_caches(kv_full, qc_full)
    sharded.bind_caches(kv, qc)
    snap = (kv.clone(), qc.clone())
    tables = torch.tensor([[3, 7, -1], [1, 9, 11], [0, 2, -1], [4, -1, -1], [5, 6, 8], [10, 12, -1]],
                          dtype=torch.int32, device=dev)
    ntok = torch.tensor([256 + 230, 512 + 255, 256 + 17, 250, 512 + 256, 256 + 225], dtype=torch.int32, device=dev)
    qids = torch.tensor([0, 1, -1, 2, 3, 4], dtype=torch.int32, device=dev)
    ids = torch.randint(0, cfg.vocab_size, (B,)).to(dev)
    one = DecodeGraphRunner(full, cfg.hidden_size, max_bs=8, max_num_blocks=4, query_cache_len=QCL, device=dev)
    want = one.run(ids, ntok, tables, qids, eager=True).clone()
    tp = DecodeGraphRunner(sharded, cfg.hidden_size, max_bs=8, max_num_blocks=4, query_cache_len=QCL, device=dev,
                           graph_bs=[8])
    got = tp.run(ids, ntok, tables, qids, eager=True).clone()
    ekv, eqc = kv.clone(), qc.clone()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 0.03 * want.float().abs().max().item(), err
    # this rank's heads of the rows the unsharded model wrote (first block: same inputs; the
    # projection runs as a GEMM of another shape, so the last bit may differ)
    d = (ekv[:, 0].float() - kv_full[:, 0, :, :, rank * hk:(rank + 1) * hk].float()).abs().max().item()
    assert d < 0.05, d
    assert not torch.equal(ekv, snap[0])
    same = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(same, got)
    assert all(torch.equal(t, got) for t in same)
    kv.copy_(snap[0]); qc.copy_(snap[1])
    tp.capture()
    assert torch.equal(kv, snap[0]) and torch.equal(qc, snap[1])
    rep = tp.run(ids, ntok, tables, qids).clone()
    assert torch.equal(rep, got) and torch.equal(kv, ekv) and torch.equal(qc, eqc)
    step = torch.tensor([1, 1, 1, 1, 0, 1], dtype=torch.int32, device=dev)
    rep2 = tp.run(ids, ntok + step, tables, qids).clone()  # a second replay, other state
    assert torch.isfinite(rep2.float()).all() and not torch.equal(rep2, rep)
    torch.cuda.synchronize()


def main():
    from zipage_b200.layers.step_ops import rms_norm
    from zipage_b200.layers.tp_comm import TPCommunicator
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    comm = TPCommunicator(max_bytes=8 << 20, timeout_ms=5000)
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        per = 16 // torch.empty((), dtype=dtype).element_size()
        for n in (per, 4096, 1000 * per + 3 * per, 256 * 4096, 2 * 1024 * 1024):
            for algo in ("one_shot", "two_shot", "auto", "flagged_lines"):
                if algo == "flagged_lines" and n * (16 // per) > (2 << 20):
                    continue                                  # that form carries at most 2 MiB
                x = torch.randn(n, device=dev, generator=g).to(dtype)
                want = expected(x, dtype)
                got = comm.all_reduce(x.clone(), algo=algo)
                assert torch.equal(got, want), (dtype, n, algo)
                out = torch.empty_like(x)
                assert comm.all_reduce(x, out=out, algo=algo) is out and torch.equal(out, want)

    # consecutive calls with nothing between them: each call's areas must survive until every
    # peer has read them, and sizes (hence grids) change from call to call
    sizes = [4096, 1 << 20, 8, 65536, 1 << 21, 512, 4096, 1 << 19] * 3
    xs = [torch.randn(n, device=dev, generator=g).to(torch.bfloat16) for n in sizes]
    wants = [expected(x, torch.bfloat16) for x in xs]
    torch.cuda.synchronize()
    dist.barrier()
    for algo in ("one_shot", "two_shot", "auto"):   # auto: flagged lines up to 2 MiB, meetings above
        outs = [comm.all_reduce(x, out=torch.empty_like(x), algo=algo) for x in xs]
        torch.cuda.synchronize()
        for o, w in zip(outs, wants):
            assert torch.equal(o, w), algo

    # fused residual add + RMSNorm
    for dtype in (torch.bfloat16, torch.float32):
        for rows, hidden in ((256, 4096), (3, 1024), (300, 2048)):
            x = torch.randn(rows, hidden, device=dev, generator=g).to(dtype)
            torch.manual_seed(7)   # residual and weight are replicated across the ranks
            res = torch.randn(rows, hidden).to(dtype).to(dev)
            w = (1 + 0.1 * torch.randn(hidden)).to(dtype).to(dev)
            for algo in ("one_shot", "two_shot", "flagged_lines"):
                if algo == "flagged_lines" and x.numel() * x.element_size() > (2 << 20):
                    continue
                y0, r0 = rms_norm(comm.all_reduce(x.clone(), algo=algo), w, 1e-6, res)
                y1, r1 = comm.all_reduce_add_rms_norm(x, res, w, 1e-6, algo=algo)
                assert torch.equal(r0, r1), (dtype, rows, hidden, algo)
                # the sum of squares is reduced over 512 threads here, 256 there: the scale can differ
                # in its last bit — a few ulps in fp32, one rounding step of T in a few bf16 elements
                if dtype == torch.float32:
                    assert torch.allclose(y0, y1, rtol=3e-6, atol=1e-6), (rows, hidden, algo)
                else:
                    d = (y0.float() - y1.float()).abs()
                    assert (d <= 2.0 ** -7 * y0.float().abs().clamp_min(1e-3)).all(), (rows, hidden, algo)
                    assert (d > 0).float().mean() < 0.01, (rows, hidden, algo, (d > 0).float().mean())

    # sampling over a sharded vocabulary == the single-GPU sampler on the concatenated logits
    # (and the CPU oracle), with given draws and with the built-in generator
    from oracle import step_ops_oracle as S
    from zipage_b200.layers.step_ops import sample
    for dtype, B, Vs in ((torch.bfloat16, 37, 5000), (torch.bfloat16, 300, 1001), (torch.bfloat16, 700, 520), (torch.float32, 64, 4096),
                         (torch.float16, 5, 75968)):
        torch.manual_seed(3)                                  # replicated inputs
        V = Vs * world
        full = (3 * torch.randn(B, V)).to(dtype).to(dev)
        temps = (0.3 + torch.rand(B)).to(dev)
        draws = torch.empty(B, V).exponential_(1.0).to(dev)
        full[3, 5] = full[3, Vs + 9] = 40.0               # an exact tie between two shards:
        draws[3, 5] = draws[3, Vs + 9] = 0.5              # the lower global index must win
        sl = slice(rank * Vs, (rank + 1) * Vs)
        tok = comm.sample(full[:, sl].contiguous(), temps, noise_shard=draws[:, sl].contiguous())
        assert torch.equal(tok, sample(full, temps, noise=draws)), (dtype, B, Vs)
        assert int(tok[3]) == 5
        assert torch.equal(tok.cpu(), S.sample_race(full.cpu(), temps.cpu(), draws.cpu())), (dtype, B, Vs)
        tok = comm.sample(full[:, sl].contiguous(), temps, seed=11)
        assert torch.equal(tok, sample(full, temps, seed=11)), (dtype, B, Vs, "generator")
        gathered = [torch.empty_like(tok) for _ in range(world)]
        dist.all_gather(gathered, tok)
        assert all(torch.equal(t, tok) for t in gathered)

    tensor_parallel_decode_step(comm, dev, rank, world)

    # timing of the 4 MiB message of a 512-sequence decode step against the library collective
    x = torch.randn(2 * 1024 * 1024, device=dev, generator=g).to(torch.bfloat16)
    y = x.clone()

    def timed(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    t1 = timed(lambda: comm.all_reduce(x, out=y, algo="one_shot"))
    t2 = timed(lambda: comm.all_reduce(x, out=y, algo="two_shot"))
    t3 = timed(lambda: dist.all_reduce(y))
    small = torch.randn(8 * 4096, device=dev, generator=g).to(torch.bfloat16)
    s1 = timed(lambda: comm.all_reduce(small, algo="one_shot"))
    s2 = timed(lambda: comm.all_reduce(small, algo="flagged_lines"))
    s3 = timed(lambda: dist.all_reduce(small))
    # the reference's route for 512 rows of a 151 936-token vocabulary: gather the shards to rank 0,
    # concatenate, sample there
    Vs = 151936 // world
    shard = torch.randn(512, Vs, device=dev, generator=g).to(torch.bfloat16)
    temps = torch.full((512,), 0.7, device=dev)
    parts = [torch.empty_like(shard) for _ in range(world)] if rank == 0 else None

    def gather_route():
        dist.gather(shard, parts, 0)
        if rank == 0:
            sample(torch.cat(parts, -1), temps, seed=5)

    g1 = timed(lambda: comm.sample(shard, temps, seed=5), 20)
    g2 = timed(gather_route, 20)
    if rank == 0:
        print(f"TPCOMM world={world} sampler 512 x 151936: sharded {g1:.1f} us, gather + sample on rank 0 {g2:.1f} us", flush=True)
    assert comm.status() == 0
    if rank == 0:
        print(f"TPCOMM world={world} 4MiB: one_shot {t1:.1f} us, two_shot {t2:.1f} us, nccl {t3:.1f} us; "
              f"64KiB: one_shot {s1:.1f} us, flagged lines {s2:.1f} us, nccl {s3:.1f} us", flush=True)
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
