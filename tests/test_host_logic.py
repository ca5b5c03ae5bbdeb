"""Host-side logic on CPU: table encoding, synthetic workloads, the benchmark's reference arm,
and KV-head sharding over two gloo ranks (per-rank results equal the full result restricted to
the rank's heads, with no exchange)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
BS = 256


def test_encode_block_tables():
    from zipage_b200.engine.compressor import encode_block_tables
    assert encode_block_tables([[5, 2, 9], [7, 3]]) == [[5, 2, -11], [7, -5, -1]]
    assert encode_block_tables([[0]]) == [[-2]]


def test_synthetic_workload_invariants():
    from zipage_b200.synthetic import algorithmic_bytes_per_unit, make_compress_workload
    w = make_compress_workload(B=6, L=2, Hkv=2, Hq=4, QCL=16, budget=2, pages_per_seq=[3, 3, 4, 5, 3, 3],
                               dtype=torch.float32, device="cpu", seed=3, with_score_cache=True,
                               compressed_prob=0.5, fresh_target_prob=1.0)
    plain = w.tables_plain
    used = plain[plain >= 0]
    assert used.unique().numel() == used.numel()            # no page shared between sequences
    for b in range(6):
        row = plain[b][plain[b] >= 0]
        n = row.numel()
        enc = w.block_tables[b]
        assert enc[n - 1] == -row[-1] - 2 and (enc[n:] == -1).all()
        tgt = w.target_tables[b]
        # a target page is either fresh or the source page at the same table position
        for i, pg in enumerate(tgt.tolist()):
            assert pg == int(row[i]) or pg not in used.tolist()
        if n > 3:
            assert not bool(w.compressed[b])
    st = algorithmic_bytes_per_unit(9, 128, 32, 4, 2, True, False, 2000)
    assert st["window_score"] == 589824 + 32768 + 4608 and st["compact"] == 2000 * 256 * 4 + 2304


def test_bench_reference_arm_prints_contract_line():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(ROOT))
    from oracle import zipage_oracle as O
    from zipage_b200.synthetic import make_compress_workload, shard_kv_heads
    torch.set_num_threads(2)
    w = make_compress_workload(B=3, L=2, Hkv=4, Hq=8, QCL=16, budget=2, pages_per_seq=[3, 4, 3],
                               dtype=torch.float32, device="cpu", seed=9, with_score_cache=True,
                               compressed_prob=0.5, similar_keys=True)
    cfg = O.CompressConfig(budget_blocks=2, query_cache_len=16, use_global_score=True,
                           use_redudancy=True, lightning_redudancy=True, enable_pooling=True)
    mine = shard_kv_heads(w, rank, world)
    _, keep = O.compress(mine.kv_cache[0], mine.kv_cache[1], mine.query_cache, mine.score_cache,
                         mine.query_ids, mine.block_tables, mine.target_tables, mine.compressed, cfg)
    gathered = [torch.empty_like(keep) for _ in range(world)]
    dist.all_gather(gathered, keep)          # test-only exchange: the op itself needs none
    kcat = [torch.empty_like(mine.kv_cache) for _ in range(world)]
    dist.all_gather(kcat, mine.kv_cache)
    if rank == 0:
        _, full = O.compress(w.kv_cache[0], w.kv_cache[1], w.query_cache, w.score_cache, w.query_ids,
                             w.block_tables, w.target_tables, w.compressed, cfg)
        ok = torch.equal(torch.cat(gathered, dim=2), full)
        ok = ok and torch.equal(torch.cat(kcat, dim=4), w.kv_cache)
        Path(tmp).write_text("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


def test_kv_head_sharding_two_ranks_gloo(tmp_path):
    port = 29500 + os.getpid() % 2000
    res = tmp_path / "result.txt"
    mp.spawn(_rank_main, args=(2, port, str(res)), nprocs=2, join=True)
    assert res.read_text() == "ok"
