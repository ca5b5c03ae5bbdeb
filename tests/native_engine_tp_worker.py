"""Rank program of the tensor-parallel serving-loop test (launched by torch.distributed.run from
tests/test_gpu_native_engine.py).  Every rank first runs the single-GPU loop on its own GPU
(greedy, recording arg-max, margin and spread per step), then the ranks run the tensor-parallel
loop together — heads, MLP columns and K/V heads split, one scheduler replica per rank, all-reduces
over peer memory (prefill batches through the library route) — fed the single-GPU tokens.  Checks:
the tensor-parallel arg-max equals the single-GPU token wherever the single-GPU margin is above
2e-2 of the logit spread; the ranks' arg-max records are identical; no communicator wait ran out.
"""
import json
import os
import sys
import types
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main():
    import test_gpu_native_engine as T
    from safetensors.torch import load_file
    from zipage_b200.compress import CompressConfig
    from zipage_b200.engine.native_engine import NativeEngine, full_state_from_hf
    from zipage_b200.layers.qwen3_block import Qwen3Model
    from zipage_b200.layers.tp_comm import TPCommunicator
    local = int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    if rank == 0:
        T._ensure_model()
    dist.barrier()
    S = T.SHAPE
    prompts = T._prompts(n=3, length=650)

    # 1. the single-GPU loop on this rank's own GPU
    single = T._engine(graph=True)
    single.argmax_log = []
    seqs = T._requests(prompts)
    out = single.generate(seqs)
    want, log1 = [out[s._h] for s in seqs], single.argmax_log
    del single
    torch.cuda.empty_cache()

    # 2. the tensor-parallel loop, fed those tokens
    comm = TPCommunicator(max_bytes=16 * S["hidden"] * 2, timeout_ms=2000, large_messages="library")
    hf = {}
    for f in sorted(T.MODEL_DIR.glob("*.safetensors")):
        hf.update(load_file(str(f)))
    full, lm_head = full_state_from_hf(hf)
    cfg = types.SimpleNamespace(hidden_size=S["hidden"], num_attention_heads=S["hq"], num_key_value_heads=S["hkv"],
                                head_dim=128, intermediate_size=S["inter"], hidden_act="silu", rms_norm_eps=1e-6,
                                vocab_size=S["vocab"], num_hidden_layers=S["layers"], max_position_embeddings=40960,
                                rope_theta=1e6)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen3Model(cfg, comm).eval()
    finally:
        torch.set_default_dtype(prev)
    model.load_full_state({k: v.to(dev) for k, v in full.items()}, rank, world)
    blocks, slots = 64, 8
    kv = torch.zeros((2, S["layers"], blocks, 256, S["hkv"] // world, 128), dtype=torch.bfloat16, device=dev)
    qc = torch.zeros((S["layers"], slots, 16, S["hq"] // world, 128), dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    sched_cfg = types.SimpleNamespace(max_num_seqs=16, max_num_batched_tokens=32768, eos=1, num_kvcache_blocks=blocks,
                                      kvcache_block_size=256, max_cache_blocks_per_seq=2, enable_prefix_cache=False,
                                      max_concurrency=slots, enable_hybrid_engine=False, query_cache_len=16)
    ccfg = CompressConfig(budget_blocks=2, query_cache_len=16, use_redudancy=True, lightning_redudancy=True,
                          redudancy_lambda=0.5, enable_pooling=True)
    # the full LM head on every rank: the test reads whole logit rows (the loop itself samples
    # over the sharded vocabulary, which has its own tests)
    eng = NativeEngine(model, lm_head.to(dev), kv, qc, sched_cfg, ccfg, S["hidden"], comm=comm, max_bs=16,
                       max_model_len=8192, greedy=True, graph=True)
    eng.forced = iter([s["tokens"] for s in log1])
    eng.argmax_log = []
    seqs2 = T._requests(prompts)
    got = eng.generate(seqs2)
    fed = [got[s._h] for s in seqs2] == want
    total = mism = unexplained = 0
    for a, b in zip(log1, eng.argmax_log):
        for ta, tb, m, sp in zip(a["tokens"], b["tokens"], a["margin"], a["spread"]):
            total += 1
            if ta != tb:
                mism += 1
                unexplained += m > 2e-2 * sp
    mine = json.dumps([s["tokens"] for s in eng.argmax_log])
    every = [None] * world
    dist.all_gather_object(every, mine)
    same = all(e == mine for e in every)
    status = comm.status()
    ok = fed and unexplained == 0 and mism <= 0.05 * total and same and status == 0 \
        and eng.time_record["compress_reqs"] == 3
    if rank == 0:
        print(f"tensor-parallel x{world}: {total} tokens, arg-max differs from the single-GPU loop on {mism}, "
              f"{unexplained} above the margin; ranks identical: {same}; comm status {status}")
        print("TP_ENGINE_OK" if ok else "TP_ENGINE_FAILED")
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
