"""The serving loop built from this library only (zipage_b200/engine/native_engine.py: native
scheduler, varlen prefill through the decoder blocks, graph-replayed decode, Compressor, LM head)
against the unmodified reference ENGINE on the same seeded model and prompts.

As in test_gpu_reference_engine.py the comparison is teacher-forced: the native loop is fed the
reference run's tokens while its own arg-max, top-2 margin and logit spread are recorded at every
step; the own arg-max must equal the reference's token wherever the reference's margin exceeds
2e-2 of the logit spread (the bf16 tolerance of the path).  That the loop takes the same steps as
the reference engine (one prefill batch, then every decode step with all requests, compressions
at the same steps) follows from the scheduler's state parity (tests/test_host_scheduler.py) and
shows here in the step counts.  A second, free-running pass checks that graph replay and
launch-by-launch decode give the same tokens.
"""
import json
import subprocess
import sys
import types
from pathlib import Path

import pytest
import torch

import ref_binding as RB

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
STEPS = 256
SHAPE = dict(layers=4, hidden=1024, inter=2048, hq=8, hkv=2, vocab=2048, seed=0)
MODEL_DIR = Path("/tmp/zp_synth_model")      # the directory tests/ref_engine.py writes by default


def _engine(graph, greedy=True, max_bs=16, prefix_cache=False):
    from safetensors.torch import load_file
    from zipage_b200.compress import CompressConfig
    from zipage_b200.engine.native_engine import NativeEngine, full_state_from_hf
    from zipage_b200.layers.qwen3_block import Qwen3Model
    dev = torch.device("cuda")
    hf = {}
    for f in sorted(MODEL_DIR.glob("*.safetensors")):
        hf.update(load_file(str(f)))
    full, lm_head = full_state_from_hf(hf)
    cfg = types.SimpleNamespace(hidden_size=SHAPE["hidden"], num_attention_heads=SHAPE["hq"],
                                num_key_value_heads=SHAPE["hkv"], head_dim=128, intermediate_size=SHAPE["inter"],
                                hidden_act="silu", rms_norm_eps=1e-6, vocab_size=SHAPE["vocab"],
                                num_hidden_layers=SHAPE["layers"], max_position_embeddings=40960, rope_theta=1e6)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen3Model(cfg).eval()
    finally:
        torch.set_default_dtype(prev)
    model.load_full_state({k: v.to(dev) for k, v in full.items()})
    blocks, slots = 64, 8
    kv = torch.zeros((2, SHAPE["layers"], blocks, 256, SHAPE["hkv"], 128), dtype=torch.bfloat16, device=dev)
    qc = torch.zeros((SHAPE["layers"], slots, 16, SHAPE["hq"], 128), dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    sched_cfg = types.SimpleNamespace(max_num_seqs=16, max_num_batched_tokens=32768, eos=1, num_kvcache_blocks=blocks,
                                      kvcache_block_size=256, max_cache_blocks_per_seq=2, enable_prefix_cache=prefix_cache,
                                      max_concurrency=slots, enable_hybrid_engine=False, query_cache_len=16)
    ccfg = CompressConfig(budget_blocks=2, query_cache_len=16, use_redudancy=True, lightning_redudancy=True,
                          redudancy_lambda=0.5, enable_pooling=True)
    return NativeEngine(model, lm_head.to(dev), kv, qc, sched_cfg, ccfg, SHAPE["hidden"], max_bs=max_bs,
                        max_model_len=8192, greedy=greedy, graph=graph)


def _prompts(n=4, length=600):
    g = torch.Generator().manual_seed(SHAPE["seed"] + 1)       # as tests/ref_engine.py draws them
    return [torch.randint(2, SHAPE["vocab"], (length,), generator=g).tolist() for _ in range(n)]


def _requests(prompts):
    from zipage_b200.engine.scheduler import SamplingParams, Sequence
    return [Sequence(p, SamplingParams(0.6, STEPS, True)) for p in prompts]


def test_native_engine_against_the_reference_engine(tmp_path):
    ok, why = RB.reference_available()
    if not ok:
        pytest.skip(why)
    out = tmp_path / "ref.json"
    cmd = [sys.executable, str(ROOT / "tests" / "ref_engine.py"), "--mode", "reference", "--out", str(out),
           "--greedy", "--lightning", "--pooling", "--requests", "4", "--prompt-len", "600",
           "--max-tokens", str(STEPS), "--budget", "2", "--qcl", "16"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if r.returncode != 0:
        pytest.skip("the reference engine does not start on this machine: " + (r.stdout + r.stderr)[-600:])
    ref = json.loads(out.read_text())
    assert all(len(t) == STEPS for t in ref["tokens"])

    # the reference's sampler is also called once while the engine warms up, before any request
    ref_steps = ref["steps"][-STEPS:]
    assert len(ref["steps"]) in (STEPS, STEPS + 1)
    eng = _engine(graph=True)
    eng.forced = iter([s["tokens"] for s in ref_steps])
    eng.argmax_log = []
    seqs = _requests(_prompts())
    got = eng.generate(seqs)
    assert [got[s._h] for s in seqs] == ref["tokens"]               # the forced tokens, all 256 of each
    assert len(eng.argmax_log) == STEPS                              # one prefill + 255 decode steps
    assert eng.time_record["compress_reqs"] == 4                     # every request crossed 769 tokens once
    total = mism = unexplained = near = 0
    for a, b in zip(ref_steps, eng.argmax_log):
        for ta, tb, m, s in zip(a["tokens"], b["tokens"], a["margin"], a["spread"]):
            total += 1
            near += m <= 2e-2 * s
            if ta != tb:
                mism += 1
                unexplained += m > 2e-2 * s
    print(f"native engine: {total} sampled tokens, own arg-max differs on {mism}, {unexplained} of them at a "
          f"margin above 2e-2 of the logit spread ({near} steps are below it)")
    assert unexplained == 0 and mism <= 0.05 * total
    c = eng.scheduler.counts()
    assert c[7] == 1 and c[3] == 0                                   # finished, every block returned


def _ensure_model():
    tag = "-".join(str(SHAPE[k]) for k in ("layers", "hidden", "inter", "hq", "hkv", "vocab", "seed"))
    if not (MODEL_DIR / "tag").exists() or (MODEL_DIR / "tag").read_text() != tag:
        sys.path.insert(0, str(ROOT / "tests"))
        import ref_engine
        ref_engine.make_model_dir(MODEL_DIR, **SHAPE)
        (MODEL_DIR / "tag").write_text(tag)


def test_graph_replay_and_launch_by_launch_give_the_same_tokens():
    _ensure_model()
    runs = []
    for graph in (True, False):
        eng = _engine(graph=graph)
        seqs = _requests(_prompts(n=3, length=700))
        got = eng.generate(seqs)
        runs.append([got[s._h] for s in seqs])
        assert eng.time_record["compress_reqs"] == 3 and all(len(t) == STEPS for t in runs[-1])
    assert runs[0] == runs[1]


def test_prefix_cache_reuses_pages_and_gives_the_same_tokens():
    """Requests that share a 512-token prefix: with the prefix cache the later ones start from
    the first one's pages (prefill over the paged keys, zipage/layers/attention.py:82-93 with
    block_table), without it every prompt is recomputed.  The cached run is fed the plain run's
    tokens; its own arg-max must agree wherever the plain run's top-2 margin is above tolerance."""
    _ensure_model()
    g = torch.Generator().manual_seed(7)
    shared = torch.randint(2, SHAPE["vocab"], (512,), generator=g).tolist()
    prompts = [shared + torch.randint(2, SHAPE["vocab"], (n,), generator=g).tolist() for n in (90, 140, 200)]
    plain = _engine(graph=True)
    plain.argmax_log = []
    seqs = _requests(prompts)
    out = plain.generate(seqs)
    want = [out[s._h] for s in seqs]

    cached = _engine(graph=True, prefix_cache=True)
    reused = []
    real_prefill = cached._prefill

    def spy(handles):
        reused.extend(int(cached.scheduler._seqs[h].num_cached_tokens) for h in handles.tolist())
        return real_prefill(handles)
    cached._prefill = spy
    cached.forced = iter([s["tokens"] for s in plain.argmax_log])
    cached.argmax_log = []
    seqs2 = _requests(prompts)
    got = cached.generate(seqs2)
    have = [got[s._h] for s in seqs2]
    first = [next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), None) for x, y in zip(have, want)]
    sizes = ([len(s["tokens"]) for s in plain.argmax_log], [len(s["tokens"]) for s in cached.argmax_log])
    assert have == want, (first, [len(x) for x in have], sizes[0][:4], sizes[1][:4], len(sizes[0]), len(sizes[1]))
    assert sorted(reused) == [0, 512, 512]            # two of the three started from the shared pages
    mism = unexplained = 0
    for a, b in zip(plain.argmax_log, cached.argmax_log):
        for ta, tb, m, sp in zip(a["tokens"], b["tokens"], a["margin"], a["spread"]):
            if ta != tb:
                mism += 1
                unexplained += m > 2e-2 * sp
    print(f"prefix cache: own arg-max differs on {mism} of {3 * STEPS} tokens, {unexplained} above the margin")
    assert unexplained == 0 and mism <= 0.05 * 3 * STEPS


def test_tensor_parallel_loop_against_the_single_gpu_loop(world=2):
    """tests/native_engine_tp_worker.py under torch.distributed.run: one scheduler replica per rank,
    all-reduces over peer memory, prefill batches through the library route."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(29700 + world),
         str(ROOT / "tests" / "native_engine_tp_worker.py")], capture_output=True, text=True, timeout=900)
    print(r.stdout[-600:])
    assert r.returncode == 0 and "TP_ENGINE_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
