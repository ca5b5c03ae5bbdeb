#!/usr/bin/env python
"""Benchmark of the compression op (the configuration the "compress HBM GB/s" metric is quoted on).

    python bench.py --gpus N --steps K --warmup W            # this repository's CUDA path
    python bench.py --impl reference ...                     # the reference's CPU formulation
    torchrun --nproc-per-node N bench.py --gpus N ...        # one rank per GPU, KV heads sharded

One step = one pass of the whole compression op (window scoring -> [global score] -> similarity
redundancy -> pooling/combine/masks/top-k -> in-place compaction) over every layer of a batch of
sequences that each hold budget+1 = 9 pages.  `value` is algorithmic bytes moved per second with
all inputs resident in HBM; `e2e` is the same through the host-facing call (host lists of block
tables -> pinned memory -> device, kernels, stream sync, read-back of the new tables).
Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "compress_hbm_gbs"
UNIT = "GB/s"
BS = 256


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="zipage_b200", choices=["zipage_b200", "reference"])
    ap.add_argument("--variant", default="lightning", choices=["lightning", "exact", "none"])
    ap.add_argument("--batch", type=int, default=512, help="sequences per GPU at N=1 (reduced to fit)")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--layer-chunk", type=int, default=0, help="layers per kernel call (0 = all)")
    ap.add_argument("--global-score", action="store_true")
    ap.add_argument("--kernel-impl", default="auto", choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-step record of the default run")
    ap.add_argument("--no-serving-loop", action="store_true", help="skip the serving-loop record of the default run")
    ap.add_argument("--engine", action="store_true",
                    help="also run the reference ENGINE (baseline/_ref) on a synthetic Qwen3-8B-shaped model, as it "
                         "is and with this library's decode path bound, and report decode tokens/s (adds minutes)")
    ap.add_argument("--also-exact", action="store_true", help="time the exact variant as well")
    ap.add_argument("--workload", default="compress", choices=["compress", "decode", "step_ops", "prefill", "decode_step", "tp_allreduce", "engine_decode", "long_prompt", "host_control", "native_engine"],
                    help="compress (default, the headline op), decode (paged decode attention kernel) or "
                         "step_ops (the element-wise ops of a decoder layer step and the sampler) or "
                         "prefill (varlen causal prefill attention, one layer) or decode_step (the decode "
                         "forward of Qwen3-8B-shaped blocks, launch by launch and as a replayed CUDA graph) or "
                         "tp_allreduce (the row-parallel projections' all-reduce + residual + RMSNorm over "
                         "peer memory against the library collective; needs --gpus >= 2 under torchrun)")
    ap.add_argument("--verbose", action="store_true", help="progress lines on stderr")
    ap.add_argument("--engine-modes", default="reference,kernels,graph",
                    help="modes of the engine_decode workload (tests/ref_engine.py): reference, kernels, full, graph, native")
    ap.add_argument("--engine-requests", type=int, default=192, help="concurrent requests of the native_engine workload")
    ap.add_argument("--engine-prompt", type=int, default=2300, help="prompt tokens per request (native_engine)")
    ap.add_argument("--engine-gen", type=int, default=600, help="generated tokens per request (native_engine)")
    ap.add_argument("--engine-prefix-cache", action="store_true", help="prefix cache on (native_engine)")
    ap.add_argument("--requests", type=int, default=2048, help="concurrent requests of the host_control workload")
    ap.add_argument("--tokens", type=int, default=32768, help="tokens per call of the step_ops workload")
    return ap.parse_args()


# workload constants: Qwen3-8B attention shapes, window 32, budget 8 pages of 256
HKV, HQ, D, QCL, BUDGET = 8, 32, 128, 32, 8
POOL, LAMBDA, TEMP = 7, 0.5, 0.4


def make_cfg(variant, global_score):
    from zipage_b200.compress import CompressConfig
    return CompressConfig(
        budget_blocks=BUDGET, query_cache_len=QCL, use_global_score=global_score, decay_factor=0.8,
        use_redudancy=variant != "none", lightning_redudancy=variant == "lightning",
        redudancy_lambda=LAMBDA, redudancy_temperature=TEMP, enable_pooling=True,
        continues_pooling=True, pooling_size=POOL)


class ClockSampler:
    """SM clock and clock-event (throttle) reasons sampled while the timed region runs: through
    NVML every 50 ms where the Python binding is present (read-only queries), else through an
    `nvidia-smi -lms 200` child process."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index
        self.sm, self.mx, self.reasons = [], 0.0, set()
        self.stop = threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nvml = None

    def _poll_nvml(self):
        n = self.nvml
        while True:
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                self.mx = max(self.mx, float(n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)))
                get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    n.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(self.handle))
                for name, bit in self.BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            if self.stop.wait(0.05):
                return

    def __enter__(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            r = [x.strip() for x in line.split(",")]
            try:
                self.sm.append(float(r[0]))
                self.mx = max(self.mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(self.NAMES, r[3:7]):
                if v.lower().startswith("active"):
                    self.reasons.add(n)

    def __exit__(self, *a):
        self.stop.set()
        if self.nvml is not None:
            self.thread.join(timeout=2)
        elif self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx or None,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


def cpu_baseline_sample(variant, global_score, threads, keep_sample=False):
    """The oracle (CPU restatement of the reference's PyTorch formulation) on a bounded sample of
    the same workload: L=2 layers, B=16 sequences of 9 pages, 8 KV heads, bf16 (256 units)."""
    import torch
    from oracle import zipage_oracle as O
    from zipage_b200.synthetic import algorithmic_bytes_per_unit, make_compress_workload
    torch.set_num_threads(threads)
    Ls, Bs = 2, 16
    w = make_compress_workload(Bs, Ls, HKV, HQ, D, QCL, BUDGET, dtype=torch.bfloat16, device="cpu",
                               seed=7, with_score_cache=global_score)
    ocfg = O.CompressConfig(budget_blocks=BUDGET, query_cache_len=QCL, use_global_score=global_score,
                            use_redudancy=variant != "none", lightning_redudancy=variant == "lightning",
                            redudancy_lambda=LAMBDA, redudancy_temperature=TEMP, enable_pooling=True,
                            continues_pooling=True, pooling_size=POOL)
    times = []
    moved = None
    sample = None
    for it in range(3):
        k, v = w.kv_cache[0].clone(), w.kv_cache[1].clone()
        sc = w.score_cache.clone() if w.score_cache is not None else None
        parts = {} if (keep_sample and it == 0) else None
        t0 = time.perf_counter()
        final, keep = O.compress(k, v, w.query_cache, sc, w.query_ids, w.block_tables, w.target_tables,
                                 w.compressed, ocfg, parts=parts)
        times.append(time.perf_counter() - t0)
        if moved is None:
            moved = moved_rows_per_unit(keep)
            if keep_sample:
                sample = dict(w=w, final=final, keep=keep, parts=parts, k_after=k, v_after=v)
    t = statistics.median(times[1:]) if len(times) > 1 else times[0]
    units = Ls * Bs * HKV
    st = algorithmic_bytes_per_unit(BUDGET + 1, D, QCL, HQ // HKV, 2, variant != "none", global_score, moved)
    if keep_sample:
        return sum(st.values()) * units / t / 1e9, t, units, sample
    return sum(st.values()) * units / t / 1e9, t, units


def parity_on_sample(sample, cfg, kernel_impl, dev):
    """The CUDA path on the inputs of the CPU-baseline sample, checked against what the oracle just
    computed there: fraction of differing keep flags, how many of them lie farther than one
    rounding step from the top-k cut (must be 0), and whether the compaction given the oracle's
    flags is bit-identical."""
    import torch
    from oracle.boundary import kept_set_report
    from zipage_b200 import kernel as K
    from zipage_b200.compress import compress_chunk
    w = sample["w"]
    kv = w.kv_cache.to(dev)
    q, qid, bt, tt, cp = (t.to(dev) for t in (w.query_cache, w.query_ids, w.block_tables,
                                               w.target_tables, w.compressed))
    sc = w.score_cache.to(dev) if w.score_cache is not None else None
    k2, v2 = kv[0].clone(), kv[1].clone()
    K.compress_kv(k2, v2, sample["keep"].to(dev), bt, tt)
    compaction_exact = bool(torch.equal(k2.cpu(), sample["k_after"]) and torch.equal(v2.cpu(), sample["v_after"]))
    dbg = compress_chunk(kv[0], kv[1], q, sc, qid, bt, tt, cp, cfg, impl=kernel_impl, return_debug=True)
    torch.cuda.synchronize()
    keep = dbg["keep"].cpu()
    L, B, Hkv = keep.shape[:3]
    rep = kept_set_report(sample["final"].reshape(L, B, Hkv, -1), sample["keep"].reshape(L, B, Hkv, -1),
                          keep.reshape(L, B, Hkv, -1), BS * BUDGET, torch.bfloat16, sample["parts"])
    fa, fb = dbg["final"].float().cpu(), sample["final"].float()
    fin = torch.isfinite(fb)
    return {"sample_units": L * B * Hkv, "kept_mismatch": rep["mismatch"], "differing_flags": rep["differing"],
            "outside_boundary": rep["outside"], "worst_gap_steps": rep["worst"],
            "score_max_rel_err": float((fa[fin] - fb[fin]).abs().max() / fb[fin].abs().max()),
            "compaction_bit_exact_given_flags": compaction_exact}


def reference_gpu_stage_times(sample, dev):
    """The reference's own Triton kernels (unmodified, from baseline/_ref when it is there) on the
    CPU-baseline sample's inputs, on this GPU: per-stage milliseconds, scaled nowhere.  This is the
    on-box bar for the kernels; the CPU arm stays the reported baseline.  None when the reference or
    Triton cannot be imported."""
    import torch
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "zipage" / "kernel").is_dir():
        return None
    try:
        sys.path.insert(0, str(ref))
        from zipage.kernel.attention_score import attention_score as r_att
        from zipage.kernel.compress_kv import compress_kv as r_ckv
        from zipage.kernel.lightning_redudancy_score import lightning_redudancy_score as r_light
        from zipage.kernel.raw_redudancy_score import raw_redudancy_score as r_raw
        from zipage_b200 import kernel as K
        w = sample["w"]
        kv = w.kv_cache.to(dev)
        q, qid, bt, tt = (t.to(dev) for t in (w.query_cache, w.query_ids, w.block_tables, w.target_tables))
        keep = sample["keep"].to(dev)

        def t_ms(fn, n=3):
            fn(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record(); torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n
        out = {"units": kv.shape[1] * bt.shape[0] * kv.shape[4]}
        pairs = {
            "attention_score": (lambda: r_att(kv[0], q, qid, bt), lambda: K.attention_score(kv[0], q, qid, bt)),
            "lightning_redudancy_score": (lambda: r_light(kv[0], bt, temperature=TEMP),
                                          lambda: K.lightning_redudancy_score(kv[0], bt, temperature=TEMP)),
            "raw_redudancy_score": (lambda: r_raw(kv[0], bt, temperature=TEMP),
                                    lambda: K.raw_redudancy_score(kv[0], bt, temperature=TEMP)),
        }
        for name, (rf, of) in pairs.items():
            out[name] = {"reference_triton_ms": t_ms(rf), "this_library_ms": t_ms(of)}
        k1, v1, k2, v2 = kv[0].clone(), kv[1].clone(), kv[0].clone(), kv[1].clone()
        out["compress_kv"] = {"reference_triton_ms": t_ms(lambda: r_ckv(k1, v1, keep, bt, tt), n=1),
                              "this_library_ms": t_ms(lambda: K.compress_kv(k2, v2, keep, bt, tt), n=1)}
        return out
    except Exception as e:  # the reference is optional here
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    finally:
        if str(ref) in sys.path:
            sys.path.remove(str(ref))


def moved_rows_per_unit(keep):
    """Mean number of kept rows whose slot changes: rows after the first dropped one."""
    import torch
    flat = keep.reshape(-1, keep.shape[-2] * keep.shape[-1])
    first_drop = (~flat).float().argmax(dim=1)
    any_drop = (~flat).any(dim=1)
    idx = torch.arange(flat.shape[1], device=flat.device)[None, :]
    moved = (flat & (idx > first_drop[:, None]) & any_drop[:, None]).sum(dim=1).float().mean().item()
    return moved


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        gbs, t, units = cpu_baseline_sample(args.variant, args.global_score, threads)
        if i >= args.warmup:
            vals.append(gbs); secs.append(t)
    v = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": statistics.mean(secs) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "compression op, Qwen3-8B attention shapes, 9->8 pages, window 32, "
                               f"pool {POOL}, lambda {LAMBDA}, {args.variant} redundancy (config 2)",
                   "sample": "L=2, B=16 sequences x 8 KV heads (256 units) per step"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "oracle.compress on L=2,B=16,Hkv=8,9 pages,bf16 (256 units); median of 2 after 1 warm-up"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_decode(args):
    """Paged decode attention over compressed tables: 512 sequences, context 2049..2304 tokens in 9
    pages, 32 query / 8 KV heads, head_dim 128, bf16, one layer per step (the per-layer call of the
    decode forward).  Reported as algorithmic HBM bytes per second: K and V rows of every context
    token once, plus q and out."""
    import torch
    from zipage_b200 import kernel as K
    from zipage_b200.layers.attention import paged_decode_attention
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, NBs = args.batch, BUDGET + 1
    g = torch.Generator(device="cpu").manual_seed(5)
    P = B * NBs
    kc = torch.empty((P, BS, HKV, D), dtype=torch.bfloat16, device=dev).normal_()
    vc = torch.empty((P, BS, HKV, D), dtype=torch.bfloat16, device=dev).normal_()
    table = torch.randperm(P, generator=g).view(B, NBs).to(torch.int32).to(dev)
    lens = torch.randint(BUDGET * BS + 1, NBs * BS + 1, (B,), generator=g).to(torch.int32).to(dev)
    q = torch.randn(B, 1, HQ, D, device=dev, dtype=torch.bfloat16)
    for _ in range(args.warmup):
        out = paged_decode_attention(q, kc, vc, lens, table)
    torch.cuda.synchronize()
    K.LAUNCHES = 0
    with ClockSampler(dev.index or 0) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = paged_decode_attention(q, kc, vc, lens, table)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    nbytes = float(lens.sum().item()) * HKV * D * 2 * 2 + 2 * B * HQ * D * 2
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    val = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "paged_decode_hbm_gbs", "value": val, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "paged decode attention, one layer, Qwen3-8B attention shapes (config 3 "
                               "per-layer call)", "sequences": B, "context": "2049..2304", "pages_per_seq": NBs,
                   "l2": "K/V of the batch (4.8 GB) far exceeds the 126 MB L2"},
        "tokens_per_s_per_layer": B / (ms * 1e-3),
        "gpu_launches": args.steps, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "paged_decode", "achieved": val, "peak": hbm_peak,
                     "unit": "GB/s", "frac": val / hbm_peak,
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                     "traffic": None},
    }))


def decode_step_record(args, own_group=True):
    """The decode forward of Qwen3-8B-shaped decoder blocks (hidden 4096, 32 q / 8 kv heads of 128,
    MLP 12288, bf16, random weights; cuBLAS projections, everything else this library's kernels)
    over compressed tables (context 2049..2304 tokens in 9 pages), timed launch by launch and as
    one replayed CUDA graph whose inputs are device state only.  `value` is the graph's rate with
    the inputs already in the graph's buffers; `e2e` copies the step's inputs from pinned host
    memory, adds the LM head and the sampler, and reads the tokens back.  Under torchrun (N = 2, 4, 8) the blocks are
    tensor-parallel over the ranks (heads and MLP columns split, the same batch: strong scaling)
    with every all-reduce fused into the norm that consumes it, over peer memory; the same step on
    NCCL all-reduce + the RMSNorm kernel is timed beside it."""
    import torch
    from types import SimpleNamespace
    from zipage_b200 import kernel as K
    from zipage_b200.engine.decode_graph import DecodeGraphRunner
    from zipage_b200.layers.qwen3_block import Qwen3Model
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = lib_comm = None
    rank = 0
    if world > 1:
        import torch.distributed as dist
        from zipage_b200.layers.tp_comm import LibraryCommunicator, TPCommunicator
        if own_group:
            dist.init_process_group("nccl", device_id=dev)
        rank = dist.get_rank()
        comm = TPCommunicator(max_bytes=min(args.batch, 256) * 4096 * 2, timeout_ms=2000)
        lib_comm = LibraryCommunicator()
    hkv = HKV // world

    def stage(msg):   # progress on stderr (the JSON line goes to stdout)
        if args.verbose:
            print(f"[decode_step rank {rank}] {msg}", file=sys.stderr, flush=True)
    B, Ln, NBs = min(args.batch, 256), min(args.layers, 36), BUDGET + 1
    cfg = SimpleNamespace(hidden_size=4096, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D,
                          intermediate_size=12288, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=151936,
                          num_hidden_layers=Ln, max_position_embeddings=40960, rope_theta=1e6)
    torch.manual_seed(1)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen3Model(cfg, comm).eval()
            lib_model = Qwen3Model(cfg, lib_comm).eval() if world > 1 else None
    finally:
        torch.set_default_dtype(prev)
    P = B * (NBs + 1)
    kv = torch.empty((2, Ln, P, BS, hkv, D), dtype=torch.bfloat16, device=dev).normal_()
    qc = torch.zeros((Ln, B, QCL, HQ // world, D), dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    g = torch.Generator(device="cpu").manual_seed(5)
    table = torch.randperm(P, generator=g)[: B * NBs].view(B, NBs).to(torch.int32).pin_memory()
    ntok = torch.randint(BUDGET * BS + 1, NBs * BS + 1, (B,), generator=g).to(torch.int32).pin_memory()
    ids = torch.randint(0, cfg.vocab_size, (B,), generator=g).pin_memory()
    qid = torch.arange(B, dtype=torch.int32).pin_memory()
    runner = DecodeGraphRunner(model, cfg.hidden_size, max_bs=B, max_num_blocks=NBs + 1, query_cache_len=QCL,
                               device=dev, graph_bs=[B])
    stage('model built'); runner.capture(); stage('captured')
    # the rest of ModelRunner.run for the end-to-end figure: LM head on this rank's vocabulary
    # shard (cuBLAS), the sampler (sharded over the ranks when there are several), tokens to the host
    from zipage_b200.layers.step_ops import sample
    vs = cfg.vocab_size // world
    lm_head = torch.empty((vs, cfg.hidden_size), dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
    temps = torch.full((B,), 0.7, device=dev)
    host_out = torch.empty(B, dtype=torch.int64).pin_memory()
    step_no = [0]
    d_args = [x.to(dev) for x in (ids, ntok, table, qid)]
    runner._fill(*d_args)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        if world > 1:   # the slowest rank
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def e2e_step():
        out = runner.run(ids.to(dev, non_blocking=True), ntok.to(dev, non_blocking=True),
                         table.to(dev, non_blocking=True), qid.to(dev, non_blocking=True))
        logits = torch.nn.functional.linear(out, lm_head)
        step_no[0] += 1
        tok = comm.sample(logits, temps, seed=step_no[0]) if world > 1 else sample(logits, temps, seed=step_no[0])
        host_out.copy_(tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    graph = runner.graphs[B]
    K.LAUNCHES = 0
    runner._step(B)
    per_step = K.LAUNCHES
    with ClockSampler(dev.index or 0) as clocks:
        ms_graph = timed(graph.replay)
    stage(f'graph {ms_graph:.3f} ms')
    ms_eager = timed(lambda: runner._step(B))
    stage(f'eager {ms_eager:.3f} ms')
    ms_e2e = timed(e2e_step)
    stage(f'e2e {ms_e2e:.3f} ms')
    ms_lib = None
    if world > 1:
        # The same step on the library collective + the stand-alone norm kernel, launch by launch
        # (compare with launch_by_launch_ms_per_step): replaying a captured decode graph that
        # holds NCCL all-reduces stalled on this software stack, so that route is not captured.
        lib_model.bind_caches(kv, qc)
        lib_runner = DecodeGraphRunner(lib_model, cfg.hidden_size, max_bs=B, max_num_blocks=NBs + 1,
                                       query_cache_len=QCL, device=dev, graph_bs=[B])
        lib_runner._fill(*d_args)
        ms_lib = timed(lambda: lib_runner._step(B))
        stage(f'library route, launch by launch {ms_lib:.3f} ms')
    h2d = ids.numel() * 8 + ntok.numel() * 4 + table.numel() * 4 + qid.numel() * 4
    # bytes a step must read once: every block's weights and the K/V rows of every context token
    wbytes = sum(p.numel() for n, p in model.named_parameters() if "embed" not in n) * 2
    kvbytes = float(ntok.sum().item()) * hkv * D * 2 * 2 * Ln
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    ach = (wbytes + kvbytes) / (ms_graph * 1e-3) / 1e9
    # One compression of every sequence per 256 decode steps (a page fills, the table is back at
    # budget + 1 pages): timed on this step's own caches through the host-facing call and folded
    # into the rate the way the engine's generate() accounts decode throughput
    # (zipage/engine/zipage_engine.py:255-265: tokens of the decode steps over the time between them).
    from zipage_b200.engine.compressor import Compressor
    qc.normal_()
    ccomp = Compressor(kv, qc, None, make_cfg("lightning", False), layer_stride=8)
    c_tables = table.tolist()
    c_qids = qid.tolist()
    c_ms = []
    for i in range(3):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        ccomp.compress_tables(c_tables, c_tables, c_qids, [True] * B)
        c_ms.append((time.perf_counter() - t0) * 1e3)
    compress_ms = min(c_ms[1:])
    if world > 1:
        t = torch.tensor([compress_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        compress_ms = float(t.item())
    tok_s_with_compress = 256.0 * B / (256.0 * ms_e2e + compress_ms) * 1e3
    allreduce_bit_exact = None
    if world > 1:
        # the peer-memory all-reduce against the fp32 sum of the gathered inputs taken in rank order
        xg = torch.Generator(device=dev).manual_seed(100 + rank)
        x = torch.randn(B, 4096, device=dev, generator=xg).to(torch.bfloat16)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        acc = parts[0].float()
        for p_ in parts[1:]:
            acc = acc + p_.float()
        got = comm.all_reduce(x.clone())
        flag = torch.tensor([int(torch.equal(got, acc.to(torch.bfloat16)))], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        allreduce_bit_exact = bool(flag.item())
        status = comm.status()
        comm.close()
        if own_group:
            dist.destroy_process_group()
        if rank != 0:
            return None
    return ({
        "metric": "decode_step_tokens_per_s", "value": B / (ms_graph * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_graph, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decode forward, Qwen3-8B-shaped blocks, compressed tables (2049..2304 tokens "
                               "in 9 pages), one CUDA graph replay per step", "sequences": B, "layers": Ln,
                   "parallelism": f"tp{world}: all-reduce fused into the norms over peer memory" if world > 1 else "none",
                   "l2": "weights + K/V of a step (%.1f GB) far exceed the 126 MB L2" % ((wbytes + kvbytes) / 1e9)},
        "launch_by_launch_ms_per_step": ms_eager, "graph_speedup": ms_eager / ms_graph,
        "library_collective_launch_by_launch_ms_per_step": ms_lib, "comm_status": status if world > 1 else None,
        "e2e": {"value": B / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": host_out.numel() * 8,
                "includes": "LM head (cuBLAS) + sampler" + (" over the sharded vocabulary" if world > 1 else "")},
        "gpu_launches": per_step * args.steps, "own_kernels_per_step": per_step, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "whole step (this rank's weights + K/V read once)", "achieved": ach,
                     "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback", "traffic": None},
        "compress_ms_per_256_steps": compress_ms,
        "tokens_per_s_with_compression": tok_s_with_compress,
        "all_reduce_bit_exact_vs_fp32_rank_order_sum": allreduce_bit_exact,
    })


def engine_decode_records(modes=("reference", "kernels", "graph"), requests=192, max_tokens=600):
    """Decode tokens/s through the reference ENGINE (ZipLLM.generate of baseline/_ref: its scheduler,
    block manager, prefill and sampler) on a synthetic Qwen3-8B-shaped model, 2300-token random
    prompts, a budget of 8 pages, lightning redundancy + pooling, two compressions per request:
    `reference` = the engine as it is (Triton + flash-attn), `kernels` = zipage_b200.kernel bound in
    model_runner.py, `graph` = also the attention layer and the decode forward as replayed CUDA
    graphs, `native` = also the native scheduler and page manager in place of the engine's.  Each mode is a child process (tests/ref_engine.py); accounting is the engine's own
    time_record (decode_sum + compress_sum)."""
    out = {"workload": f"Qwen3-8B shapes, random-init bf16, {requests} concurrent requests, prompts of 2300 "
                       f"uniform-random ids, {max_tokens} generated tokens each, budget 8 x 256, temperature 0.6"}
    if not (ROOT / "baseline" / "_ref" / "zipage" / "llm.py").is_file():
        out["unavailable"] = "the reference is not installed under baseline/_ref"
        return out
    common = ["--layers", "36", "--hidden", "4096", "--inter", "12288", "--hq", "32", "--hkv", "8", "--vocab", "151936",
              "--requests", str(requests), "--prompt-len", "2300", "--max-tokens", str(max_tokens), "--budget", "8",
              "--qcl", "32", "--lightning", "--pooling", "--max-model-len", "4096", "--model-dir", "/tmp/zp_q8b",
              "--gpu-mem", "0.62", "--warmup-requests", "4"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")}
    for i, m in enumerate(modes):
        res = Path("/tmp") / f"zp_engine_{m}.json"
        try:
            r = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_engine.py"), "--mode", m, "--out", str(res),
                                "--port", str(2411 + i), *common], capture_output=True, text=True, timeout=900, env=env)
            if r.returncode != 0:
                out[m] = {"unavailable": (r.stderr or r.stdout)[-300:]}
                continue
            d = json.loads(res.read_text())
            e = d["engine_time_record"]
            out[m] = {"decode_tokens_per_s": d["decode_tok_per_s"],
                      "decode_tokens_per_s_excluding_compress": d["decode_tok_per_s_excluding_compress"],
                      "prefill_tokens_per_s": d["prefill_tok_per_s"], "decode_s": e.get("decode_sum"),
                      "compress_s": e.get("compress_sum"), "decode_tokens": d["decode_tokens"],
                      "wall_s": d["wall_s"], "generated_tokens_per_wall_s": d["generated_tokens"] / d["wall_s"]}
        except Exception as ex:
            out[m] = {"unavailable": f"{type(ex).__name__}: {ex}"[:300]}
    ref = out.get("reference", {}).get("decode_tokens_per_s")
    for m in modes:
        if ref and out.get(m, {}).get("decode_tokens_per_s"):
            out[m]["vs_reference_engine"] = out[m]["decode_tokens_per_s"] / ref
    return out


def run_engine_decode(args):
    rec = engine_decode_records(tuple(args.engine_modes.split(",")))
    g = rec.get("graph", {})
    print(json.dumps({"metric": "engine_decode_tokens_per_s", "value": g.get("decode_tokens_per_s"), "unit": "tokens/s",
                      "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "config": {"workload": rec["workload"]},
                      "modes": rec}))


def run_long_prompt(args):
    """First compression after a long prompt (config 5): Qwen3-32B attention shapes as ONE rank of a
    TP=8 job sees them (64 layers, 8 query heads and 1 KV head of 128 per rank), `--batch` sequences
    whose tables hold 64..128 full pages (16k..32k tokens) compressed into 8 (+1) pages, bf16, window
    32 (G*QCL = 256 window rows: two passes of the window kernel), lightning and exact similarity;
    and the varlen prefill attention of one 32 768-token prompt at the same per-rank head counts."""
    import torch
    from zipage_b200 import kernel as K
    from zipage_b200.compress import CompressConfig, compress_chunk
    from zipage_b200.engine.compressor import Compressor
    from zipage_b200.layers.attention import varlen_prefill_attention
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, L, hkv, hq = min(args.batch, 64), 64, 1, 8
    g = torch.Generator().manual_seed(17)
    pages = torch.randint(64, 129, (B,), generator=g).tolist()
    pages[0], pages[1] = 128, 64
    w = make_compress_workload(B, L, hkv, hq, D, QCL, BUDGET, pages_per_seq=pages, dtype=torch.bfloat16,
                               device=dev, seed=5, compressed_prob=0.0, fresh_target_prob=0.5)
    out = {}
    chunk = 8   # layer_stride of the engine
    for variant in ("lightning", "exact"):
        cfg = make_cfg(variant, False)
        comp = Compressor(w.kv_cache, w.query_cache, None, cfg, layer_stride=chunk)
        tables = [[int(x) for x in row if x != -1] for row in w.tables_plain.cpu().tolist()]
        targets = w.target_tables.cpu().tolist()
        ts = None
        for it in range(2):   # the compaction is in place: the second pass recompresses (same shapes, same work)
            comp.time_record.clear()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            comp.compress_tables(tables, targets, w.query_ids.cpu().tolist(), [False] * B, timed=True)
            wall = time.perf_counter() - t0
            ts = {k: v * 1e3 for k, v in comp.time_record.items() if k.endswith("_sum")}
        tok = sum(pages) * BS
        flops = sum(2.0 * (p_ * BS) ** 2 * D for p_ in pages) * L * hkv
        out[variant] = {"ms": sum(ts.values()), "wall_ms": wall * 1e3, "stage_ms": ts,
                        "tokens_scored_per_s": tok * L / (sum(ts.values()) * 1e-3)}
        if variant == "exact":
            out[variant]["similarity_tflops_dense_count"] = flops / (ts["redudancy_score_sum"] * 1e-3) / 1e12
        del comp
    # prefill attention of one 32k prompt at the per-rank head counts
    S = 32768
    q = torch.randn(S, hq, D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(S, hkv, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(S, hkv, D, device=dev, dtype=torch.bfloat16)
    cu = torch.tensor([0, S], device=dev, dtype=torch.int32)
    fn = lambda: varlen_prefill_attention(q, k, v, S, cu, S, cu, impl="tcgen05")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    out["prefill_1x32768_8q_1kv"] = {"ms": ms, "tflops": 4.0 * D * (S * S / 2.0) * hq / (ms * 1e-3) / 1e12}
    print(json.dumps({
        "metric": "first_compression_ms", "value": out["lightning"]["ms"], "unit": "ms", "n_gpus": 1,
        "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "first compression of long prompts, one TP=8 rank of Qwen3-32B (config 5)",
                   "sequences": B, "layers": L, "pages_per_seq": "64..128", "kv_heads_per_rank": hkv,
                   "q_heads_per_rank": hq, "window": QCL, "total_pages": sum(pages)},
        "results": out}))


def run_decode_step(args):
    rec = decode_step_record(args, own_group=True)
    if rec is not None:
        print(json.dumps(rec))


def run_tp_allreduce(args):
    """The all-reduce of a row-parallel projection's output for a 512-sequence decode step of a
    hidden-4096 model (4 MiB of bf16 per rank) followed by the residual add + RMSNorm of the block:
    one fused launch over peer memory against dist.all_reduce + the RMSNorm kernel.  A step = one
    such reduction, `steps` of them replayed as one CUDA graph; times are CUDA events, the maximum
    over the ranks."""
    import torch
    import torch.distributed as dist
    from zipage_b200.layers.step_ops import rms_norm
    from zipage_b200.layers.tp_comm import TPCommunicator
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        print(json.dumps({"metric": "allreduce_add_rms_norm_us", "unavailable": "needs 2, 4 or 8 ranks (torchrun)"}))
        return
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    rows, hidden = args.batch, 4096
    comm = TPCommunicator(max_bytes=rows * hidden * 2)
    g = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
    res = torch.randn(rows, hidden, device=dev, generator=g).to(torch.bfloat16)
    w = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    y = x.clone()

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    flagged_ok = rows * hidden * 2 <= (2 << 20)

    def nccl_step():
        y.copy_(x)
        dist.all_reduce(y)
        rms_norm(y, w, 1e-6, res)

    cases = {
        "fused_auto": lambda: comm.all_reduce_add_rms_norm(x, res, w, 1e-6),
        "fused_one_shot": lambda: comm.all_reduce_add_rms_norm(x, res, w, 1e-6, algo="one_shot"),
        "fused_two_shot": lambda: comm.all_reduce_add_rms_norm(x, res, w, 1e-6, algo="two_shot"),
        "plain_one_shot": lambda: comm.all_reduce(x, out=y, algo="one_shot"),
        "plain_two_shot": lambda: comm.all_reduce(x, out=y, algo="two_shot"),
        "plain_flagged_lines": (lambda: comm.all_reduce(x, out=y, algo="flagged_lines")) if flagged_ok else None,
        "fused_flagged_lines": (lambda: comm.all_reduce_add_rms_norm(x, res, w, 1e-6, algo="flagged_lines")) if flagged_ok else None,
        "nccl_all_reduce": lambda: dist.all_reduce(y),
        "nccl_all_reduce_then_rms_norm": nccl_step,
    }
    # Launch by launch, a 20 us collective is bound by the host's call overhead on both sides of the
    # comparison; the device time shows when `steps` calls are replayed as one CUDA graph (which is
    # how a decode step issues them).
    def graphed(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(); dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.steps):
                fn()
        return graph

    graphs = {k: graphed(fn) for k, fn in cases.items() if fn is not None}

    def timed_graph(graph):
        graph.replay()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cases = {k: v for k, v in cases.items() if v is not None}
    runs = {k: [] for k in cases}
    gruns = {k: [] for k in cases}
    with ClockSampler(dev.index or 0) as clocks:
        for _ in range(3):            # three rounds over all cases; the median of each is reported
            for k, fn in cases.items():
                runs[k].append(timed(fn))
                gruns[k].append(timed_graph(graphs[k]))
    t_eager = {k: sorted(v)[1] for k, v in runs.items()}
    t = {k: sorted(v)[1] for k, v in gruns.items()}
    del graphs
    status = comm.status()
    comm.close()
    msg = rows * hidden * 2
    two_shot = world > 2
    link_bytes = msg * (2 * (world - 1) / world if two_shot else world - 1)   # into each GPU
    target_us = link_bytes / 770e9 * 1e6
    if rank == 0:
        print(json.dumps({
            "metric": "allreduce_add_rms_norm_us", "value": t["fused_auto"], "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t["fused_auto"] / 1e3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "all-reduce + residual + RMSNorm of one row-parallel projection, decode step",
                       "rows": rows, "hidden": hidden, "message_bytes": msg,
                       "l2": "4 MiB messages live in L2 by design; no flush"},
            "times_us": t, "launch_by_launch_times_us": t_eager, "comm_status": status,
            "gpu_launches": args.steps * 3 * 5 * 2, "clocks": clocks.summary(),
            "roofline": {"bound": "nvlink", "kernel": "all_reduce_kernel (fused)", "bytes_into_each_gpu": link_bytes,
                         "peak": 770.0, "unit": "GB/s", "achieved": link_bytes / (t["fused_auto"] * 1e-6) / 1e9,
                         "frac": target_us / t["fused_auto"], "peak_source": "measured peer copy, per direction",
                         "traffic": None},
        }))
    dist.destroy_process_group()


def run_step_ops(args):
    """The per-step ops of one decoder layer at Qwen3-8B sizes (hidden 4096, intermediate 12288,
    32 query / 8 KV heads of 128) on a prefill-sized batch of tokens, so that every input is larger
    than the L2, plus the sampler at the full vocabulary.  Each op is timed alone with CUDA events
    and reported as algorithmic HBM bytes per second (what the op must read and write once)."""
    import torch
    from zipage_b200 import kernel as K
    from zipage_b200.layers import step_ops as P
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    N, H, I, V, Bs = args.tokens, 4096, 12288, 151936, 512
    bf = torch.bfloat16
    x = torch.randn(N, H, device=dev, dtype=bf)
    res = torch.randn(N, H, device=dev, dtype=bf)
    w = torch.ones(H, device=dev, dtype=bf)
    gate_up = torch.randn(N, 2 * I, device=dev, dtype=bf)
    qkv = torch.randn(N, (HQ + 2 * HKV) * D, device=dev, dtype=bf)
    wq, wk = torch.ones(D, device=dev, dtype=bf), torch.ones(D, device=dev, dtype=bf)
    pos = torch.randint(0, 32768, (N,), device=dev)
    cs = P.rope_cos_sin_cache(D, 32768, 1e6, dev)
    pages = (N + BS - 1) // BS
    kc = torch.empty((pages * BS, HKV, D), device=dev, dtype=bf)
    vc = torch.empty_like(kc)
    # a prefill batch: consecutive tokens fill consecutive slots of a page, the pages are scattered
    tok = torch.arange(N, device=dev)
    slots = (torch.randperm(pages, device=dev)[tok // BS] * BS + tok % BS).to(torch.int32)
    logits = torch.randn(Bs, V, device=dev, dtype=bf)
    temps = torch.full((Bs,), 0.6, device=dev)
    e = 2
    ops = {
        "add_rms_norm": (lambda: P.rms_norm(x, w, 1e-6, residual=res), N * H * e * 4 + H * e),
        "silu_and_mul": (lambda: P.silu_and_mul(gate_up), N * I * e * 3),
        "qk_norm_rope_store": (lambda: P.qk_norm_rope_store(qkv, pos, cs, wq, wk, 1e-6, HQ, HKV, D, k_cache=kc,
                                                            v_cache=vc, slot_mapping=slots, return_k=False),
                               N * (HQ + 2 * HKV) * D * e + N * HQ * D * e + 2 * N * HKV * D * e + N * (D * 4 + 12)),
        "sample (built-in draws)": (lambda: P.sample(logits, temps, seed=1), Bs * V * e + Bs * 12),
    }
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    per_op, total_ms, total_bytes = {}, 0.0, 0.0
    K.LAUNCHES = 0
    with ClockSampler(dev.index or 0) as clocks:
        for name, (fn, nbytes) in ops.items():
            for _ in range(args.warmup):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            gbs = nbytes / (ms * 1e-3) / 1e9
            per_op[name] = {"ms": ms, "algorithmic_bytes": nbytes, "gbs": gbs, "frac": gbs / hbm_peak}
            total_ms += ms
            total_bytes += nbytes
    val = total_bytes / (total_ms * 1e-3) / 1e9
    worst = min(per_op, key=lambda k_: per_op[k_]["frac"])
    print(json.dumps({
        "metric": "step_ops_hbm_gbs", "value": val, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "per-step ops of one Qwen3-8B decoder layer + sampler", "tokens": N,
                   "sampler_rows": Bs, "vocab": V,
                   "l2": "every op's input is larger than the 126 MB L2 (sampler: 155 MB of logits)"},
        "per_op": per_op, "gpu_launches": K.LAUNCHES, "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": worst, "achieved": per_op[worst]["gbs"], "peak": hbm_peak,
                     "unit": "GB/s", "frac": per_op[worst]["frac"],
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback", "traffic": None},
    }))


def run_prefill(args):
    """Varlen causal prefill attention of one layer at Qwen3-8B head shapes (32 query / 8 KV heads of
    128, bf16): 4 sequences of 4096 tokens and one of 16 384 (config 5 sizes), dense K/V.  Reported
    as causal attention flops per second, 4 * D * sum(len^2) / 2 per query head, for the tcgen05
    kernel, with the mma.sync kernel timed beside it."""
    import torch
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks = {}
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    peak = peaks.get("bf16_tflops", 1590.0)
    res = {}
    launches = 0
    with ClockSampler(dev.index or 0) as clocks:
        for S, B in [(4096, 4), (16384, 1)]:
            q = torch.randn(B * S, HQ, D, device=dev, dtype=torch.bfloat16)
            k = torch.randn(B * S, HKV, D, device=dev, dtype=torch.bfloat16)
            v = torch.randn(B * S, HKV, D, device=dev, dtype=torch.bfloat16)
            cu = torch.arange(0, (B + 1) * S, S, device=dev, dtype=torch.int32)
            flops = 4.0 * D * (S * S / 2.0) * HQ * B
            for impl in ("tcgen05", "simt"):
                fn = lambda: varlen_prefill_attention(q, k, v, S, cu, S, cu, impl=impl)
                for _ in range(args.warmup):
                    fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.steps):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / args.steps
                res[f"{B}x{S} {'tcgen05' if impl == 'tcgen05' else 'mma.sync'}"] = {
                    "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}
                launches += args.steps if impl == "tcgen05" else 0
    head = res["1x16384 tcgen05"]
    print(json.dumps({
        "metric": "prefill_attention_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "varlen causal prefill attention, one layer, 32 q / 8 kv heads of 128, 1 x 16384 tokens "
                               "(headline) and 4 x 4096 tokens", "l2": "q, k, v and out of a call: 168 MB > 126 MB L2"},
        "cases": res, "gpu_launches": launches, "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "kernel": "prefill_tc_kernel", "achieved": head["tflops"], "peak": peak,
                     "unit": "TFLOP/s", "frac": head["tflops"] / peak,
                     "executed": head["tflops"] * 1.5,
                     "executed_note": "the kernel recomputes Q.K^T in its second pass: 3 tile products per 2 counted",
                     "peak_source": "measured burst cuBLAS bf16 (MEASURED_PEAKS.json)" if peaks else "fallback",
                     "traffic": None},
    }))


def native_engine_record(args, own_group=True):
    """Decode tokens/s through the serving loop built from this library only
    (zipage_b200/engine/native_engine.py): same workload and accounting as the engine_decode
    workload (Qwen3-8B shapes, random-init bf16, `--engine-requests` concurrent requests with
    2300-token prompts, 600 sampled tokens each at temperature 0.6, budget 8 pages, lightning
    redundancy + pooling; decode tokens over decode_sum + compress_sum).  Under torchrun the loop
    runs tensor-parallel: every rank its own scheduler replica, all-reduces over peer memory,
    sampling over the sharded vocabulary."""
    import torch
    from types import SimpleNamespace
    from zipage_b200.compress import CompressConfig
    from zipage_b200.engine.native_engine import NativeEngine
    from zipage_b200.engine.scheduler import SamplingParams, Sequence
    from zipage_b200.layers.qwen3_block import Qwen3Model
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm, rank = None, 0
    R, PROMPT, GEN = args.engine_requests, args.engine_prompt, args.engine_gen
    if world > 1:
        import torch.distributed as dist
        from zipage_b200.layers.tp_comm import TPCommunicator
        if own_group:
            dist.init_process_group("nccl", device_id=dev)
        rank = dist.get_rank()
        comm = TPCommunicator(max_bytes=256 * 4096 * 2, timeout_ms=2000, large_messages="library")
    Ln = min(args.layers, 36)
    cfg = SimpleNamespace(hidden_size=4096, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D,
                          intermediate_size=12288, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=151936,
                          num_hidden_layers=Ln, max_position_embeddings=40960, rope_theta=1e6)
    torch.manual_seed(1)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen3Model(cfg, comm).eval()
    finally:
        torch.set_default_dtype(prev)
    pages = R * (BUDGET + 2) + 64
    lm_head = torch.empty((cfg.vocab_size // world, cfg.hidden_size), dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
    # no more pages than fit beside the weights (the scheduler then admits and preempts as the
    # reference's does when blocks run out)
    page_bytes = 2 * Ln * BS * (HKV // world) * D * 2
    free = torch.cuda.mem_get_info(dev)[0] - R * Ln * QCL * (HQ // world) * D * 2 - (32 << 30)
    pages = max(R * 3, min(pages, int(free // page_bytes)))
    kv = torch.zeros((2, Ln, pages, BS, HKV // world, D), dtype=torch.bfloat16, device=dev)
    qc = torch.zeros((Ln, R, QCL, HQ // world, D), dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    sched_cfg = SimpleNamespace(max_num_seqs=R, max_num_batched_tokens=32768, eos=-1, num_kvcache_blocks=pages,
                                kvcache_block_size=BS, max_cache_blocks_per_seq=BUDGET,
                                enable_prefix_cache=bool(args.engine_prefix_cache),
                                max_concurrency=R, enable_hybrid_engine=False, query_cache_len=QCL)
    ccfg = CompressConfig(budget_blocks=BUDGET, query_cache_len=QCL, use_redudancy=True, lightning_redudancy=True,
                          redudancy_lambda=0.5, enable_pooling=True)
    eng = NativeEngine(model, lm_head, kv, qc, sched_cfg, ccfg, cfg.hidden_size, comm=comm, max_bs=R,
                       max_model_len=4096, greedy=False)
    g = torch.Generator().manual_seed(1)
    sp = SamplingParams(0.6, GEN, True)

    def requests(n, length, max_tokens):
        return [Sequence(torch.randint(2, cfg.vocab_size, (length,), generator=g).tolist(),
                         SamplingParams(0.6, max_tokens, True)) for _ in range(n)]
    eng.generate(requests(4, (BUDGET + 1) * BS - 4, 8))      # warm-up across one compression
    eng.time_record.clear()
    torch.cuda.synchronize()
    with ClockSampler(dev.index or 0) as clocks:
        t0 = time.perf_counter()
        out = eng.generate(requests(R, PROMPT, GEN))
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    tr = eng.time_record
    gen = sum(len(v) for v in out.values())
    decode_s = tr["decode_sum"] + tr["compress_sum"]
    status = comm.status() if comm is not None else 0
    rec = None
    if rank == 0:
        rec = {
            "metric": "engine_decode_tokens_per_s", "value": tr["decode_tokens"] / decode_s, "unit": "tokens/s",
            "n_gpus": world, "steps": int(tr["decode_tokens"] // R), "warmup": 1, "ms_per_step": decode_s / (tr["decode_tokens"] / R) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"own serving loop, Qwen3-8B shapes ({Ln} blocks), random-init bf16, {R} concurrent requests, "
                                   f"prompts of {PROMPT} uniform-random ids, {GEN} sampled tokens each, budget {BUDGET} x {BS}, "
                                   "lightning redundancy + pooling", "parallelism": f"tp{world}",
                       "kv_pages": pages, "prefix_cache": bool(args.engine_prefix_cache)},
            "decode_tokens": int(tr["decode_tokens"]), "decode_s": tr["decode_sum"], "compress_s": tr["compress_sum"],
            "compressions": int(tr["compress_reqs"]), "prefill_tokens_per_s": R * PROMPT / tr["prefill_sum"],
            "decode_tokens_per_s_excluding_compress": tr["decode_tokens"] / tr["decode_sum"],
            "wall_s": wall, "generated_tokens": gen, "generated_tokens_per_wall_s": gen / wall,
            "comm_status": status, "clocks": clocks.summary(),
        }
    if comm is not None:
        comm.close()
    return rec


def run_native_engine(args):
    rec = native_engine_record(args, own_group=True)
    if rec is not None:
        print(json.dumps(rec))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def run_host_control(args):
    """Host time per decode step of the control plane at `--requests` concurrent requests: the
    native scheduler's array calls (schedule, the runner's input arrays, postprocess) and, when an
    installed copy of the reference is present under baseline/_ref, the reference's Python
    Scheduler.schedule() + postprocess() on the same request stream (its prepare_decode list
    building, model_runner.py:633-675, is not included: it needs the GPU runner).  No GPU work."""
    import random
    import statistics
    import types
    import numpy as np
    from zipage_b200.engine import scheduler as own
    n = args.requests
    cfg = types.SimpleNamespace(max_num_seqs=n, max_num_batched_tokens=1 << 22, eos=-1, num_kvcache_blocks=n * 12,
                                kvcache_block_size=256, max_cache_blocks_per_seq=8, enable_prefix_cache=False,
                                max_concurrency=n, enable_hybrid_engine=False, query_cache_len=32)
    rng = random.Random(0)
    prompts = [[rng.randrange(1000) for _ in range(600 + (i % 200))] for i in range(n)]
    steps = 2200      # every sequence crosses 2304 tokens: first compressions are inside the window

    def drive_own():
        s = own.Scheduler(cfg)
        for p in prompts:
            s.add(own.Sequence(p, own.SamplingParams(0.6, 100000, True)))
        out = {k: np.empty(n, np.int32) for k in ("input_ids", "num_tokens", "query_ids")}
        out["block_tables"] = np.empty((n, 10), np.int32)
        tok = np.ones(n, np.int32)
        times, compressions = [], 0
        while True:
            h, pf = s.schedule_batch()
            if not pf:
                break
            s.mark_prefilled(h)
            s.postprocess_batch(h, tok[:len(h)])
        first = True
        for _ in range(steps):
            t0 = time.perf_counter()
            if not first:
                h, pf = s.schedule_batch()
            first = False
            d = s.decode_inputs(h, table_width=10, out=out)
            due = s.compress_due(h)
            if len(due):
                compressions += len(due)
                s.compress_inputs(due, table_width=10)
                s.postprocess_batch(due)
            s.postprocess_batch(h, tok[:len(h)])
            times.append(time.perf_counter() - t0)
        return times, compressions

    def drive_reference():
        ref = ROOT / "baseline" / "_ref"
        if not (ref / "zipage" / "engine" / "scheduler.py").exists():
            return None
        sys.path.insert(0, str(ref))
        try:
            from zipage.engine.scheduler import Scheduler
            from zipage.engine.sequence import Sequence
            from zipage.sampling_params import SamplingParams
        except Exception:
            return None
        s = Scheduler(cfg)
        for p in prompts:
            s.add(Sequence(p, SamplingParams(temperature=0.6, max_tokens=100000, ignore_eos=True)))
        while True:
            seqs, pf = s.schedule()
            if not pf:
                break
            for q in seqs:
                q.num_cached_tokens = len(q)
            s.postprocess(seqs, [1] * len(seqs))
        times, first = [], True
        for _ in range(steps):
            t0 = time.perf_counter()
            if not first:
                seqs, pf = s.schedule()
            first = False
            due = [q for q in seqs if q.require_compress]
            if due:
                s.postprocess(due)
            s.postprocess(seqs, [1] * len(seqs))
            times.append(time.perf_counter() - t0)
        return times

    t_own, compressions = drive_own()
    t_ref = drive_reference()
    rec = {
        "metric": "host_control_ms_per_decode_step", "value": statistics.mean(t_own) * 1e3, "unit": "ms",
        "n_gpus": 0, "steps": steps, "warmup": 0, "ms_per_step": statistics.mean(t_own) * 1e3,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": f"host control plane, {n} concurrent requests of 600..800 prompt tokens decoded past "
                               "their first compression (budget 8 pages)", "requests": n},
        "native": {"mean_ms": statistics.mean(t_own) * 1e3, "median_ms": statistics.median(t_own) * 1e3,
                   "max_ms": max(t_own) * 1e3, "compressions": compressions,
                   "calls_per_step": "schedule + decode_inputs + postprocess (+ compress_inputs + postprocess when due)"},
        "reference_python": None if t_ref is None else {
            "mean_ms": statistics.mean(t_ref) * 1e3, "median_ms": statistics.median(t_ref) * 1e3,
            "max_ms": max(t_ref) * 1e3, "calls_per_step": "Scheduler.schedule + postprocess (no prepare_decode)"},
        "gpu_launches": 0,
    }
    print(json.dumps(rec))


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "host_control":
        return run_host_control(args)
    if args.workload == "native_engine":
        return run_native_engine(args)
    if args.workload == "prefill":
        return run_prefill(args)
    if args.workload == "decode":
        return run_decode(args)
    if args.workload == "step_ops":
        return run_step_ops(args)
    if args.workload == "decode_step":
        return run_decode_step(args)
    if args.workload == "tp_allreduce":
        return run_tp_allreduce(args)
    if args.workload == "engine_decode":
        return run_engine_decode(args)
    if args.workload == "long_prompt":
        return run_long_prompt(args)

    import torch
    import torch.distributed as dist
    from zipage_b200 import kernel as K
    from zipage_b200.compress import compress_chunk
    from zipage_b200.engine.compressor import Compressor
    from zipage_b200.synthetic import (algorithmic_bytes_per_unit, bytes_per_sequence,
                                       make_compress_workload)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # KV heads are sharded over ranks; per-rank work is held fixed (weak scaling): with 1/world of
    # the heads per page a rank serves world x the sequences, as the engine's concurrency would.
    hkv, hq = HKV // world, HQ // world
    L = args.layers
    itemsize = 2
    per_seq = bytes_per_sequence(L, BUDGET + 1, hkv, hq, D, QCL, itemsize, args.global_score)
    per_seq += L * hkv * (BUDGET + 1) * BS * 8  # scores, redundancy logits, flags, final
    free, total = torch.cuda.mem_get_info()
    B = min(args.batch * world, int((free - (8 << 30)) // per_seq))
    B -= B % 8
    assert B > 0, "no room for a single sequence"
    cfg = make_cfg(args.variant, args.global_score)
    w = make_compress_workload(B, L, hkv, hq, D, QCL, BUDGET, dtype=torch.bfloat16, device=dev,
                               seed=1234 + rank, with_score_cache=args.global_score)
    chunk = args.layer_chunk or L
    comp = Compressor(w.kv_cache, w.query_cache, w.score_cache, cfg, layer_stride=chunk,
                      impl=args.kernel_impl)
    if args.variant == "exact":
        comp._ensure_workspace(B, BUDGET + 1)
    seq_tables = w.tables_plain.cpu().tolist()
    seq_targets = w.target_tables.cpu().tolist()
    seq_qids = w.query_ids.cpu().tolist()
    seq_comp = w.compressed.cpu().tolist()

    nb_last = BUDGET   # table position of the page that is appended to between compressions
    last_pages = w.tables_plain[:, nb_last].long()
    fresh = torch.empty((B, BS, hkv, D), dtype=torch.bfloat16, device=dev)
    rgen = torch.Generator(device=dev).manual_seed(99 + rank)

    def refresh():
        """Between steps, outside every timed event: the engine's steady state.  A compression leaves
        8 compacted pages and the page new tokens are appended to; 256 decode steps later that page
        is full of new keys and the window holds new queries.  Refilling both makes every step the
        same work on fresh data instead of a recompression of its own output."""
        for t in range(2):
            for l in range(L):
                fresh.normal_(generator=rgen)
                w.kv_cache[t, l].index_copy_(0, last_pages, fresh)
        w.query_cache.normal_(generator=rgen)

    class StageTimers:
        """Per-stage CUDA events of one step, on the stream the kernels are launched on."""
        def __init__(self):
            self.events = []

        def __call__(self, name):
            outer = self

            class _Ctx:
                def __enter__(self_):
                    self_.st = torch.cuda.Event(enable_timing=True)
                    self_.ed = torch.cuda.Event(enable_timing=True)
                    self_.st.record()

                def __exit__(self_, *a):
                    self_.ed.record()
                    outer.events.append((name, self_.st, self_.ed))
                    return False
            return _Ctx()

        def totals(self):
            out = {}
            for name, st, ed in self.events:
                out[name] = out.get(name, 0.0) + st.elapsed_time(ed)
            return out

    def device_step(timers=None, want_keep=False):
        moved = []
        for l0 in range(0, L, chunk):
            sl = slice(l0, min(L, l0 + chunk))
            keep = compress_chunk(w.kv_cache[0, sl], w.kv_cache[1, sl], w.query_cache[sl],
                                  None if w.score_cache is None else w.score_cache[sl], w.query_ids,
                                  w.block_tables, w.target_tables, w.compressed, cfg, impl=args.kernel_impl,
                                  workspace=comp.workspace, timers=timers, return_keep=want_keep)
            if want_keep:
                moved.append((keep, sl.stop - sl.start))
        return moved

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        refresh()
        device_step()
    barrier()
    K.LAUNCHES = 0
    step_ms, stage_sums, moved_steps = [], {}, []
    region0 = time.perf_counter()
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            refresh()
            torch.cuda.synchronize()
            timers = StageTimers()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            kept = device_step(timers, want_keep=True)
            ev1.record()
            torch.cuda.synchronize()
            step_ms.append(ev0.elapsed_time(ev1))
            for name, ms in timers.totals().items():
                stage_sums[name] = stage_sums.get(name, 0.0) + ms
            # moved rows of THIS step, every layer (a device-side reduction, outside the events)
            tot = sum(moved_rows_per_unit(k) * n for k, n in kept) / L
            moved_steps.append(tot)
            del kept
        barrier()
    region_s = time.perf_counter() - region0
    launches = K.LAUNCHES
    dev_ms = sum(step_ms)
    stage_ms = {k + "_sum": v / args.steps for k, v in stage_sums.items()}
    moved = statistics.mean(moved_steps)

    # end to end through the host-facing call: host lists -> pinned -> H2D, kernels, sync, D2H
    e2e_times = []
    for i in range(2 + args.steps):   # two untimed calls first: staging buffers and scratch get allocated
        refresh()
        barrier()
        t0 = time.perf_counter()
        new_tables, ctx_lens = comp.compress_tables(seq_tables, seq_targets, seq_qids, seq_comp)
        if i >= 2:
            e2e_times.append(time.perf_counter() - t0)
    e2e_s = statistics.mean(e2e_times)
    h2d = comp.last_h2d_bytes
    d2h = comp.last_d2h_bytes

    # the engine's real call shape: ModelRunner.compress gets at most 600 // table_len sequences per
    # call (zipage/engine/zipage_engine.py:143-156) and walks the layers 8 at a time (config.py:45)
    eng = None
    if world == 1 and not args.no_cpu_baseline:
        nb_seq = min(B, 600 // (BUDGET + 1))
        small = Compressor(w.kv_cache, w.query_cache, w.score_cache, cfg, layer_stride=8,
                           impl=args.kernel_impl)
        ts = []
        for i in range(args.warmup + args.steps):
            refresh()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            small.compress_tables(seq_tables[:nb_seq], seq_targets[:nb_seq], seq_qids[:nb_seq], seq_comp[:nb_seq])
            if i >= args.warmup:
                ts.append(time.perf_counter() - t0)
        for _ in range(2):   # the second call's stage events are free of allocator stalls
            refresh()
            torch.cuda.synchronize()
            small.time_record.clear()
            small.compress_tables(seq_tables[:nb_seq], seq_targets[:nb_seq], seq_qids[:nb_seq],
                                  seq_comp[:nb_seq], timed=True)
        kern_ms = sum(v for k, v in small.time_record.items() if k.endswith("_sum")) * 1e3
        eng = {"sequences": nb_seq, "layer_stride": 8, "ms_per_call": statistics.mean(ts) * 1e3,
               "kernel_ms_per_call": kern_ms, "units_per_call": nb_seq * L * hkv}

    stages = algorithmic_bytes_per_unit(BUDGET + 1, D, QCL, hq // hkv, itemsize,
                                        args.variant != "none", args.global_score, moved)
    units = L * B * hkv
    bytes_step = sum(stages.values()) * units

    t = torch.tensor([dev_ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    ms_step = dev_ms / args.steps
    value = bytes_step * world / (ms_step * 1e-3) / 1e9
    e2e_val = bytes_step * world / (e2e_ms * 1e-3) / 1e9

    exact = None
    if rank == 0 and world == 1 and args.variant == "lightning" and not args.no_cpu_baseline:
        # the exact-similarity variant of the same step (two passes, the second timed)
        xcfg = make_cfg("exact", args.global_score)
        xcomp = Compressor(w.kv_cache, w.query_cache, w.score_cache, xcfg, layer_stride=min(chunk, 6),
                           impl=args.kernel_impl)
        xt = None
        for i in range(2):
            refresh()
            xcomp.time_record.clear()
            xcomp.compress_tables(seq_tables, seq_targets, seq_qids, seq_comp, timed=True)
            xt = {k: v * 1e3 for k, v in xcomp.time_record.items() if k.endswith("_sum")}
        n_tok = (BUDGET + 1) * BS
        flops = 2.0 * n_tok * n_tok * D * units
        red_ms = xt.get("redudancy_score_sum", 0.0)
        exact = {"ms_per_step": sum(xt.values()), "stage_ms": xt,
                 "similarity_tflops_dense_count": flops / (red_ms * 1e-3) / 1e12 if red_ms else None,
                 "similarity_tflops_issued": flops * (BUDGET + 2) / (2.0 * (BUDGET + 1)) / (red_ms * 1e-3) / 1e12
                 if red_ms else None}
        del xcomp

    # The other half of the metric: decode tokens/s at the 2048-token budget.  The compression
    # workload is released first; the decode step (full depth, tensor-parallel over the ranks
    # when there are several) then runs in this same process and process group.
    decode = serving = None
    if not args.no_decode:
        del w, comp, fresh, last_pages
        small = xcomp = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        from types import SimpleNamespace
        d_args = SimpleNamespace(**vars(args))
        d_args.batch, d_args.layers = 256, 36
        d_args.steps, d_args.warmup = max(args.steps, 10), max(args.warmup, 3)
        try:
            decode = decode_step_record(d_args, own_group=False)
        except Exception as e:   # the headline line must still come out
            decode = {"unavailable": f"{type(e).__name__}: {e}"[:300]} if rank == 0 else None
        # ... and the same through a whole serving loop (scheduler, prefill, graph decode,
        # compressions when they fall due, sampler), tensor-parallel under torchrun
        if not args.no_serving_loop:
            gc.collect()
            torch.cuda.empty_cache()
            try:
                serving = native_engine_record(d_args, own_group=False)
            except Exception as e:
                serving = {"unavailable": f"{type(e).__name__}: {e}"[:300]} if rank == 0 else None

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        # dominant kernel by the per-stage split (mean over the timed steps)
        top = max(stage_ms, key=stage_ms.get) if stage_ms else "attention_score_sum"
        stage_key = {"attention_score_sum": "window_score", "redudancy_score_sum": "redundancy",
                     "topk_mask_sum": "select", "compress_kv_sum": "compact",
                     "global_score_sum": "window_score"}.get(top, "window_score")
        nlaunch = (L + chunk - 1) // chunk
        top_ms = stage_ms.get(top, ms_step) / nlaunch
        # DRAM bytes per unit of each kernel from the committed ncu capture of a small case
        # (traffic grows in proportion to the units of a launch)
        ncu_bytes_per_unit = {}
        tf = ROOT / "profiles" / "compress_op_dram_bytes_per_unit.json"
        if tf.exists():
            ncu_bytes_per_unit = json.loads(tf.read_text()).get("bytes_per_unit", {})
        if stage_key == "redundancy" and args.variant == "exact":
            # algorithmic flops = the reference's dense N x N x D similarity product per unit; the
            # kernel skips the page tiles below the diagonal (S is symmetric), so it executes
            # NB*(NB+1)/2 of the NB*NB page tiles: both figures are reported.  The stage time also
            # holds the key-statistics pre-pass (one more read of K) and two small kernels.
            n_tok = (BUDGET + 1) * BS
            nbp = BUDGET + 1
            flops = 2.0 * n_tok * n_tok * D * units / nlaunch
            peak = peaks.get("bf16_tflops_sustained", 1400.0)
            achieved = flops / (top_ms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "redundancy_exact_tc (exact similarity stage)",
                        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "executed": achieved * (nbp + 1) / (2.0 * nbp),
                        "executed_note": "flops issued to the tensor pipe: upper-triangle page tiles only",
                        "peak_source": "measured sustained cuBLAS bf16 (MEASURED_PEAKS.json)" if peaks
                        else "fallback", "traffic": None}
        else:
            achieved = stages[stage_key] * units / nlaunch / (top_ms * 1e-3) / 1e9
            traffic = None
            if args.variant == "lightning" and args.kernel_impl != "simt" and stage_key in ncu_bytes_per_unit:
                traffic = ncu_bytes_per_unit[stage_key] * units / nlaunch
            roofline = {"bound": "hbm", "kernel": stage_key, "achieved": achieved, "peak": hbm_peak,
                        "unit": "GB/s", "frac": achieved / hbm_peak,
                        "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                        "traffic": traffic}
        per_stage = {}
        for sk, key in (("attention_score_sum", "window_score"), ("redudancy_score_sum", "redundancy"),
                        ("topk_mask_sum", "select"), ("compress_kv_sum", "compact")):
            if sk in stage_ms and stage_ms[sk] > 0 and stages.get(key):
                gbs = stages[key] * units / (stage_ms[sk] * 1e-3) / 1e9
                per_stage[key] = {"ms": stage_ms[sk], "gbs": gbs, "frac_of_hbm_peak": gbs / hbm_peak}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": "compression op, Qwen3-8B attention shapes, 9->8 pages, window 32, "
                            f"pool {POOL}, lambda {LAMBDA}, {args.variant} redundancy (config 2)",
                "sequences_per_gpu": B, "layers": L, "kv_heads_per_gpu": hkv, "q_heads_per_gpu": hq,
                "head_dim": D, "pages_per_seq": BUDGET + 1, "budget_pages": BUDGET,
                "units_per_gpu": units, "global_score": args.global_score,
                "kernel_impl": args.kernel_impl, "layer_chunk": chunk,
                "l2": "inputs (K/V pages of all sequences) are far larger than the 126 MB L2",
                "steady_state": "between steps, outside the per-step events, the appended page of every "
                                "sequence and the window queries are refilled with fresh N(0,1) data",
                "parallelism": f"kv-head sharding x{world}, no data-path collective",
            },
            "units_per_s": units * world / (ms_step * 1e-3),
            "algorithmic_bytes_per_unit": stages, "moved_rows_per_unit": moved,
            "moved_rows_per_unit_by_step": moved_steps,
            "stage_ms": stage_ms, "stage_ms_total": sum(stage_ms.values()), "per_stage": per_stage,
            "timed_region_s": region_s,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
            "roofline": roofline,
        }
        if decode is not None:
            line["decode"] = decode
        if serving is not None:
            line["serving_loop"] = serving
        if args.engine and world == 1:
            line["engine_decode"] = engine_decode_records()
        if eng is not None:
            line["e2e_engine_call_shape"] = eng
        if exact is not None:
            line["exact_variant"] = exact
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            gbs, secs, cu, sample = cpu_baseline_sample(args.variant, args.global_score, threads, keep_sample=True)
            line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"oracle.compress on {cu} units (L=2,B=16,Hkv=8,9 pages,bf16), {secs:.2f}s per pass"}
            line["parity"] = parity_on_sample(sample, cfg, args.kernel_impl, dev)
            ref_gpu = reference_gpu_stage_times(sample, dev)
            if ref_gpu is not None:
                line["reference_gpu"] = ref_gpu
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
