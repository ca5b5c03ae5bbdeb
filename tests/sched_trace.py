"""Drives a Scheduler implementation (the reference's or zipage_b200's) through a seeded request
stream the way LLMEngine.step / async_step do (zipage/engine/zipage_engine.py:99-186), without a
model: tokens come from a seeded generator.  After every step it records a checksum of the whole
host state, so two implementations can be compared step by step.
"""
from __future__ import annotations

import random
import types
import zlib

SCENARIOS = {
    # name: (config overrides, workload)
    "plain": (dict(), dict(n=40, prompt=(60, 900), max_tokens=(200, 1400))),
    "tight_pool_suspends": (dict(num_kvcache_blocks=70), dict(n=40, prompt=(60, 900), max_tokens=(200, 1400))),
    "prefix_cache": (dict(enable_prefix_cache=True, num_kvcache_blocks=120),
                     dict(n=40, prompt=(300, 1100), max_tokens=(100, 900), shared_prefix=(256, 512, 768))),
    "prefix_cache_tight": (dict(enable_prefix_cache=True, num_kvcache_blocks=60),
                           dict(n=36, prompt=(300, 900), max_tokens=(100, 900), shared_prefix=(256, 512))),
    "hybrid_few_query_slots": (dict(enable_hybrid_engine=True, max_concurrency=6),
                               dict(n=30, prompt=(60, 700), max_tokens=(300, 1300))),
    "hybrid_tight_pool_preempts": (dict(enable_hybrid_engine=True, max_concurrency=5, num_kvcache_blocks=40),
                                   dict(n=30, prompt=(60, 700), max_tokens=(300, 1300))),
    "async_compress": (dict(), dict(n=32, prompt=(60, 900), max_tokens=(300, 1400), async_delay=3)),
    "eos_and_late_arrivals": (dict(eos=7), dict(n=48, prompt=(20, 600), max_tokens=(50, 1200), ignore_eos=False,
                                                 vocab=40, arrive_every=25)),
    "small_batches": (dict(max_num_seqs=8, max_num_batched_tokens=1500),
                      dict(n=30, prompt=(60, 700), max_tokens=(100, 900))),
    "long_prompts_first_compress": (dict(num_kvcache_blocks=400),
                                    dict(n=12, prompt=(1500, 4000), max_tokens=(300, 700))),
}


def make_config(**over):
    cfg = dict(max_num_seqs=64, max_num_batched_tokens=16384, eos=-1, num_kvcache_blocks=260,
               kvcache_block_size=256, max_cache_blocks_per_seq=3, enable_prefix_cache=False,
               max_concurrency=64, enable_hybrid_engine=False, query_cache_len=32)
    cfg.update(over)
    return types.SimpleNamespace(**cfg)


def _state_checksum(sched, seqs, index_of, scheduled, is_prefill):
    parts = [int(is_prefill), [index_of[id(s)] for s in scheduled],
             [index_of[id(s)] for s in sched.waiting], [index_of[id(s)] for s in sched.running],
             list(sched.block_manager.free_block_ids), list(sched.free_query_ids)]
    for s in seqs:
        parts.append((len(s), s.num_cached_tokens, s.query_id, list(s.block_table), list(s.new_block_table),
                      list(s.block_to_release), bool(s.require_compress), bool(s.compressed),
                      bool(s.prefilled), s.status.name, s.last_token))
    return zlib.crc32(repr(parts).encode())


def run_trace(Scheduler, Sequence, SamplingParams, scenario, seed=0, max_steps=6000, detail=False):
    """-> list of per-step checksums (ends with "raised" if the scheduler raised an exception).  With `detail`, a list of (checksum, scheduled indices, is_prefill) instead."""
    over, wl = SCENARIOS[scenario]
    cfg = make_config(**over)
    rng = random.Random(seed * 1000003 + zlib.crc32(scenario.encode()))
    vocab = wl.get("vocab", 5000)
    prefixes = {p: [rng.randrange(vocab) for _ in range(p)] for p in wl.get("shared_prefix", ())}
    pending = []
    for _ in range(wl["n"]):
        n = rng.randint(*wl["prompt"])
        toks = [rng.randrange(vocab) for _ in range(n)]
        if prefixes and rng.random() < 0.7:
            p = rng.choice(sorted(prefixes))
            if p < n:
                toks[:p] = prefixes[p]
        sp = SamplingParams(temperature=0.6, max_tokens=rng.randint(*wl["max_tokens"]),
                            ignore_eos=wl.get("ignore_eos", True))
        pending.append((toks, sp))
    sched = Scheduler(cfg)
    seqs, index_of = [], {}

    def admit(k):
        for _ in range(k):
            if pending:
                toks, sp = pending.pop(0)
                s = Sequence(toks, sp)
                index_of[id(s)] = len(seqs)
                seqs.append(s)
                sched.add(s)

    every = wl.get("arrive_every", 0)
    admit(wl["n"] if not every else 8)
    delay = wl.get("async_delay", 0)
    in_flight = []          # (due step, sequences whose compression "runs")
    trace = []
    step = 0
    try:
        while (not sched.is_finished() or pending) and step < max_steps:
            if every and step % every == 0:
                admit(4)
            done = [c for c in in_flight if c[0] <= step]
            for c in done:                      # an asynchronous compression finishes
                in_flight.remove(c)
                sched.postprocess(c[1])
            scheduled, is_prefill = sched.schedule()
            run = scheduled
            if is_prefill:
                for s in scheduled:
                    s.num_cached_tokens = len(s)      # model_runner.py:387
            else:
                due = [s for s in scheduled if s.require_compress]
                if delay:
                    run = [s for s in scheduled if not s.require_compress]
                    busy = {id(s) for c in in_flight for s in c[1]}
                    fresh = [s for s in due if id(s) not in busy]
                    if fresh and not in_flight:
                        in_flight.append((step + delay, fresh))
                elif due:
                    sched.postprocess(due)
            tokens = [rng.randrange(vocab) for _ in run]
            sched.postprocess(run, tokens)
            c = _state_checksum(sched, seqs, index_of, scheduled, is_prefill)
            trace.append((c, [index_of[id(s)] for s in scheduled], is_prefill) if detail else c)
            step += 1
    except (AssertionError, IndexError, ValueError) as e:
        trace.append("raised")
    return trace
