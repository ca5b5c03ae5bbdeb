"""Host control plane (native scheduler + page manager) against the reference's Python objects.

Golden: tests/golden/sched_traces.json holds, for every scenario of tests/sched_trace.py, the
running CRC of the unmodified reference's whole host state after every step (made by
tests/golden/make_sched_golden.py).  Where the reference itself can be imported (an installed
copy under baseline/_ref), two more seeds are compared live, step by step.  No GPU anywhere.
"""
import json
import random
import sys
import zlib
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
sys.path.insert(0, str(HERE))

import sched_trace as T  # noqa: E402
from zipage_b200.engine.scheduler import BlockManager, SamplingParams, Scheduler, Sequence, SequenceStatus  # noqa: E402

GOLDEN = json.loads((HERE / "golden" / "sched_traces.json").read_text())


def _fold(trace, every=25):
    raised = bool(trace) and trace[-1] == "raised"
    steps = trace[:-1] if raised else trace
    run, marks = 0, []
    for i, c in enumerate(steps):
        run = zlib.crc32(c.to_bytes(4, "little"), run)
        if (i + 1) % every == 0:
            marks.append(run)
    marks.append(run)
    return len(steps), marks, raised


@pytest.mark.parametrize("scenario", sorted(T.SCENARIOS))
def test_state_after_every_step_equals_the_reference(scenario):
    """The first 1200 steps of every scenario (the golden marks are running CRCs every 25 steps, so
    a prefix of the run can be compared); scenarios that end earlier are compared to their end."""
    want = GOLDEN["traces"][scenario]
    limit = 1200
    steps, marks, raised = _fold(T.run_trace(Scheduler, Sequence, SamplingParams, scenario, seed=0, max_steps=limit))
    whole = min(steps, want["steps"]) // 25
    first = next((i for i in range(whole) if marks[i] != want["marks"][i]), None)
    assert first is None, f"state differs from the reference's within steps {first * 25}..{first * 25 + 24}"
    if want["steps"] <= limit:
        assert (steps, raised, marks[-1]) == (want["steps"], want["raised"], want["marks"][-1])
    else:
        assert steps == limit and whole == limit // 25


def test_block_hash_known_answers():
    for case in GOLDEN["hashes"]:
        assert BlockManager.compute_hash(case["tokens"], case["prefix"]) == case["hash"]


def _reference_classes():
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "zipage" / "engine" / "scheduler.py").exists():
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, str(ref))
    try:
        from zipage.engine.scheduler import Scheduler as RS
        from zipage.engine.sequence import Sequence as RQ
        from zipage.sampling_params import SamplingParams as RP
    except Exception as e:  # its imports pull in torch extensions that may be absent
        pytest.skip(f"the reference does not import here: {e!r}")
    return RS, RQ, RP


@pytest.mark.parametrize("scenario", ["prefix_cache_tight", "hybrid_tight_pool_preempts", "async_compress",
                                      "eos_and_late_arrivals"])
def test_live_against_the_installed_reference(scenario):
    RS, RQ, RP = _reference_classes()
    for seed in (1,):
        want = T.run_trace(RS, RQ, RP, scenario, seed=seed, max_steps=1200)
        got = T.run_trace(Scheduler, Sequence, SamplingParams, scenario, seed=seed, max_steps=1200)
        first = next((i for i, (a, b) in enumerate(zip(want, got)) if a != b), None)
        assert first is None and len(want) == len(got), (scenario, seed, first)


def _running_scheduler(n=24, seed=3, **over):
    cfg = T.make_config(**over)
    rng = random.Random(seed)
    s = Scheduler(cfg)
    seqs = [Sequence([rng.randrange(5000) for _ in range(rng.randint(40, 900))],
                     SamplingParams(0.6, rng.randint(300, 1200), True)) for _ in range(n)]
    for q in seqs:
        s.add(q)
    return s, seqs, rng


def test_array_calls_agree_with_the_sequence_attributes():
    s, seqs, rng = _running_scheduler()
    compressions = 0
    for step in range(1400):
        handles, is_prefill = s.schedule_batch()
        if is_prefill:
            s.mark_prefilled(handles)
        else:
            due = [h for h in handles.tolist() if s._seqs[h].require_compress]
            assert s.compress_due(handles).tolist() == due
            if due:
                compressions += len(due)
                c = s.compress_inputs(due)
                for i, h in enumerate(due):
                    q = s._seqs[h]
                    t = q.block_table
                    want = t[:-1] + [-t[-1] - 2] + [-1] * (c["tables"].shape[1] - len(t))
                    assert c["tables"][i].tolist() == want
                    assert c["targets"][i].tolist() == q.new_block_table
                    assert c["query_ids"][i] == q.query_id and bool(c["compressed"][i]) == q.compressed
                s.postprocess_batch(due)
            assert s.temperatures(handles).tolist() == [np.float32(0.6)] * len(handles)
            d = s.decode_inputs(handles, table_width=6)
            for i, h in enumerate(handles.tolist()):
                q = s._seqs[h]
                assert d["input_ids"][i] == q.last_token and d["num_tokens"][i] == len(q)
                assert d["query_ids"][i] == q.query_id
                t = q.block_table
                assert d["block_tables"][i].tolist() == t + [-1] * (6 - len(t))
                # what the device-side bookkeeping derives from these (model_runner.py:633-675)
                assert (len(t) - 1) * 256 + q.last_block_num_tokens == len(q) or q.compressed
        done = s.postprocess_batch(handles, np.asarray([rng.randrange(5000) for _ in handles], np.int32))
        assert sorted(done.tolist()) == sorted(h for h in handles.tolist() if s._seqs[h].status == SequenceStatus.FINISHED)
        assert all(s._seqs[h].is_finished for h in done.tolist())
        if s.is_finished():
            break
    assert s.is_finished() and compressions > 10
    assert all(q.status == SequenceStatus.FINISHED and q.block_table == [] for q in seqs)
    c = s.counts()
    assert c[2] == 260 and c[3] == 0 and c[4] == 64      # every block and query slot came back


def test_postprocess_consumes_the_callers_token_list_like_the_reference():
    s, seqs, _ = _running_scheduler(n=4)
    scheduled, is_prefill = s.schedule()
    for q in scheduled:
        q.num_cached_tokens = len(q)
    tokens = [11, 12, 13, 14, 99]
    s.postprocess(scheduled, tokens)
    assert tokens == [99] and [q.last_token for q in scheduled] == [11, 12, 13, 14]
    assert scheduled[0].completion_token_ids == [11] and scheduled[0].num_completion_tokens == 1


def test_errors_are_reported_not_swallowed():
    from zipage_b200 import _hostlib as H
    s, seqs, _ = _running_scheduler(n=2)
    with pytest.raises(H.SchedulerError):
        s.postprocess_batch(np.asarray([57], np.int32), np.asarray([1], np.int32))   # unknown handle
    long = Sequence(list(range(600)), SamplingParams(0.6, 10, True))     # three blocks
    s.add(long)
    s.schedule_batch()
    with pytest.raises(H.SchedulerError):
        s.decode_inputs(np.asarray([long._h], np.int32), table_width=2)   # table wider than the output
    lib = H.load()
    assert lib.zp_sched_schedule(s._obj, None, 0, None) == -1 and b"null" in lib.zp_sched_last_error()
    assert lib.zp_sched_create(None) is None
    with pytest.raises(AssertionError):      # the reference asserts here too (scheduler.py:137)
        q = seqs[0]
        while not q.compressed:
            hs, pf = s.schedule_batch()
            if pf:
                s.mark_prefilled(hs)
            due = [h for h in hs.tolist() if s._seqs[h].require_compress]
            s.postprocess_batch(due)
            s.postprocess_batch(hs, np.zeros(len(hs), np.int32))
        s.preempt(q)


def _replica_main(rank, world, port, tmp):
    """Tensor-parallel ranks each run their own scheduler replica: the sampled tokens are the same
    on every rank (the sharded sampler leaves every rank with the winners), so the replicas take the
    same decisions and no per-step message from rank 0 is needed (the reference pickles the
    scheduled sequences into shared memory every step, model_runner.py:151-203)."""
    import os
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    s, seqs, _ = _running_scheduler(n=16, seed=5, num_kvcache_blocks=60, enable_prefix_cache=True)
    ok, steps = True, 0
    while not s.is_finished() and steps < 1500:
        handles, is_prefill = s.schedule_batch()
        if is_prefill:
            s.mark_prefilled(handles)
        else:
            s.postprocess_batch([h for h in handles.tolist() if s._seqs[h].require_compress])
        # every rank draws candidates for its own shard of the vocabulary; the largest key wins
        g = torch.Generator().manual_seed(steps * world + rank)
        keys = torch.randint(0, 1 << 20, (len(handles),), generator=g) * 4096 + torch.randint(0, 1024, (len(handles),), generator=g) * world + rank
        dist.all_reduce(keys, op=dist.ReduceOp.MAX)
        tokens = (keys % 4096).to(torch.int32).numpy()
        d = s.decode_inputs(handles, table_width=5)
        state = torch.tensor([zlib.crc32(handles.tobytes() + tokens.tobytes() + d["block_tables"].tobytes()
                                         + d["num_tokens"].tobytes() + d["query_ids"].tobytes())], dtype=torch.int64)
        every = [torch.zeros_like(state) for _ in range(world)]
        dist.all_gather(every, state)
        ok = ok and all(int(e) == int(state) for e in every)
        s.postprocess_batch(handles, tokens)
        steps += 1
    if rank == 0:
        Path(tmp).write_text("ok" if ok and s.is_finished() else f"diverged or unfinished after {steps} steps")
    dist.barrier()
    dist.destroy_process_group()


def test_scheduler_replicas_on_two_ranks_stay_in_step_gloo(tmp_path):
    import os
    import torch.multiprocessing as mp
    port = 31500 + os.getpid() % 2000
    res = tmp_path / "result.txt"
    mp.spawn(_replica_main, args=(2, port, str(res)), nprocs=2, join=True)
    assert res.read_text() == "ok"


def _prepare_prefill_lists(seqs, block_size, qcl):
    """The list building of ModelRunner.prepare_prefill / get_query_slot_mapping
    (zipage/engine/model_runner.py:319-339, :352-388), restated on the reference's attribute names."""
    ids, pos, slots, triples, cu_q, cu_k = [], [], [], [], [0], [0]
    for s in seqs:
        seqlen, cached = len(s), s.num_cached_tokens
        toks = s.token_ids
        ids += toks[cached:]
        pos += list(range(cached, seqlen))
        lq = seqlen - cached
        if s.query_id != -1:
            nb = (lq + block_size - 1) // block_size
            if nb and lq - (nb - 1) * block_size > block_size - qcl:
                start = nb * block_size - qcl
                triples += [(cu_q[-1] + p, s.query_id, i) for i, p in enumerate(range(start, lq))]
        cu_q.append(cu_q[-1] + lq)
        cu_k.append(cu_k[-1] + seqlen)
        table = s.block_table
        for i in range(cached // block_size, s.num_blocks):
            start = table[i] * block_size
            slots += list(range(start, start + (block_size if i != s.num_blocks - 1 else s.last_block_num_tokens)))
    return ids, pos, slots, triples, cu_q, cu_k


@pytest.mark.parametrize("prefix_cache", [False, True])
def test_prefill_inputs_equal_the_reference_list_building(prefix_cache):
    rng = random.Random(21)
    cfg = T.make_config(enable_prefix_cache=prefix_cache, num_kvcache_blocks=200, max_num_seqs=16,
                        max_num_batched_tokens=6000)
    s = Scheduler(cfg)
    shared = [rng.randrange(5000) for _ in range(512)]
    lengths = [40, 225, 250, 256, 257, 480, 500, 512, 700, 760, 1000, 1023, 1300]   # around the window limits
    for n in lengths * 2:
        toks = [rng.randrange(5000) for _ in range(n)]
        if prefix_cache and n > 600:
            toks[:512] = shared
        s.add(Sequence(toks, SamplingParams(0.6, 4, True)))
    seen_cached = seen_rows = batches = 0
    while True:
        seqs, is_prefill = s.schedule()
        if not is_prefill:
            break
        batches += 1
        seen_cached += sum(q.num_cached_tokens > 0 for q in seqs)
        want = _prepare_prefill_lists(seqs, 256, 32)
        got = s.prefill_inputs(s._handles_of(seqs))
        assert got["input_ids"].tolist() == want[0] and got["positions"].tolist() == want[1]
        assert got["slot_mapping"].tolist() == want[2]
        assert [tuple(r) for r in got["query_triples"].tolist()] == want[3]
        assert got["cu_seqlens_q"].tolist() == want[4] and got["cu_seqlens_k"].tolist() == want[5]
        assert got["max_seqlen_q"] == max(b - a for a, b in zip(want[4], want[4][1:]))
        assert got["max_seqlen_k"] == max(len(q) for q in seqs)
        assert (got["block_tables"] is not None) == (want[5][-1] > want[4][-1])
        if got["block_tables"] is not None:
            for row, q in zip(got["block_tables"].tolist(), seqs):
                assert [b for b in row if b >= 0] == q.block_table
        assert all(q.num_cached_tokens == len(q) for q in seqs)      # marked prefilled
        seen_rows += len(want[3])
        s.postprocess(seqs, [1] * len(seqs))
    assert batches >= 2 and seen_rows > 0 and (seen_cached > 0) == prefix_cache


def test_calls_from_a_second_thread_are_serialised():
    """The reference engine's asynchronous mode touches the scheduler from its compression thread
    (zipage_engine.py:88-96).  A second thread reads queues, counters and sequence state as fast as
    it can while the main thread runs a whole scenario: the run must end in the golden state."""
    import threading
    stop = threading.Event()
    seen = []
    holder = {}

    class Watched(Scheduler):
        def __init__(self, config):
            super().__init__(config)
            holder["s"] = self

    def reader():
        n = 0
        while not stop.is_set():
            s = holder.get("s")
            if s is None:
                continue
            c = s.counts()
            s._queue(1), s._queue(2), s._queue(3)
            for q in list(s._seqs)[:8]:
                q._cache.clear()
                _ = (q.num_tokens, q.block_table)
            assert c[2] + c[3] == s._cfg.num_blocks        # a consistent snapshot: free + used = all
            n += 1
        seen.append(n)

    t = threading.Thread(target=reader)
    t.start()
    try:
        steps, marks, raised = _fold(T.run_trace(Watched, Sequence, SamplingParams, "prefix_cache", seed=0,
                                                 max_steps=3000))
    finally:
        stop.set()
        t.join()
    want = GOLDEN["traces"]["prefix_cache"]
    assert marks == want["marks"] and steps == want["steps"] and seen and seen[0] > 100


def test_random_configurations_live_against_the_installed_reference():
    """Differential run over random scheduler configurations and request streams (block pool,
    budget, prefix cache, hybrid engine, slots, batch limits, window length, EOS, shared prefixes,
    asynchronous compression, late arrivals): every step's state equal to the reference's."""
    RS, RQ, RP = _reference_classes()
    rng = random.Random(2024)
    try:
        for it in range(8):
            over = dict(num_kvcache_blocks=rng.choice([24, 40, 64, 100, 200]),
                        max_cache_blocks_per_seq=rng.choice([1, 2, 3, 4]),
                        enable_prefix_cache=rng.random() < 0.5, enable_hybrid_engine=rng.random() < 0.4,
                        max_concurrency=rng.choice([2, 4, 8, 32]), max_num_seqs=rng.choice([4, 8, 16, 64]),
                        max_num_batched_tokens=rng.choice([1200, 3000, 16384]),
                        query_cache_len=rng.choice([16, 32, 64]), eos=rng.choice([-1, 3]))
            wl = dict(n=rng.choice([6, 12, 24]), prompt=(rng.choice([10, 100, 250]), rng.choice([300, 600, 1100])),
                      max_tokens=(rng.choice([5, 100]), rng.choice([300, 700])), ignore_eos=rng.random() < 0.6,
                      vocab=rng.choice([12, 5000]))
            if rng.random() < 0.5:
                wl["shared_prefix"] = (256, 512)
            if rng.random() < 0.3:
                wl["async_delay"] = rng.choice([1, 2, 5])
            if rng.random() < 0.3:
                wl["arrive_every"] = rng.choice([3, 20])
            T.SCENARIOS["random"] = (over, wl)
            want = T.run_trace(RS, RQ, RP, "random", seed=it, max_steps=1200)
            got = T.run_trace(Scheduler, Sequence, SamplingParams, "random", seed=it, max_steps=1200)
            first = next((i for i, (a, b) in enumerate(zip(want, got)) if a != b), None)
            assert first is None and len(want) == len(got), (it, over, wl, first)
    finally:
        T.SCENARIOS.pop("random", None)


def test_page_accounting_invariants_hold_at_every_step():
    """Independent of the reference: at every step of a run with a small page pool, prefix sharing
    and preemptions, (a) free + used = all pages, (b) a page's reference count equals the number of
    live tables (block_table, or new_block_table / block_to_release of a pending compression) that
    hold it, (c) free pages are held by no table, (d) no table is longer than the budget + 1 pages
    after its first compression, (e) query slots are unique among running sequences."""
    from collections import Counter
    rng = random.Random(77)
    cfg = T.make_config(enable_prefix_cache=True, num_kvcache_blocks=48, max_concurrency=12, enable_hybrid_engine=True)
    s = Scheduler(cfg)
    shared = [rng.randrange(5000) for _ in range(512)]
    seqs = []
    for i in range(20):
        toks = [rng.randrange(5000) for _ in range(rng.randint(300, 900))]
        if i % 2 and len(toks) > 520:
            toks[:512] = shared
        seqs.append(Sequence(toks, SamplingParams(0.6, rng.randint(200, 800), True)))
        s.add(seqs[-1])
    steps = preempted = 0
    while not s.is_finished() and steps < 4000:
        scheduled, is_prefill = s.schedule()
        if is_prefill:
            s.mark_prefilled(s._handles_of(scheduled))
        else:
            due = [q for q in scheduled if q.require_compress]
            if due and steps % 3 == 0:            # otherwise the compression stays pending for a while
                s.postprocess(due)
            scheduled = [q for q in scheduled if not q.require_compress]
        s.postprocess(scheduled, [rng.randrange(5000) for _ in scheduled])
        steps += 1
        c = s.counts()
        assert c[2] + c[3] == 48
        held = Counter()
        for q in seqs:
            pending = q.require_compress
            pages = set(q.block_table) | (set(q.new_block_table) | set(q.block_to_release) if pending else set())
            held.update(pages)
            if q.compressed and not pending:
                assert len(q.block_table) <= cfg.max_cache_blocks_per_seq + 1
        free = set(s.block_manager.free_block_ids)
        assert len(free) == c[2] and not (free & set(held))
        for page, n in held.items():
            assert s.block_manager.block_state(page)[0] == n, (steps, page, n)
        slots = [q.query_id for q in s.running if q.query_id != -1]
        assert len(slots) == len(set(slots)) and len(slots) + len(s.free_query_ids) == 12
        preempted += sum(1 for q in s.waiting if q.num_completion_tokens > 0)
    assert s.is_finished() and preempted > 0
