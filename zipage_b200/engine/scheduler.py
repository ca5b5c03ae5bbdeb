"""Host control plane: the reference's Scheduler / BlockManager / Sequence interface over the
native scheduler of include/zipage_b200_host.h.

Two ways in:

* the reference's own calls — `Scheduler(config)`, `add(seq)`, `schedule() -> (seqs, is_prefill)`,
  `postprocess(seqs, token_ids)`, `preempt(seq)`, `is_finished()`, `block_manager.block_occupancy`,
  and `Sequence` objects with the reference's attributes (zipage/engine/scheduler.py:10-167,
  block_manager.py:26-210, sequence.py:14-119), so `LLMEngine.step` (zipage_engine.py:99-135) and
  `ModelRunner` read them unchanged.  State lives in the native object; a `Sequence` is a handle
  whose attributes are read from it on access;
* the array calls a native runner uses, with no per-sequence Python at all: `schedule_batch()`,
  `postprocess_batch()`, `mark_prefilled()`, `decode_inputs()` (what
  `ModelRunner.prepare_decode`, model_runner.py:633-675, builds element by element) and
  `compress_inputs()` (model_runner.py:424-463).
"""
from __future__ import annotations

import ctypes as C
import time
from contextlib import contextmanager
from dataclasses import dataclass
from enum import Enum
from itertools import count

import numpy as np

from .. import _hostlib as H


@dataclass
class SamplingParams:
    """zipage/sampling_params.py:4-11."""
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False

    def __post_init__(self):
        assert self.temperature > 1e-10, "greedy sampling is not permitted"


class SequenceStatus(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class Sequence:
    """A request.  Before `Scheduler.add` it only holds the prompt; afterwards every attribute is
    read from the native scheduler (field names as in zipage/engine/sequence.py)."""
    block_size = 256
    counter = count()

    def __init__(self, token_ids, sampling_params=SamplingParams()):
        self.request_id = next(Sequence.counter)
        self._prompt = [int(t) for t in token_ids]
        self._params = sampling_params
        self.temperature = sampling_params.temperature     # never change: kept on the handle
        self.max_tokens = sampling_params.max_tokens
        self.ignore_eos = sampling_params.ignore_eos
        self._sched = None
        self._h = -1
        self._cache = {}
        self._finished = False

    # -- native state -------------------------------------------------------------------------
    # Reads are cached until the scheduler's next mutating call (its epoch), so a runner that
    # looks at a few attributes of every scheduled sequence pays one C call per sequence and list.
    def _cached(self, key, fetch):
        cache, epoch = self.__dict__["_cache"], self._sched._epoch
        hit = cache.get(key)
        if hit is None or hit[0] != epoch:
            hit = cache[key] = (epoch, fetch())
        return hit[1]

    def _info(self):
        def fetch():
            out = (C.c_int32 * 16)()
            H.check(self._sched._lib.zp_sched_seq_info(self._sched._obj, self._h, out), "seq_info")
            return list(out)
        return self._cached("info", fetch)

    def _list(self, which):
        def fetch():
            lib, obj = self._sched._lib, self._sched._obj
            n = lib.zp_sched_seq_list(obj, self._h, which, None, 0)
            out = np.empty(max(n, 1), dtype=np.int32)
            H.check(lib.zp_sched_seq_list(obj, self._h, which, _ptr(out), n), "seq_list")
            return out[:n].tolist()
        return list(self._cached(which, fetch))

    def _times(self):
        t, temp = (C.c_double * 2)(), C.c_float()
        H.check(self._sched._lib.zp_sched_seq_times(self._sched._obj, self._h, t, C.byref(temp)), "seq_times")
        return t[0], t[1], temp.value

    _FIELD = {"num_tokens": 1, "num_prompt_tokens": 2, "num_cached_tokens": 3, "last_token": 4, "query_id": 5}
    _FLAG = {"require_compress": 6, "compressed": 7, "prefilled": 8}

    def __getattr__(self, name):   # only reached for names that are not plain attributes
        if name in Sequence._FIELD or name in Sequence._FLAG:
            if self.__dict__.get("_sched") is None:   # not added yet: the constructor's values
                p = self.__dict__["_prompt"]
                before = {"num_tokens": len(p), "num_prompt_tokens": len(p), "num_cached_tokens": 0,
                          "last_token": p[-1], "query_id": -1,
                          "require_compress": False, "compressed": False, "prefilled": False}
                return before[name]
            info = self._info()
            return info[Sequence._FIELD[name]] if name in Sequence._FIELD else bool(info[Sequence._FLAG[name]])
        raise AttributeError(name)

    @property
    def status(self):
        return SequenceStatus.WAITING if self._sched is None else SequenceStatus(self._info()[0])

    @property
    def token_ids(self):
        return list(self._prompt) if self._sched is None else self._list(3)

    @property
    def block_table(self):
        return [] if self._sched is None else self._list(0)

    @property
    def new_block_table(self):
        return [] if self._sched is None else self._list(1)

    @property
    def block_to_release(self):
        return [] if self._sched is None else self._list(2)

    @property
    def time_prefilled(self):
        return 0 if self._sched is None else self._times()[0]

    @property
    def time_finished(self):
        return 0 if self._sched is None else self._times()[1]

    def set_num_cached_tokens(self, value):
        """The one field the model runner writes (model_runner.py:387)."""
        with self._sched._mutating():
            H.check(self._sched._lib.zp_sched_seq_set_num_cached(self._sched._obj, self._h, int(value)), "set_num_cached")

    def __setattr__(self, name, value):
        if name == "num_cached_tokens":
            self.set_num_cached_tokens(value)
        else:
            object.__setattr__(self, name, value)

    # -- derived, as in the reference -----------------------------------------------------------
    def __len__(self):
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def is_finished(self):
        # a sequence finishes only inside Scheduler.postprocess, which flags its handle
        return self._finished

    @property
    def num_completion_tokens(self):
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self):
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def completion_token_ids(self):
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_blocks(self):
        return (self.num_tokens + self.block_size - 1) // self.block_size

    @property
    def last_block_num_tokens(self):
        return self.num_tokens - (self.num_blocks - 1) * self.block_size

    @property
    def num_cached_blocks(self):
        return self.num_cached_tokens // self.block_size

    def block(self, i):
        assert 0 <= i < self.num_blocks
        return self.token_ids[i * self.block_size: (i + 1) * self.block_size]

    def last_n_completion_tokens(self, n):
        toks = self.token_ids
        return toks[-n:] if n >= self.num_completion_tokens else toks[self.num_prompt_tokens:]


class BlockManager:
    """Read-only view of the native page manager with the reference's attribute names
    (zipage/engine/block_manager.py:26-57); the scheduler drives it."""

    def __init__(self, sched):
        self._s = sched
        self.block_size = sched.block_size
        self.max_blocks_per_seq = sched._cfg.max_blocks_per_seq
        self.enable_prefix_cache = bool(sched._cfg.enable_prefix_cache)

    @classmethod
    def compute_hash(cls, token_ids, prefix=-1):
        tok = np.ascontiguousarray(token_ids, dtype=np.int32)
        return int(H.load().zp_sched_hash_tokens(_ptr(tok), len(tok), int(prefix != -1), max(int(prefix), 0)))

    @property
    def free_block_ids(self):
        return self._s._queue(2)

    @property
    def num_free_blocks(self):
        return self._s.counts()[2]

    @property
    def num_used_blocks(self):
        return self._s.counts()[3]

    @property
    def block_occupancy(self):
        c = self._s.counts()
        return c[3] / (c[3] + c[2])

    def block_state(self, block_id):
        """(ref_count, hash or -1) of one block (block_manager.py:9-23)."""
        out, h = (C.c_int32 * 2)(), C.c_uint64()
        H.check(self._s._lib.zp_sched_block_info(self._s._obj, int(block_id), out, C.byref(h)), "block_info")
        return out[0], (int(h.value) if out[1] else -1)


class Scheduler:
    """zipage/engine/scheduler.py:10-167 over the native object."""

    def __init__(self, config):
        self._lib = H.load()
        self._cfg = H.SchedConfig(
            num_blocks=config.num_kvcache_blocks, block_size=config.kvcache_block_size,
            max_blocks_per_seq=config.max_cache_blocks_per_seq + 1,
            enable_prefix_cache=int(bool(config.enable_prefix_cache)), max_num_seqs=config.max_num_seqs,
            max_num_batched_tokens=config.max_num_batched_tokens,
            eos=-1 if config.eos is None else config.eos, max_concurrency=config.max_concurrency,
            enable_hybrid_engine=int(bool(config.enable_hybrid_engine)), query_cache_len=config.query_cache_len)
        self._obj = self._lib.zp_sched_create(C.byref(self._cfg))
        if not self._obj:
            raise H.SchedulerError(self._lib.zp_sched_last_error().decode())
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.enable_prefix_cache = bool(config.enable_prefix_cache)
        self.enable_hybrid_engine = bool(config.enable_hybrid_engine)
        self.query_cache_len = config.query_cache_len
        self.block_size = config.kvcache_block_size
        self.block_manager = BlockManager(self)
        self._seqs = []                                   # handle -> Sequence
        self._epoch = 0                                   # bumped by every call that changes state
        self._handles = np.empty(config.max_num_seqs, dtype=np.int32)

    def __del__(self):
        obj, self._obj = getattr(self, "_obj", None), None
        if obj:
            self._lib.zp_sched_destroy(obj)

    # -- helpers --------------------------------------------------------------------------------
    @contextmanager
    def _mutating(self):
        """Cached reads of the handles are keyed by this epoch.  It moves before AND after a call
        that changes native state: a read that another thread starts in between stores its (old)
        result under an epoch that is already over when the call returns."""
        self._epoch += 1
        try:
            yield
        finally:
            self._epoch += 1

    def counts(self):
        out = (C.c_int32 * 8)()
        H.check(self._lib.zp_sched_counts(self._obj, out), "counts")
        return list(out)

    def _queue(self, which):
        n = self._lib.zp_sched_queue(self._obj, which, None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        H.check(self._lib.zp_sched_queue(self._obj, which, _ptr(out), n), "queue")
        return out[:n].tolist()

    @property
    def waiting(self):
        return [self._seqs[h] for h in self._queue(0)]

    @property
    def running(self):
        return [self._seqs[h] for h in self._queue(1)]

    @property
    def free_query_ids(self):
        return self._queue(3)

    @property
    def used_query_ids(self):
        free = set(self._queue(3))
        return {q for q in range(self._cfg.max_concurrency) if q not in free}

    @staticmethod
    def _handles_of(seqs):
        return np.fromiter((s._h for s in seqs), dtype=np.int32, count=len(seqs))

    # -- the reference's calls ------------------------------------------------------------------
    def is_finished(self):
        return bool(self.counts()[7])

    def add(self, seq: Sequence):
        tok = np.ascontiguousarray(seq._prompt, dtype=np.int32)
        p = seq._params
        h = H.check(self._lib.zp_sched_add(self._obj, _ptr(tok), len(tok), float(p.temperature),
                                           int(p.max_tokens), int(bool(p.ignore_eos))), "add")
        assert h == len(self._seqs)
        self._epoch += 1
        self._seqs.append(seq)
        object.__setattr__(seq, "_h", h)
        object.__setattr__(seq, "_sched", self)
        object.__setattr__(seq, "_prompt", None)     # the tokens live in the native object from here on

    def schedule(self):
        handles, is_prefill = self.schedule_batch()
        seqs = [self._seqs[h] for h in handles.tolist()]
        # the engine looks at every scheduled sequence right away (zipage_engine.py:101-105): fetch
        # their scalar state in one call instead of one call per sequence
        info = np.empty((max(len(seqs), 1), 16), dtype=np.int32)
        epoch = self._epoch       # taken before the read: a change meanwhile makes these entries stale
        H.check(self._lib.zp_sched_seq_info_batch(self._obj, _ptr(handles), len(seqs), _ptr(info)), "seq_info_batch")
        for q, row in zip(seqs, info.tolist()):
            q._cache["info"] = (epoch, row)
        return seqs, is_prefill

    def postprocess(self, seqs, token_ids=None):
        n = len(seqs)
        toks = None
        if token_ids is not None:
            toks = np.ascontiguousarray(token_ids[:n], dtype=np.int32)
            del token_ids[:n]          # the reference pops one token per sequence off the caller's list
        self.postprocess_batch(self._handles_of(seqs), toks)

    def preempt(self, seq: Sequence):
        with self._mutating():
            H.check(self._lib.zp_sched_preempt(self._obj, seq._h), "preempt")

    # -- array calls ----------------------------------------------------------------------------
    def schedule_batch(self):
        """-> (handles of the scheduled sequences as an int32 array, is_prefill)."""
        flag = C.c_int32(0)
        with self._mutating():
            n = H.check(self._lib.zp_sched_schedule(self._obj, _ptr(self._handles), len(self._handles),
                                                    C.byref(flag)), "schedule")
            return self._handles[:n].copy(), bool(flag.value)

    def postprocess_batch(self, handles, token_ids=None, now=None):
        """-> the handles that finished in this call (int32 array)."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        toks = None if token_ids is None else np.ascontiguousarray(token_ids, dtype=np.int32)
        if toks is not None and len(toks) != len(handles):
            raise ValueError("one token per sequence")
        done = np.empty(max(len(handles), 1), dtype=np.int32)
        with self._mutating():
            n = H.check(self._lib.zp_sched_postprocess(self._obj, _ptr(handles), len(handles),
                                                       None if toks is None else _ptr(toks),
                                                       time.time() if now is None else now, _ptr(done)), "postprocess")
        for h in done[:n].tolist():
            object.__setattr__(self._seqs[h], "_finished", True)
        return done[:n]

    def mark_prefilled(self, handles):
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        with self._mutating():
            H.check(self._lib.zp_sched_mark_prefilled(self._obj, _ptr(handles), len(handles)), "mark_prefilled")

    def decode_inputs(self, handles, table_width=None, out=None):
        """One decode step's host arrays: dict(input_ids, num_tokens, query_ids, block_tables
        [n, table_width], widest).  `out` may hold preallocated int32 arrays of those names (for
        example numpy views of pinned buffers)."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        n = len(handles)
        w = table_width or self._cfg.max_blocks_per_seq + 1
        out = out or {"input_ids": np.empty(n, np.int32), "num_tokens": np.empty(n, np.int32),
                      "query_ids": np.empty(n, np.int32), "block_tables": np.empty((n, w), np.int32)}
        widest = H.check(self._lib.zp_sched_decode_inputs(
            self._obj, _ptr(handles), n, _ptr(out["input_ids"]), _ptr(out["num_tokens"]), _ptr(out["query_ids"]),
            _ptr(out["block_tables"]), w), "decode_inputs")
        out["widest"] = widest
        return out

    def temperatures(self, handles, out=None):
        """float32 array of the sequences' sampling temperatures (`out`: a preallocated one)."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        out = np.empty(max(len(handles), 1), dtype=np.float32) if out is None else out
        H.check(self._lib.zp_sched_temperatures(self._obj, _ptr(handles), len(handles), _ptr(out)), "temperatures")
        return out[:len(handles)]

    def prefill_inputs(self, handles):
        """One prefill step's host arrays (model_runner.py:352-422): dict(input_ids, positions,
        slot_mapping [new tokens], cu_seqlens_q, cu_seqlens_k [n + 1], query_triples [rows, 3],
        max_seqlen_q, max_seqlen_k, block_tables or None).  `block_tables` ([n, widest], -1 padded)
        is set when some sequence starts from cached prefix blocks, as in the reference.  Marks the
        sequences prefilled."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        n = len(handles)
        sizes = (C.c_int32 * 4)()
        H.check(self._lib.zp_sched_prefill_sizes(self._obj, _ptr(handles), n, sizes), "prefill_sizes")
        tokens, rows = sizes[0], sizes[1]
        out = {"input_ids": np.empty(max(tokens, 1), np.int32), "positions": np.empty(max(tokens, 1), np.int32),
               "slot_mapping": np.empty(max(tokens, 1), np.int32), "cu_seqlens_q": np.zeros(n + 1, np.int32),
               "cu_seqlens_k": np.zeros(n + 1, np.int32), "query_triples": np.empty((max(rows, 1), 3), np.int32)}
        tables = None
        width = (sizes[3] + self.block_size - 1) // self.block_size + 1
        d = self.decode_inputs(handles, table_width=width)
        with self._mutating():
            got = H.check(self._lib.zp_sched_prefill_inputs(
                self._obj, _ptr(handles), n, _ptr(out["input_ids"]), _ptr(out["positions"]), _ptr(out["slot_mapping"]),
                _ptr(out["cu_seqlens_q"]), _ptr(out["cu_seqlens_k"]), _ptr(out["query_triples"])), "prefill_inputs")
        assert got == rows
        for k in ("input_ids", "positions", "slot_mapping"):
            out[k] = out[k][:tokens]
        out["query_triples"] = out["query_triples"][:rows]
        if n and out["cu_seqlens_k"][-1] > out["cu_seqlens_q"][-1]:
            tables = d["block_tables"][:, :d["widest"]]
        out.update(max_seqlen_q=sizes[2], max_seqlen_k=sizes[3], block_tables=tables)
        return out

    def compress_due(self, handles):
        """The handles among `handles` whose sequence waits for a compression (int32 array)."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        out = np.empty(max(len(handles), 1), dtype=np.int32)
        n = H.check(self._lib.zp_sched_compress_due(self._obj, _ptr(handles), len(handles), _ptr(out)), "compress_due")
        return out[:n]

    def compress_inputs(self, handles, table_width=None):
        """The host arrays of one compression: dict(tables [n, table_width] with -1 padding and
        the last page as -(id)-2, targets [n, max_blocks_per_seq], query_ids, compressed, widest)."""
        handles = np.ascontiguousarray(handles, dtype=np.int32)
        n, nt = len(handles), self._cfg.max_blocks_per_seq
        w = table_width or max((self._seqs[h]._info()[11] for h in handles.tolist()), default=1)
        out = {"tables": np.empty((n, w), np.int32), "targets": np.empty((n, nt), np.int32),
               "query_ids": np.empty(n, np.int32), "compressed": np.empty(n, np.uint8)}
        out["widest"] = H.check(self._lib.zp_sched_compress_inputs(
            self._obj, _ptr(handles), n, _ptr(out["tables"]), w, _ptr(out["targets"]), nt,
            _ptr(out["query_ids"]), _ptr(out["compressed"])), "compress_inputs")
        return out
