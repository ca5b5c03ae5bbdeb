"""One rank of a serving loop built from this library only: the native scheduler and page manager
(host arrays, no per-sequence Python), prefill through the decoder blocks' varlen path, the decode
forward as replayed CUDA graphs, compression through `Compressor`, the LM head and the sampler.

It follows the reference engine's step protocol (zipage/engine/zipage_engine.py:99-135:
schedule -> compress the sequences that are due -> run -> postprocess) and its accounting
(`time_record` keys prefill_sum / decode_sum / compress_sum, decode throughput = decode tokens over
decode_sum + compress_sum).  Under tensor parallelism every rank runs this same loop on the same
requests: the sharded sampler leaves every rank with the step's tokens, so the schedulers stay in
step without any message (the reference pickles the scheduled sequences to its worker ranks every
step, model_runner.py:151-203).
"""
from __future__ import annotations

import time
from collections import defaultdict

import numpy as np
import torch

from .. import _lib as L
from ..layers.step_ops import sample
from ..utils.context import reset_context, set_context
from .compressor import Compressor
from .decode_graph import DecodeGraphRunner
from .scheduler import Scheduler


def full_state_from_hf(hf_state):
    """A Hugging Face Qwen3 state dict (separate q/k/v and gate/up projections, `model.` prefix)
    -> (the unsharded state `Qwen3Model.load_full_state` takes, the LM head weight)."""
    out = {}
    for name, w in hf_state.items():
        if not name.startswith("model."):
            continue
        name = name[len("model."):]
        if ".self_attn.q_proj." in name:
            base = name.replace("q_proj", "{}")
            out[base.format("qkv_proj")] = torch.cat([hf_state["model." + base.format(p)] for p in ("q_proj", "k_proj", "v_proj")], 0)
        elif ".mlp.gate_proj." in name:
            base = name.replace("gate_proj", "{}")
            out[base.format("gate_up_proj")] = torch.cat([hf_state["model." + base.format(p)] for p in ("gate_proj", "up_proj")], 0)
        elif not any(k in name for k in (".k_proj.", ".v_proj.", ".up_proj.")):
            out[name] = w
    return out, hf_state.get("lm_head.weight", hf_state.get("model.embed_tokens.weight"))


class NativeEngine:
    def __init__(self, model, lm_head, kv_cache, query_cache, sched_config, compress_cfg, hidden_size,
                 comm=None, max_bs=256, max_model_len=4096, score_cache=None, layer_stride=8,
                 greedy=False, graph=True, seed=0):
        self.model, self.lm_head, self.comm = model, lm_head, comm
        self.device = kv_cache.device
        self.block_size = int(kv_cache.shape[3])
        self.qcl = sched_config.query_cache_len
        self.scheduler = Scheduler(sched_config)
        self.compressor = Compressor(kv_cache, query_cache, score_cache, compress_cfg, layer_stride=layer_stride)
        self.width = (max_model_len + self.block_size - 1) // self.block_size + 1
        self.max_bs = max_bs
        self.runner = DecodeGraphRunner(model, hidden_size, max_bs=max_bs, max_num_blocks=self.width,
                                        query_cache_len=self.qcl, block_size=self.block_size,
                                        dtype=kv_cache.dtype, device=self.device)
        self.graph = graph
        if graph:
            self.runner.capture()
        self.greedy, self.seed, self.step_no = greedy, seed, 0
        self.forced = None          # optional iterator of token lists (teacher forcing in tests)
        self.argmax_log = None      # optional list: own arg-max of every step
        self.time_record = defaultdict(float)
        pin = lambda *shape: torch.empty(*shape, dtype=torch.int32).pin_memory()
        self._staged = {"input_ids": pin(max_bs), "num_tokens": pin(max_bs), "query_ids": pin(max_bs),
                        "block_tables": pin(max_bs, self.width)}
        self._views = {k: v.numpy() for k, v in self._staged.items()}
        if sched_config.max_num_seqs > max_bs:
            raise ValueError(f"max_num_seqs {sched_config.max_num_seqs} exceeds the {max_bs} rows of the decode graphs")
        self._tokens_host = torch.empty(max(max_bs, sched_config.max_num_seqs), dtype=torch.int64).pin_memory()
        self._pin_err = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._temps_host = torch.empty(max(max_bs, sched_config.max_num_seqs), dtype=torch.float32).pin_memory()
        self._temps_view = self._temps_host.numpy()

    # -- requests -------------------------------------------------------------------------------
    def add_request(self, seq):
        self.scheduler.add(seq)
        return seq._h

    def is_finished(self):
        return self.scheduler.is_finished()

    # -- one step -------------------------------------------------------------------------------
    def _sample(self, logits, handles):
        n = logits.shape[0]
        self.step_no += 1
        if self.argmax_log is not None:
            lf = logits.float()
            top = lf.topk(2, dim=-1)
            self.argmax_log.append({"tokens": logits.argmax(dim=-1).tolist(),   # what `greedy` emits
                                    "margin": (top.values[:, 0] - top.values[:, 1]).tolist(),
                                    "spread": (lf.max(dim=-1).values - lf.min(dim=-1).values).tolist()})
        if self.forced is not None:
            return np.asarray(next(self.forced), dtype=np.int32)
        if self.greedy:
            tok = logits.argmax(dim=-1)
        else:
            self.scheduler.temperatures(handles, out=self._temps_view)
            temps = self._temps_host[:n].to(self.device, non_blocking=True)
            seed = self.seed * 1000003 + self.step_no
            tok = self.comm.sample(logits, temps, seed=seed) if self.comm is not None else sample(logits, temps, seed=seed)
        self._tokens_host[:n].copy_(tok, non_blocking=True)
        # a tensor-core kernel whose bounded wait ran out (prefill attention) leaves its code in the
        # device error word: read it with the tokens, on this stream only
        L.check(L.load().zp_device_error_async(L.ptr(self._pin_err), L.stream_ptr()), "device_error")
        torch.cuda.current_stream().synchronize()
        if int(self._pin_err[0]) != 0:
            code = int(self._pin_err[0])
            L.device_error(reset=True)
            raise L.ZipageError(f"a kernel of this step gave up on a barrier wait (code {code})")
        return self._tokens_host[:n].numpy().astype(np.int32)

    @torch.inference_mode()
    def _prefill(self, handles):
        p = self.scheduler.prefill_inputs(handles)
        self._last_prefill_tokens = len(p["input_ids"])
        dev = self.device
        to = lambda a, dt=torch.int32: torch.from_numpy(np.ascontiguousarray(a)).to(dev, dtype=dt, non_blocking=False)
        cu_q = to(p["cu_seqlens_q"])
        triples = to(p["query_triples"]) if len(p["query_triples"]) else None
        set_context(True, cu_q, to(p["cu_seqlens_k"]), int(p["max_seqlen_q"]), int(p["max_seqlen_k"]),
                    to(p["slot_mapping"]), query_slot_mapping=triples, context_lens=None,
                    block_tables=None if p["block_tables"] is None else to(p["block_tables"]))
        try:
            hidden = self.model(to(p["input_ids"], torch.int64), to(p["positions"], torch.int64))
        finally:
            reset_context()
        last = hidden[(cu_q[1:] - 1).long()]
        return torch.nn.functional.linear(last, self.lm_head)

    @torch.inference_mode()
    def _decode(self, handles):
        n = len(handles)
        d = self.scheduler.decode_inputs(handles, table_width=self.width, out=self._views)
        dev, st = self.device, self._staged
        hidden = self.runner.run(st["input_ids"][:n].to(dev, non_blocking=True), st["num_tokens"][:n].to(dev, non_blocking=True),
                                 st["block_tables"][:n, :d["widest"]].to(dev, non_blocking=True),
                                 st["query_ids"][:n].to(dev, non_blocking=True), eager=not self.graph)
        return torch.nn.functional.linear(hidden, self.lm_head)

    def step(self):
        """-> (handles that finished, tokens of the step: > 0 prefill tokens, < 0 decode tokens)."""
        sched = self.scheduler
        handles, is_prefill = sched.schedule_batch()
        n = len(handles)
        if n == 0:
            return handles, 0
        if n > self.max_bs and not is_prefill:
            raise RuntimeError(f"{n} sequences scheduled, the decode graphs hold {self.max_bs}")
        if not is_prefill:
            due = sched.compress_due(handles)
            if len(due):
                t0 = time.perf_counter()
                c = sched.compress_inputs(due)
                self.compressor.compress_tables(c["tables"], c["targets"], c["query_ids"], c["compressed"], encoded=True)
                sched.postprocess_batch(due)
                self.time_record["compress_sum"] += time.perf_counter() - t0
                self.time_record["compress_reqs"] += len(due)
        t0 = time.perf_counter()
        if is_prefill:
            logits = self._prefill(handles)
        else:
            logits = self._decode(handles)
        tokens = self._sample(logits, handles)
        done = sched.postprocess_batch(handles, tokens)
        dt = time.perf_counter() - t0
        if is_prefill:
            self.time_record["prefill_sum"] += dt
            return done, int(self._last_prefill_tokens)
        self.time_record["decode_sum"] += dt
        self.time_record["decode_tokens"] += n
        return done, -n

    def generate(self, seqs):
        """Runs the requests to completion; -> {handle: completion token ids}."""
        for s in seqs:
            self.add_request(s)
        while not self.is_finished():
            self.step()
        return {s._h: s.completion_token_ids for s in seqs}
