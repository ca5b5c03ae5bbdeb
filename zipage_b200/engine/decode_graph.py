"""The decode step as CUDA graphs, one per batch-size bucket.

Counterpart of `ModelRunner.capture_cudagraph` (zipage/engine/model_runner.py:747-787) and of the
replay branch of `run_model` (:709-724), which the reference leaves disabled: its decode step
builds `slot_mapping`, `context_lens`, `positions` and a variable-length list of window-query
triples on the host every step (`prepare_decode`, :633-675), and a list whose length changes
cannot be an input of a replayed graph.  Here those four are built by one kernel from device
state inside the graph, the triple list has a fixed capacity with its valid count kept on the
device, so a replay needs only `input_ids`, `num_tokens`, `block_tables` and `query_ids` copied
into the graph's input buffers.  Rows past the live batch carry `num_tokens = 0`: they store
nothing and attend to nothing.
"""
from __future__ import annotations

import torch

from ..layers.step_ops import prepare_decode
from ..utils.context import reset_context, set_context


class DecodeGraphRunner:
    def __init__(self, model, hidden_size, max_bs, max_num_blocks, query_cache_len, block_size=256,
                 dtype=torch.bfloat16, device="cuda", graph_bs=None):
        self.model = model
        self.qcl, self.block_size = query_cache_len, block_size
        self.max_bs = max_bs
        dev = torch.device(device)
        self.input_ids = torch.zeros(max_bs, dtype=torch.int64, device=dev)
        self.num_tokens = torch.zeros(max_bs, dtype=torch.int32, device=dev)
        self.block_tables = torch.full((max_bs, max_num_blocks), -1, dtype=torch.int32, device=dev)
        self.query_ids = torch.full((max_bs,), -1, dtype=torch.int32, device=dev)
        self.outputs = torch.zeros(max_bs, hidden_size, dtype=dtype, device=dev)
        self.graph_bs = sorted(graph_bs) if graph_bs else \
            [b for b in (1, 2, 4, 8) if b <= max_bs] + list(range(16, max_bs + 1, 16))
        if self.graph_bs[-1] < max_bs:
            self.graph_bs.append(max_bs)
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_pool = None

    def _step(self, bs):
        """One decode forward over the first `bs` rows of the input buffers."""
        pos, ctx, slot, trip, ntrip = prepare_decode(self.num_tokens[:bs], self.block_tables[:bs],
                                                     self.query_ids[:bs], self.qcl, self.block_size)
        set_context(False, slot_mapping=slot, context_lens=ctx, block_tables=self.block_tables[:bs],
                    query_slot_mapping=trip, query_slot_count=ntrip)
        try:
            return self.model(self.input_ids[:bs], pos)
        finally:
            reset_context()

    @torch.inference_mode()
    def capture(self):
        """Warm up and capture every bucket, largest first so the smaller graphs share its pool.
        The input buffers hold `num_tokens = 0` here: the captured launches write no cache row."""
        self.num_tokens.zero_()
        for bs in reversed(self.graph_bs):
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.outputs[:bs] = self._step(bs)  # warm-up: lazy tables, workspaces, cuBLAS handles
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, self.graph_pool):
                self.outputs[:bs] = self._step(bs)
            if self.graph_pool is None:
                self.graph_pool = graph.pool()
            self.graphs[bs] = graph
            torch.cuda.synchronize()

    def _fill(self, input_ids, num_tokens, block_tables, query_ids):
        bs = input_ids.shape[0]
        assert bs <= self.max_bs and block_tables.shape[1] <= self.block_tables.shape[1]
        self.input_ids[:bs] = input_ids
        self.num_tokens.zero_()
        self.num_tokens[:bs] = num_tokens
        self.block_tables.fill_(-1)
        self.block_tables[:bs, : block_tables.shape[1]] = block_tables
        self.query_ids.fill_(-1)
        self.query_ids[:bs] = query_ids
        return bs

    @torch.inference_mode()
    def run(self, input_ids, num_tokens, block_tables, query_ids, eager=False):
        """input_ids [bs] i64, num_tokens [bs] i32 (len(seq) with the fed token), block_tables
        [bs, w] i32 (-1 padded), query_ids [bs] i32 (-1 = no window) -> hidden states [bs, H]
        (a view of the graph's output buffer, valid until the next call)."""
        bs = self._fill(input_ids, num_tokens, block_tables, query_ids)
        if eager:
            self.outputs[:bs] = self._step(bs)
            return self.outputs[:bs]
        if not self.graphs:
            raise RuntimeError("DecodeGraphRunner.run: capture() has not been called")
        self.graphs[next(x for x in self.graph_bs if x >= bs)].replay()
        return self.outputs[:bs]
