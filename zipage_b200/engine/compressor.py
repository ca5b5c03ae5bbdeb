"""Host side of the compression op: the `ModelRunner.compress(seqs)` contract.

`Compressor` owns nothing but references to the runner's caches (kv_cache [2,L,P,BS,Hkv,D],
query_cache [L,C,QCL,Hq,D], score_cache [L,P,BS,Hkv]) and a private CUDA stream.  `compress(seqs)`
takes the same sequence objects as the reference (fields query_id, block_table, new_block_table,
compressed; zipage/engine/model_runner.py:424-463), builds the four small index tensors in pinned
memory, copies them to the device on the compress stream, runs the kernels layer chunk by layer
chunk, synchronises that stream only, and fills `time_record` with the reference's stage names
(model_runner.py:623-630).  It never touches the run stream, so decode of other sequences
overlaps (zipage/engine/zipage_engine.py:137-186).
"""
from __future__ import annotations

from collections import defaultdict
from contextlib import contextmanager

import torch

from .. import kernel as K
from ..compress import CompressConfig, compress_chunk


def encode_block_tables(tables):
    """Pad the sequences' page lists to a rectangle with -1 and mark each last page as -(id)-2
    (zipage/engine/model_runner.py:440-441, :457-463)."""
    nb = max(len(t) for t in tables)
    return [list(t[:-1]) + [-t[-1] - 2] + [-1] * (nb - len(t)) for t in tables]


class Compressor:
    def __init__(self, kv_cache, query_cache, score_cache, cfg: CompressConfig, layer_stride=8,
                 impl="auto", stream=None, block_size=256):
        self.kv_cache, self.query_cache, self.score_cache = kv_cache, query_cache, score_cache
        self.cfg, self.layer_stride, self.impl = cfg, layer_stride, impl
        self.block_size = block_size
        self.num_layers = kv_cache.shape[1]
        self.device = kv_cache.device
        self.compress_stream = stream or torch.cuda.Stream(device=self.device)
        self.time_record = defaultdict(float)
        self.workspace = None
        self.last_h2d_bytes = self.last_d2h_bytes = 0
        if cfg.use_redudancy and not cfg.lightning_redudancy:
            self._exact_ws = True
        else:
            self._exact_ws = False

    # -- reference-facing entry point -------------------------------------------------------
    def compress(self, seqs):
        """Same call as ModelRunner.compress(seqs): compacts each sequence's pages into its
        `new_block_table` in place and returns the sequences."""
        tables = [list(s.block_table) for s in seqs]
        targets = [list(s.new_block_table) for s in seqs]
        self.compress_tables(tables, targets, [s.query_id for s in seqs],
                             [bool(s.compressed) for s in seqs], timed=True)
        return seqs

    # -- list-based variant -------------------------------------------------------------------
    def compress_tables(self, tables, targets, query_ids, compressed, timed=False):
        """tables: per-sequence page lists (plain ids, last entry = the page holding the window);
        targets: per-sequence destination pages (budget+1 each).  Returns (new_tables, context_lens)
        as host lists read back from the device-side table update."""
        B = len(tables)
        if B == 0:
            return [], []
        enc = encode_block_tables(tables)
        nb = len(enc[0])
        pin = lambda data, dt: torch.tensor(data, dtype=dt, pin_memory=True)
        h_tables, h_targets = pin(enc, torch.int32), pin(targets, torch.int32)
        h_qids, h_comp = pin(query_ids, torch.int32), pin(compressed, torch.bool)
        self.last_h2d_bytes = sum(t.numel() * t.element_size() for t in (h_tables, h_targets, h_qids, h_comp))
        events = []

        @contextmanager
        def stage(name):
            if not timed:
                yield
                return
            st, ed = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record(self.compress_stream)
            yield
            ed.record(self.compress_stream)
            events.append((name, st, ed))

        with torch.cuda.stream(self.compress_stream):
            d_tables = h_tables.to(self.device, non_blocking=True)
            d_targets = h_targets.to(self.device, non_blocking=True)
            d_qids = h_qids.to(self.device, non_blocking=True)
            d_comp = h_comp.to(self.device, non_blocking=True)
            if self._exact_ws:
                self._ensure_workspace(B, nb)
            for l0 in range(0, self.num_layers, self.layer_stride):
                sl = slice(l0, min(self.num_layers, l0 + self.layer_stride))
                compress_chunk(self.kv_cache[0, sl], self.kv_cache[1, sl], self.query_cache[sl],
                               None if self.score_cache is None else self.score_cache[sl], d_qids,
                               d_tables, d_targets, d_comp, self.cfg, impl=self.impl,
                               workspace=self.workspace, timers=stage)
            new_tables, ctx, _ = K.update_tables(d_targets)
            h_new = new_tables.to("cpu", non_blocking=True)
            h_ctx = ctx.to("cpu", non_blocking=True)
        self.compress_stream.synchronize()
        self.last_d2h_bytes = h_new.numel() * 4 + h_ctx.numel() * 4
        if timed:
            per = defaultdict(list)
            for name, st, ed in events:
                t = st.elapsed_time(ed) / 1000
                per[name].append(t)
                self.time_record[name + "_sum"] += t
            for name, ts in per.items():
                self.time_record[name] = sum(ts) / len(ts)
        return h_new.tolist(), h_ctx.tolist()

    def _ensure_workspace(self, B, nb):
        from .. import _lib as L
        Hkv = self.kv_cache.shape[4]
        need = L.load().zp_redundancy_exact_workspace_bytes(
            min(self.layer_stride, self.num_layers), B, nb, Hkv, self.block_size)
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
