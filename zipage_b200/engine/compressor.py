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

from .. import _lib as L
from .. import kernel as K
from ..compress import CompressConfig, compress_batch, compress_chunk


def encode_block_tables(tables):
    """Pad the sequences' page lists to a rectangle with -1 and mark each last page as -(id)-2
    (zipage/engine/model_runner.py:440-441, :457-463)."""
    nb = max(len(t) for t in tables)
    return [list(t[:-1]) + [-t[-1] - 2] + [-1] * (nb - len(t)) for t in tables]


class Compressor:
    def __init__(self, kv_cache, query_cache, score_cache, cfg: CompressConfig, layer_stride=8,
                 impl="auto", stream=None, block_size=None):
        self.kv_cache, self.query_cache, self.score_cache = kv_cache, query_cache, score_cache
        self.cfg, self.layer_stride, self.impl = cfg, layer_stride, impl
        self.block_size = int(block_size or kv_cache.shape[3])
        self.num_layers = kv_cache.shape[1]
        self.device = kv_cache.device
        self.compress_stream = stream or torch.cuda.Stream(device=self.device)
        self.time_record = defaultdict(float)
        self.workspace = None      # scratch of the exact similarity kernels (stage-by-stage path)
        self._batch_ws = None      # scratch of the single-call path
        self.last_h2d_bytes = self.last_d2h_bytes = 0
        self._exact_ws = bool(cfg.use_redudancy and not cfg.lightning_redudancy)
        # pinned staging, allocated once and grown on demand (pinned allocation is a slow,
        # synchronising call; the engine compresses a few dozen sequences every few steps)
        self._pin_i32 = None      # tables | targets | query ids | new tables | context lengths
        self._pin_u8 = None       # compressed flags
        self._pin_err = torch.zeros(1, dtype=torch.int32).pin_memory()

    # -- reference-facing entry point -------------------------------------------------------
    def compress(self, seqs):
        """Same call as ModelRunner.compress(seqs): compacts each sequence's pages into its
        `new_block_table` in place and returns the sequences."""
        tables = [list(s.block_table) for s in seqs]
        targets = [list(s.new_block_table) for s in seqs]
        self.compress_tables(tables, targets, [s.query_id for s in seqs],
                             [bool(s.compressed) for s in seqs], timed=True)
        return seqs

    def _staging(self, n_i32, n_u8):
        if self._pin_i32 is None or self._pin_i32.numel() < n_i32:
            self._pin_i32 = torch.empty(max(n_i32, 4096), dtype=torch.int32).pin_memory()
        if self._pin_u8 is None or self._pin_u8.numel() < n_u8:
            self._pin_u8 = torch.empty(max(n_u8, 1024), dtype=torch.uint8).pin_memory()
        return self._pin_i32, self._pin_u8

    # -- list-based variant -------------------------------------------------------------------
    def compress_tables(self, tables, targets, query_ids, compressed, timed=False, encoded=False):
        """tables: per-sequence page lists (plain ids, last entry = the page holding the window), or,
        with `encoded`, the rectangular table already padded with -1 and with the last page written
        as -(id)-2 (what the native scheduler's compress_inputs returns; arrays are fine);
        targets: per-sequence destination pages (budget+1 each).  Returns (new_tables, context_lens)
        as host lists read back from the device-side table update.  With `timed` the stages run
        as separate launches between CUDA events and `time_record` gets the reference's keys
        (model_runner.py:623-630); otherwise each layer chunk is one C call."""
        B = len(tables)
        if B == 0:
            return [], []
        enc = tables if encoded else encode_block_tables(tables)
        nb, nt = len(enc[0]), len(targets[0])
        # one pinned block: [tables B*nb | targets B*nt | qids B | out: new tables B*nt | ctx B]
        o_t, o_g, o_q = 0, B * nb, B * nb + B * nt
        o_new, o_ctx = o_q + B, o_q + B + B * nt
        pin, pin8 = self._staging(o_ctx + B, B)
        pin[o_t:o_g] = torch.tensor(enc, dtype=torch.int32).view(-1)
        pin[o_g:o_q] = torch.tensor(targets, dtype=torch.int32).view(-1)
        pin[o_q:o_new] = torch.tensor(query_ids, dtype=torch.int32)
        pin8[:B] = torch.tensor(compressed, dtype=torch.uint8)
        self.last_h2d_bytes = (o_new - o_t) * 4 + B
        events = []

        @contextmanager
        def stage(name):
            st, ed = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record(self.compress_stream)
            yield
            ed.record(self.compress_stream)
            events.append((name, st, ed))

        with torch.cuda.stream(self.compress_stream):
            d_in = pin[o_t:o_new].to(self.device, non_blocking=True)
            d_tables = d_in[o_t:o_g].view(B, nb)
            d_targets = d_in[o_g:o_q].view(B, nt)
            d_qids = d_in[o_q:o_new]
            d_comp = pin8[:B].to(self.device, non_blocking=True)
            if self._exact_ws and timed:
                self._ensure_workspace(B, nb)
            for l0 in range(0, self.num_layers, self.layer_stride):
                sl = slice(l0, min(self.num_layers, l0 + self.layer_stride))
                sc = None if self.score_cache is None else self.score_cache[sl]
                if timed:
                    compress_chunk(self.kv_cache[0, sl], self.kv_cache[1, sl], self.query_cache[sl], sc,
                                   d_qids, d_tables, d_targets, d_comp.view(torch.bool), self.cfg,
                                   impl=self.impl, workspace=self.workspace, timers=stage)
                else:
                    self._batch_ws = compress_batch(
                        self.kv_cache[0, sl], self.kv_cache[1, sl], self.query_cache[sl], sc, d_qids,
                        d_tables, d_targets, d_comp, self.cfg, impl=self.impl, workspace=self._batch_ws,
                        return_workspace=True)
            new_tables, ctx, _ = K.update_tables(d_targets, block_size=self.block_size)
            pin[o_new:o_ctx].copy_(new_tables.view(-1), non_blocking=True)
            pin[o_ctx:o_ctx + B].copy_(ctx, non_blocking=True)
            # a tensor-core kernel whose bounded wait ran out leaves a wrong keep set behind:
            # read its error word with the results (4 bytes, this stream only)
            L.check(L.load().zp_device_error_async(L.ptr(self._pin_err), L.stream_ptr()), "device_error")
        self.compress_stream.synchronize()
        if int(self._pin_err[0]) != 0:
            code = int(self._pin_err[0])
            L.device_error(reset=True)
            raise L.ZipageError(f"compression kernels gave up on a barrier wait (code {code}); "
                                "the caches of this call are not valid")
        self.last_d2h_bytes = (B * nt + B) * 4 + 4
        if timed:
            per = defaultdict(list)
            for name, st, ed in events:
                t = st.elapsed_time(ed) / 1000
                per[name].append(t)
                self.time_record[name + "_sum"] += t
            for name, ts in per.items():
                self.time_record[name] = sum(ts) / len(ts)
        return pin[o_new:o_ctx].view(B, nt).tolist(), pin[o_ctx:o_ctx + B].tolist()

    def _ensure_workspace(self, B, nb):
        Hkv = self.kv_cache.shape[4]
        need = L.load().zp_redundancy_exact_workspace_bytes(
            min(self.layer_stride, self.num_layers), B, nb, Hkv, self.block_size)
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
