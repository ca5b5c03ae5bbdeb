"""Edge cases of the compression path on the GPU: empty batches, long ragged tables with fresh
target pages (first compression of a long prompt), group sizes the tensor-core kernel does not
cover, tables shorter than the budget, oversized rows."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BS = 256


def _run_both(w, cfg_kwargs, dtype, impl="auto"):
    from oracle import zipage_oracle as O
    from zipage_b200.compress import CompressConfig, compress_chunk
    ko, vo = w.kv_cache[0].cpu().clone(), w.kv_cache[1].cpu().clone()
    sco = None if w.score_cache is None else w.score_cache.cpu().clone()
    parts = {}
    final_o, keep_o = O.compress(ko, vo, w.query_cache.cpu(), sco, w.query_ids.cpu(), w.block_tables.cpu(),
                                 w.target_tables.cpu(), w.compressed.cpu(), O.CompressConfig(**cfg_kwargs),
                                 parts=parts)
    dbg = compress_chunk(w.kv_cache[0], w.kv_cache[1], w.query_cache, w.score_cache, w.query_ids,
                         w.block_tables, w.target_tables, w.compressed, CompressConfig(**cfg_kwargs),
                         impl=impl, return_debug=True)
    torch.cuda.synchronize()
    dbg["oracle_parts"] = parts
    return (final_o, keep_o, ko, vo), dbg


def test_empty_batch_is_a_noop():
    from zipage_b200 import kernel as K
    dev = torch.device("cuda:0")
    k = torch.zeros(2, 4, BS, 2, 128, device=dev, dtype=torch.bfloat16)
    q = torch.zeros(2, 3, 16, 4, 128, device=dev, dtype=torch.bfloat16)
    bt = torch.zeros(0, 3, dtype=torch.int32, device=dev)
    s = K.attention_score(k, q, torch.zeros(0, dtype=torch.int32, device=dev), bt)
    assert s.shape == (2, 0, 2, 3, BS)
    K.compress_kv(k, k.clone(), torch.zeros(2, 0, 2, 3, BS, dtype=torch.bool, device=dev), bt,
                  torch.zeros(0, 3, dtype=torch.int32, device=dev))
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_prompt_first_compression(dtype):
    """Tables of 9..40 pages compressed to 8 (+1), some targets starting with fresh pages."""
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    w = make_compress_workload(B=4, L=1, Hkv=2, Hq=8, QCL=16, budget=8, pages_per_seq=[40, 9, 17, 12],
                               dtype=dtype, device=dev, seed=5, with_score_cache=True, compressed_prob=0.5,
                               fresh_target_prob=0.7, similar_keys=True)
    cfg = dict(budget_blocks=8, query_cache_len=16, use_global_score=True, use_redudancy=True,
               lightning_redudancy=True, enable_pooling=True)
    (final_o, keep_o, ko, vo), dbg = _run_both(w, cfg, dtype)
    keep = dbg["keep"].cpu()
    assert (keep.flatten(3).sum(-1) == 8 * BS).all()
    if dtype == torch.float32:
        assert torch.equal(keep, keep_o)
        assert torch.equal(w.kv_cache[0].cpu(), ko) and torch.equal(w.kv_cache[1].cpu(), vo)
    else:
        from oracle.boundary import kept_set_report
        L, B, Hkv = keep.shape[:3]
        rep = kept_set_report(final_o.reshape(L, B, Hkv, -1), keep_o.reshape(L, B, Hkv, -1),
                              keep.reshape(L, B, Hkv, -1), 8 * BS, dtype, dbg["oracle_parts"])
        assert rep["outside"] == 0 and rep["mismatch"] < 1e-2, rep


@pytest.mark.parametrize("reduced", ["mean", "max"])
def test_group_of_eight_with_window_32_takes_two_passes(reduced):
    """G*QCL = 256 window rows: the tensor-core kernel runs two passes of 128 rows whose per-key
    sums meet in a workspace; without a workspace the call falls back to the portable kernel."""
    from oracle import zipage_oracle as O
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    w = make_compress_workload(B=3, L=2, Hkv=1, Hq=8, QCL=32, budget=2, pages_per_seq=[3, 4, 3],
                               dtype=torch.bfloat16, device=dev, seed=8)
    o = O.attention_score(w.kv_cache[0].cpu(), w.query_cache.cpu(), w.query_ids.cpu(),
                          w.block_tables.cpu(), reduced=reduced).float()
    a = K.attention_score(w.kv_cache[0], w.query_cache, w.query_ids, w.block_tables, reduced=reduced,
                          impl="tcgen05").float().cpu()
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    b = K.attention_score(w.kv_cache[0], w.query_cache, w.query_ids, w.block_tables, reduced=reduced,
                          impl="simt").float().cpu()
    assert (a - o).abs().max() <= 2e-2 * o.abs().max()
    assert (b - o).abs().max() <= 2e-2 * o.abs().max()
    assert (a != o).float().mean() < 0.02
    # the whole op through the single entry point (its workspace covers two passes)
    from zipage_b200.compress import CompressConfig, compress_batch
    cfg = dict(budget_blocks=2, query_cache_len=32, use_redudancy=True, lightning_redudancy=True,
               enable_pooling=True)
    from oracle.boundary import kept_set_report
    from zipage_b200.compress import compress_chunk
    ko, vo = w.kv_cache[0].cpu().clone(), w.kv_cache[1].cpu().clone()
    k2, v2 = w.kv_cache[0].clone(), w.kv_cache[1].clone()
    parts = {}
    final_o, keep_o = O.compress(ko, vo, w.query_cache.cpu(), None, w.query_ids.cpu(), w.block_tables.cpu(),
                                 w.target_tables.cpu(), w.compressed.cpu(), O.CompressConfig(**cfg), parts=parts)
    # stage by stage on a copy, to see the kept set: it may differ from the oracle's only at the cut
    dbg = compress_chunk(k2, v2, w.query_cache, None, w.query_ids, w.block_tables, w.target_tables,
                         w.compressed, CompressConfig(**cfg), return_debug=True)
    compress_batch(w.kv_cache[0], w.kv_cache[1], w.query_cache, None, w.query_ids, w.block_tables,
                   w.target_tables, w.compressed, CompressConfig(**cfg))
    torch.cuda.synchronize()
    keep = dbg["keep"].cpu()
    L, B, Hkv = keep.shape[:3]
    rep = kept_set_report(final_o.reshape(L, B, Hkv, -1), keep_o.reshape(L, B, Hkv, -1),
                          keep.reshape(L, B, Hkv, -1), 2 * BS, torch.bfloat16, parts)
    assert rep["outside"] == 0 and rep["mismatch"] < 1e-2, rep
    # and the single entry point leaves the caches exactly as the stage-by-stage path does
    assert torch.equal(w.kv_cache[0], k2) and torch.equal(w.kv_cache[1], v2)


def test_table_not_longer_than_budget_keeps_everything():
    from zipage_b200 import kernel as K
    dev = torch.device("cuda:0")
    scores = torch.rand(1, 2, 2, 2 * BS, device=dev)
    keep = K.topk_mask(scores, 4 * BS)
    assert keep.all()
    keep = K.topk_mask(scores, 2 * BS)
    assert keep.all()


def test_oversized_row_is_rejected_cleanly():
    from zipage_b200 import kernel as K, _lib
    dev = torch.device("cuda:0")
    scores = torch.zeros(1, 1, 1, 300 * BS, device=dev)  # 76 800 fp32 scores > shared memory
    with pytest.raises(_lib.ZipageError, match="shared memory"):
        K.topk_mask(scores, 8 * BS)


def test_config5_first_compression_from_128_and_64_pages():
    """The long-prompt case at its own scale: tables of 128 and 64 full pages (32k / 16k tokens)
    compressed into 8 (+1), one KV head with 8 query heads (a TP=8 rank of Qwen3-32B), window 32
    (256 window rows: two passes of the tensor-core window kernel), bf16, lightning redundancy."""
    from oracle.boundary import kept_set_report
    from zipage_b200 import _lib
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    w = make_compress_workload(B=2, L=1, Hkv=1, Hq=8, QCL=32, budget=8, pages_per_seq=[128, 64],
                               dtype=torch.bfloat16, device=dev, seed=9, compressed_prob=0.0,
                               fresh_target_prob=1.0)
    cfg = dict(budget_blocks=8, query_cache_len=32, use_redudancy=True, lightning_redudancy=True,
               redudancy_lambda=0.5, enable_pooling=True)
    (final_o, keep_o, ko, vo), dbg = _run_both(w, cfg, torch.bfloat16)
    assert _lib.device_error() == 0
    keep = dbg["keep"].cpu()
    assert (keep.flatten(3).sum(-1) == 8 * BS).all()
    rep = kept_set_report(final_o.reshape(1, 2, 1, -1), keep_o.reshape(1, 2, 1, -1), keep.reshape(1, 2, 1, -1),
                          8 * BS, torch.bfloat16, dbg["oracle_parts"])
    print(f"128 / 64 pages -> 8: {rep}")
    assert rep["outside"] == 0 and rep["mismatch"] < 1e-3, rep


def test_select_rows_too_long_for_two_arrays_recompute_the_redundancy():
    """A row of 240 pages in bf16 with redundancy needs 2 x 120 KB of shared memory for scores and
    scaled logits; the kernel then keeps only the scores there and recomputes the logits per pass.
    Same kept set as the oracle's selection on the same scores."""
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    dev = torch.device("cuda:0")
    NB = 240
    g = torch.Generator().manual_seed(2)
    scores = (torch.rand(1, 1, 2, NB, BS, generator=g) / (NB * BS)).to(torch.bfloat16)
    red = torch.randn(1, 1, 2, NB, BS, generator=g).to(torch.bfloat16)
    table = torch.arange(NB, dtype=torch.int32).view(1, NB)
    table[0, -1] = -table[0, -1] - 2
    comp = torch.zeros(1, dtype=torch.bool)
    keep, final = K.select_keep(scores.to(dev), table.to(dev), comp.to(dev), 8 * BS, 16, red_logits=red.to(dev),
                                redundancy="lightning", redudancy_lambda=0.5, redudancy_temperature=0.4,
                                pooling_size=5, return_final=True)
    s = O.pool_scores(scores.clone(), comp, 5, False)
    r = red.view(1, 1, 2, -1).clone()
    r = r.div_(0.4 * BS)
    r = (r - r.max(dim=-1, keepdim=True).values).softmax(dim=-1).view(1, 1, 2, NB, BS)
    f = O.combine_scores(s, r, 0.5).contiguous()
    O.window_mask(f, table, 16)
    O.pad_mask_(f, table)
    fin = torch.isfinite(f.float())
    assert torch.equal(final.cpu().float()[~fin], f.float()[~fin])
    assert (final.cpu().float()[fin] - f.float()[fin]).abs().max() <= 2e-2 * f.float()[fin].abs().max()
    want = O.topk_mask(final.cpu().view(1, 1, 2, -1), 8 * BS)
    assert torch.equal(keep.cpu().view(1, 1, 2, -1), want)


@pytest.mark.parametrize("variant", ["lightning", "exact", "none"])
def test_single_entry_point_equals_stage_by_stage(variant):
    """zp_compress_batch (one C call) leaves the caches exactly as the stage-by-stage path does."""
    from zipage_b200.compress import CompressConfig, compress_batch, compress_chunk
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    mk = lambda: make_compress_workload(B=3, L=2, Hkv=2, Hq=8, QCL=16, budget=2, pages_per_seq=[3, 5, 3],
                                        dtype=torch.bfloat16, device=dev, seed=12, with_score_cache=True,
                                        compressed_prob=0.5, fresh_target_prob=0.5, similar_keys=True)
    cfg = CompressConfig(budget_blocks=2, query_cache_len=16, use_global_score=True, decay_factor=0.8,
                         use_redudancy=variant != "none", lightning_redudancy=variant == "lightning",
                         enable_pooling=True, use_attention_sink=True, sink_len=4)
    a, b = mk(), mk()
    compress_chunk(a.kv_cache[0], a.kv_cache[1], a.query_cache, a.score_cache, a.query_ids, a.block_tables,
                   a.target_tables, a.compressed, cfg)
    new_table, ctx, nxt = compress_batch(b.kv_cache[0], b.kv_cache[1], b.query_cache, b.score_cache,
                                         b.query_ids, b.block_tables, b.target_tables, b.compressed, cfg,
                                         update_tables=True)
    torch.cuda.synchronize()
    assert torch.equal(a.kv_cache, b.kv_cache) and torch.equal(a.score_cache, b.score_cache)
    assert torch.equal(new_table, b.target_tables) and ctx.tolist() == [2 * BS + 1] * 3
    assert nxt.tolist() == (b.target_tables[:, -1] * BS).tolist()


def test_exact_similarity_on_tables_longer_than_64_pages():
    """The tensor-core kernel of the exact similarity walks tables of any length (the long-prompt
    case: 64..128 pages); checked against the portable kernel, which the oracle pins, on a ragged
    pair of 70 and 66 pages with padding inside the rectangle."""
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    w = make_compress_workload(B=2, L=1, Hkv=2, Hq=8, QCL=16, budget=8, pages_per_seq=[70, 66],
                               dtype=torch.bfloat16, device=dev, seed=13, compressed_prob=0.0, similar_keys=True)
    a = K.redundancy_logits(w.kv_cache[0], w.block_tables, 0.5, exact=True, impl="tcgen05").float()
    b = K.redundancy_logits(w.kv_cache[0], w.block_tables, 0.5, exact=True, impl="simt").float()
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin)
    assert (a[fin] - b[fin]).abs().max() <= 2e-2 * b[fin].abs().max()
    assert (a[fin] != b[fin]).float().mean() < 0.05
