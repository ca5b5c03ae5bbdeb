"""bf16 parity of the benchmarked configuration, as a proof rather than a tolerance.

A slice of the headline workload — 32 query / 8 KV heads, head_dim 128, window of 32 queries,
9 pages compressed into 8, pooling kernel 7, lambda 0.5, redundancy temperature 0.4, bf16 caches,
the tcgen05 kernels — is run through the C ABI and through the CPU oracle.  Checked:
  * attention scores and selection scores within 2e-2 relative of the oracle (the bf16 tolerance);
  * every index on which the kept sets differ has an oracle selection score within ONE bf16
    rounding step of the row's k-th score (oracle/boundary.py states the rule); the count of
    such indices and the worst gap are printed;
  * given the oracle's keep flags, the CUDA compaction reproduces the oracle's caches bit for bit.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

BS = 256


def _slice(seed, dtype, B=8, L=2):
    from zipage_b200.synthetic import make_compress_workload
    return make_compress_workload(B=B, L=L, Hkv=8, Hq=32, QCL=32, budget=8, dtype=dtype,
                                  device="cuda:0", seed=seed)


@pytest.mark.parametrize("variant", ["lightning", "exact"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_headline_configuration_kept_sets_differ_only_at_the_cut(variant, dtype):
    from oracle import zipage_oracle as O
    from oracle.boundary import kept_set_report
    from zipage_b200 import _lib, kernel as K
    from zipage_b200.compress import CompressConfig, compress_chunk
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    cfg = dict(budget_blocks=8, query_cache_len=32, use_redudancy=True,
               lightning_redudancy=variant == "lightning", redudancy_lambda=0.5,
               redudancy_temperature=0.4, enable_pooling=True, pooling_size=7)
    w = _slice(21, dtype)
    L, B, Hkv, NB = 2, 8, 8, 9
    # oracle on copies
    ko, vo = w.kv_cache[0].cpu().clone(), w.kv_cache[1].cpu().clone()
    att_o = O.attention_score(ko, w.query_cache.cpu(), w.query_ids.cpu(), w.block_tables.cpu())
    parts = {}
    final_o, keep_o = O.compress(ko, vo, w.query_cache.cpu(), None, w.query_ids.cpu(),
                                 w.block_tables.cpu(), w.target_tables.cpu(), w.compressed.cpu(),
                                 O.CompressConfig(**cfg), parts=parts)
    # compaction alone, fed the oracle's flags
    k2, v2 = w.kv_cache[0].clone(), w.kv_cache[1].clone()
    K.compress_kv(k2, v2, keep_o.cuda(), w.block_tables, w.target_tables)
    assert torch.equal(k2.cpu(), ko) and torch.equal(v2.cpu(), vo)
    # the whole op on the tensor-core kernels
    att = K.attention_score(w.kv_cache[0], w.query_cache, w.query_ids, w.block_tables, impl="tcgen05")
    dbg = compress_chunk(w.kv_cache[0], w.kv_cache[1], w.query_cache, None, w.query_ids,
                         w.block_tables, w.target_tables, w.compressed, CompressConfig(**cfg),
                         impl="tcgen05", return_debug=True)
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    a, b = att.float().cpu(), att_o.float()
    assert (a - b).abs().max() <= 2e-2 * b.abs().max()
    fa, fb = dbg["final"].float().cpu(), final_o.float()
    fin = torch.isfinite(fb)
    assert torch.equal(fa[~fin], fb[~fin])
    assert (fa[fin] - fb[fin]).abs().max() <= 2e-2 * fb[fin].abs().max()
    keep = dbg["keep"].cpu()
    assert (keep.flatten(3).sum(-1) == 8 * BS).all()
    rep = kept_set_report(final_o.view(L, B, Hkv, -1), keep_o.view(L, B, Hkv, -1),
                          keep.view(L, B, Hkv, -1), 8 * BS, dtype, parts)
    print(f"config-2 slice {variant} {dtype}: scores differing from the oracle "
          f"{(a != b).float().mean().item():.2e}, kept-set mismatch {rep['mismatch']:.2e} "
          f"({rep['differing']} flags), outside one step of the cut {rep['outside']}, "
          f"worst gap {rep['worst']:.2f} steps")
    assert rep["outside"] == 0, rep
    assert rep["mismatch"] < 2e-3, rep
