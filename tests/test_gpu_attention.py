"""Paged decode and varlen prefill attention against the fp32 oracle (parity unpinned: the
reference calls flash-attn here, which has no golden vectors in its tree)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BS = 256


def _setup(dtype, P=40, Hkv=8, D=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
    vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
    return g, kc, vc


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 2e-2), (torch.float32, 1e-3)])
@pytest.mark.parametrize("Hq,Hkv,B", [(32, 8, 5), (8, 8, 3), (16, 2, 70), (64, 8, 2)])
def test_paged_decode(dtype, tol, Hq, Hkv, B):
    from oracle import zipage_oracle as O
    from zipage_b200.layers.attention import paged_decode_attention
    dev = torch.device("cuda:0")
    P = max(40, B * 2 + 4)
    g, kc, vc = _setup(dtype, P=P, Hkv=Hkv)
    NBmax = 9
    lens = torch.randint(1, NBmax * BS + 1, (B,), generator=g).to(torch.int32)
    lens[0] = 2049
    lens[-1] = 1
    if B > 2:
        lens[1] = NBmax * BS
    table = torch.full((B, NBmax), -1, dtype=torch.int32)
    for b in range(B):
        npg = (int(lens[b]) + BS - 1) // BS
        table[b, :npg] = torch.randperm(P, generator=g)[:npg].to(torch.int32)
    q = torch.randn(B, 1, Hq, 128, generator=g).to(dtype)
    ref = O.paged_decode_attention(q, kc, vc, lens, table)
    out = paged_decode_attention(q.to(dev), kc.to(dev), vc.to(dev), lens.to(dev), table.to(dev)).cpu()
    err = (out.float() - ref.float()).abs().max().item()
    assert err <= tol * ref.float().abs().max().item(), err


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-3)])
def test_varlen_prefill_dense_and_paged(dtype, tol):
    from oracle import zipage_oracle as O
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    Hq, Hkv, D = 8, 2, 128
    g, kc, vc = _setup(dtype, P=12, Hkv=Hkv)
    lens_k = [300, 1, 64, 517]
    # dense: q and k lengths equal
    cu = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    tot = int(cu[-1])
    q = torch.randn(tot, Hq, D, generator=g).to(dtype)
    k = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    v = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    ref = O.varlen_prefill_attention(q, k, v, cu, cu)
    out = varlen_prefill_attention(q.to(dev), k.to(dev), v.to(dev), max(lens_k), cu.to(dev),
                                   max(lens_k), cu.to(dev)).cpu()
    assert (out.float() - ref.float()).abs().max() <= tol * ref.float().abs().max()
    # paged with a cached prefix: fewer queries than keys, bottom-right aligned
    lens_q = [44, 1, 64, 5]
    cuq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    table = torch.full((4, 3), -1, dtype=torch.int32)
    perm = torch.randperm(12, generator=g)
    pos = 0
    for b, lk in enumerate(lens_k):
        npg = (lk + BS - 1) // BS
        table[b, :npg] = perm[pos:pos + npg].to(torch.int32)
        pos += npg
    q2 = torch.randn(int(cuq[-1]), Hq, D, generator=g).to(dtype)
    ref2 = O.varlen_prefill_attention(q2, kc, vc, cuq, cu, block_table=table)
    out2 = varlen_prefill_attention(q2.to(dev), kc.to(dev), vc.to(dev), max(lens_q), cuq.to(dev),
                                    max(lens_k), cu.to(dev), block_table=table.to(dev)).cpu()
    assert (out2.float() - ref2.float()).abs().max() <= tol * ref2.float().abs().max()


def test_attention_layer_contract():
    """Attention.forward: store K/V + window queries, then decode attention, as the reference layer."""
    from oracle import zipage_oracle as O
    from zipage_b200.layers.attention import Attention
    from zipage_b200.utils.context import reset_context, set_context
    dev = torch.device("cuda:0")
    dtype = torch.bfloat16
    Hq, Hkv, D, QCL, B = 8, 2, 128, 16, 3
    g, kc, vc = _setup(dtype, P=10, Hkv=Hkv)
    layer = Attention(Hq, D, D ** -0.5, Hkv)
    kc_d, vc_d = kc.to(dev), vc.to(dev)
    qcache = torch.zeros(4, QCL, Hq, D, dtype=dtype)
    layer.k_cache, layer.v_cache, layer.q_cache = kc_d, vc_d, qcache.to(dev)
    lens = torch.tensor([250, 513, 7], dtype=torch.int32)
    table = torch.tensor([[3, -1, -1], [0, 5, 8], [9, -1, -1]], dtype=torch.int32)
    slots = torch.tensor([3 * BS + 249, 8 * BS + 0, 9 * BS + 6], dtype=torch.int32)
    triples = torch.tensor([[0, 2, 249 - (BS - QCL)]], dtype=torch.int32)
    q = torch.randn(B, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, D, generator=g).to(dtype)
    set_context(False, slot_mapping=slots.to(dev), context_lens=lens.to(dev),
                block_tables=table.to(dev), query_slot_mapping=triples.to(dev))
    out = layer(q.to(dev), k.to(dev), v.to(dev)).cpu()
    reset_context()
    O.store_kvcache(k, v, kc, vc, slots)
    O.store_query_cache(q, qcache, triples)
    ref = O.paged_decode_attention(q.unsqueeze(1), kc, vc, lens, table)
    assert torch.equal(kc_d.cpu(), kc) and torch.equal(layer.q_cache.cpu(), qcache)
    assert (out.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()


def test_compress_then_decode_over_compacted_tables():
    """The path end to end on device: compress a batch, update the tables on the GPU, append one
    token with store_kvcache at the slot the table update names, and decode over the compacted
    pages.  The result must equal fp32 attention over exactly the kept tokens plus the new one."""
    from oracle import zipage_oracle as O
    from zipage_b200 import kernel as K
    from zipage_b200.compress import CompressConfig, compress_chunk
    from zipage_b200.layers.attention import paged_decode_attention
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    Hkv, Hq, D, budget = 2, 8, 128, 2
    w = make_compress_workload(B=3, L=1, Hkv=Hkv, Hq=Hq, QCL=16, budget=budget, pages_per_seq=[3, 4, 3],
                               dtype=torch.bfloat16, device=dev, seed=77, spare_pages=1,
                               compressed_prob=0.5, fresh_target_prob=1.0)
    k0, v0 = w.kv_cache[0, 0].clone().cpu(), w.kv_cache[1, 0].clone().cpu()
    cfg = CompressConfig(budget_blocks=budget, query_cache_len=16, use_redudancy=True,
                         lightning_redudancy=True, enable_pooling=True)
    dbg = compress_chunk(w.kv_cache[0], w.kv_cache[1], w.query_cache, None, w.query_ids,
                         w.block_tables, w.target_tables, w.compressed, cfg, return_debug=True)
    new_tables, ctx, nxt = K.update_tables(w.target_tables)
    # one new token per sequence goes to the first slot of the page after the budget
    g = torch.Generator().manual_seed(1)
    kn = torch.randn(3, Hkv, D, generator=g).to(torch.bfloat16)
    vn = torch.randn(3, Hkv, D, generator=g).to(torch.bfloat16)
    q = torch.randn(3, 1, Hq, D, generator=g).to(torch.bfloat16)
    K.store_kvcache(kn.to(dev), vn.to(dev), w.kv_cache[0, 0], w.kv_cache[1, 0], nxt)
    out = paged_decode_attention(q.to(dev), w.kv_cache[0, 0], w.kv_cache[1, 0], ctx, new_tables).cpu()
    torch.cuda.synchronize()
    assert ctx.cpu().tolist() == [budget * BS + 1] * 3
    keep = dbg["keep"].cpu()[0]                      # [B,Hkv,NB,BS]
    plain = w.tables_plain.cpu()
    for b in range(3):
        for h in range(Hkv):
            idx = keep[b, h].flatten().nonzero().flatten()
            pages = plain[b][idx // BS].long()
            kk = torch.cat([k0[pages, idx % BS, h], kn[b, h][None]]).float()
            vv = torch.cat([v0[pages, idx % BS, h], vn[b, h][None]]).float()
            G = Hq // Hkv
            qq = q[b, 0, h * G:(h + 1) * G].float()
            p = torch.softmax(qq @ kk.t() * D ** -0.5, dim=-1)
            ref = p @ vv
            got = out[b, 0, h * G:(h + 1) * G].float()
            assert (got - ref).abs().max() <= 2e-2 * ref.abs().max()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_varlen_prefill_long_ragged(dtype):
    """Several 64-key tiles, ragged lengths around tile and page boundaries, GQA group of 4."""
    from oracle import zipage_oracle as O
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    Hq, Hkv, D = 8, 2, 128
    g = torch.Generator().manual_seed(11)
    lens = [1000, 63, 64, 65, 257, 1, 512]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    tot = int(cu[-1])
    q = torch.randn(tot, Hq, D, generator=g).to(dtype)
    k = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    v = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    ref = O.varlen_prefill_attention(q, k, v, cu, cu)
    out = varlen_prefill_attention(q.to(dev), k.to(dev), v.to(dev), max(lens), cu.to(dev), max(lens),
                                   cu.to(dev)).cpu()
    assert (out.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()


def test_async_compress_overlaps_decode_on_another_stream():
    """The overlap contract of async_step: compression of some sequences runs on the compress
    stream from a worker thread while the main thread decodes OTHER sequences on its own stream.
    Both results must equal the sequential ones (the library keeps no global state)."""
    import threading
    from zipage_b200.compress import CompressConfig
    from zipage_b200.engine.compressor import Compressor
    from zipage_b200.layers.attention import paged_decode_attention
    from zipage_b200.synthetic import make_compress_workload
    dev = torch.device("cuda:0")
    Hkv, Hq, budget = 2, 8, 2
    cfg = CompressConfig(budget_blocks=budget, query_cache_len=16, use_redudancy=True,
                         lightning_redudancy=True, enable_pooling=True)

    def make():
        return make_compress_workload(B=6, L=4, Hkv=Hkv, Hq=Hq, QCL=16, budget=budget, pages_per_seq=3,
                                      dtype=torch.bfloat16, device=dev, seed=3, spare_pages=0)
    w_seq, w_par = make(), make()
    tables = w_seq.tables_plain.cpu().tolist()
    # sequences 0-2 are compressed, sequences 3-5 are decoded meanwhile (disjoint pages)
    comp_tables, comp_targets = tables[:3], w_seq.target_tables.cpu().tolist()[:3]
    qids, flags = w_seq.query_ids.cpu().tolist()[:3], [True] * 3
    dec_table = w_seq.tables_plain[3:].contiguous()
    lens = torch.tensor([3 * BS, 2 * BS + 5, 700], dtype=torch.int32, device=dev)
    q = torch.randn(3, 1, Hq, 128, device=dev, dtype=torch.bfloat16)

    c1 = Compressor(w_seq.kv_cache, w_seq.query_cache, None, cfg, layer_stride=2)
    c1.compress_tables(comp_tables, comp_targets, qids, flags)
    ref = [paged_decode_attention(q, w_seq.kv_cache[0, l], w_seq.kv_cache[1, l], lens, dec_table) for l in range(4)]
    torch.cuda.synchronize()

    c2 = Compressor(w_par.kv_cache, w_par.query_cache, None, cfg, layer_stride=2)
    err = []

    def worker():
        try:
            c2.compress_tables(comp_tables, comp_targets, qids, flags)
        except Exception as e:  # noqa: BLE001
            err.append(e)
    th = threading.Thread(target=worker)
    run_stream = torch.cuda.Stream()
    th.start()
    with torch.cuda.stream(run_stream):
        got = [paged_decode_attention(q, w_par.kv_cache[0, l], w_par.kv_cache[1, l], lens, dec_table)
               for l in range(4) for _ in range(3)][::3]
    th.join()
    torch.cuda.synchronize()
    assert not err, err
    assert torch.equal(w_par.kv_cache, w_seq.kv_cache)
    for a, b in zip(got, ref):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_varlen_prefill_tcgen05_matches_mma_and_oracle(dtype):
    """The tcgen05 kernel against the mma.sync kernel and the oracle: dense with ragged lengths
    around the 128-key tile, and paged with a cached prefix (fewer queries than keys), whose last
    page holds NaN beyond the context (the kernel must not let masked keys leak into the output)."""
    from oracle import zipage_oracle as O
    from zipage_b200 import _lib
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    Hq, Hkv, D = 8, 2, 128
    g = torch.Generator().manual_seed(23)
    lens = [700, 127, 128, 129, 1, 385, 256]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    tot = int(cu[-1])
    q = torch.randn(tot, Hq, D, generator=g).to(dtype)
    k = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    v = torch.randn(tot, Hkv, D, generator=g).to(dtype)
    ref = O.varlen_prefill_attention(q, k, v, cu, cu).float()
    outs = {}
    for impl in ("simt", "tcgen05"):
        outs[impl] = varlen_prefill_attention(q.to(dev), k.to(dev), v.to(dev), max(lens), cu.to(dev), max(lens),
                                              cu.to(dev), impl=impl).float().cpu()
        assert (outs[impl] - ref).abs().max() <= 2e-2 * ref.abs().max(), impl
    assert (outs["simt"] - outs["tcgen05"]).abs().max() <= 1e-2 * ref.abs().max()
    # paged, prefix cached: queries are the last lq tokens of each sequence
    lens_k = [300, 1, 640, 517, 256]
    lens_q = [44, 1, 300, 5, 256]
    cuk = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    cuq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    P = sum((n + BS - 1) // BS for n in lens_k) + 2
    kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
    vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype)
    table = torch.full((len(lens_k), 3), -1, dtype=torch.int32)
    perm = torch.randperm(P, generator=g)
    pos = 0
    for b, lk in enumerate(lens_k):
        npg = (lk + BS - 1) // BS
        table[b, :npg] = perm[pos:pos + npg].to(torch.int32)
        pos += npg
    q2 = torch.randn(int(cuq[-1]), Hq, D, generator=g).to(dtype)
    ref2 = O.varlen_prefill_attention(q2, kc, vc, cuq, cuk, block_table=table).float()
    kd, vd = kc.to(dev), vc.to(dev)
    for b, lk in enumerate(lens_k):          # poison everything past the context in the last page
        if lk % BS:
            page = int(table[b, (lk - 1) // BS])
            kd[page, lk % BS:] = float("nan")
            vd[page, lk % BS:] = float("nan")
    for impl in ("simt", "tcgen05"):
        out2 = varlen_prefill_attention(q2.to(dev), kd, vd, max(lens_q), cuq.to(dev), max(lens_k), cuk.to(dev),
                                        block_table=table.to(dev), impl=impl).float().cpu()
        assert torch.isfinite(out2).all(), impl
        assert (out2 - ref2).abs().max() <= 2e-2 * ref2.abs().max(), impl
    torch.cuda.synchronize()
    assert _lib.device_error() == 0


def test_varlen_prefill_tcgen05_is_refused_where_it_cannot_run():
    from zipage_b200 import _lib
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    cu = torch.tensor([0, 5], dtype=torch.int32, device=dev)
    q = torch.randn(5, 4, 128, device=dev)                      # fp32
    with pytest.raises(_lib.ZipageError):
        varlen_prefill_attention(q, q[:, :2].contiguous(), q[:, :2].contiguous(), 5, cu, 5, cu, impl="tcgen05")
    out = varlen_prefill_attention(q, q[:, :2].contiguous(), q[:, :2].contiguous(), 5, cu, 5, cu)   # auto: fp32 kernel
    assert torch.isfinite(out).all()


def test_varlen_prefill_tcgen05_long_sequences_against_mma():
    """Config-5 sizes (4 x 4096 and 1 x 16384 tokens, 32 query / 8 KV heads): hundreds of key tiles
    per block, every ring stage and barrier phase wrapping many times; the mma.sync kernel is the
    reference at this size.  Also a property of causal attention: the first query attends to one key,
    so its output is exactly that key's value row."""
    from zipage_b200 import _lib
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    Hq, Hkv, D = 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(1)
    for S, B in [(4096, 4), (16384, 1)]:
        q = torch.randn(B * S, Hq, D, device=dev, dtype=torch.bfloat16, generator=g)
        k = torch.randn(B * S, Hkv, D, device=dev, dtype=torch.bfloat16, generator=g)
        v = torch.randn(B * S, Hkv, D, device=dev, dtype=torch.bfloat16, generator=g)
        cu = torch.arange(0, (B + 1) * S, S, device=dev, dtype=torch.int32)
        a = varlen_prefill_attention(q, k, v, S, cu, S, cu, impl="tcgen05").float()
        b = varlen_prefill_attention(q, k, v, S, cu, S, cu, impl="simt").float()
        torch.cuda.synchronize()
        assert _lib.device_error() == 0
        assert torch.isfinite(a).all()
        assert (a - b).abs().max() <= 1e-2 * b.abs().max()
        first = torch.arange(B, device=dev) * S
        want = v[first].float().repeat_interleave(Hq // Hkv, dim=1)   # query head h reads kv head h // G
        assert torch.equal(a[first], want)


def test_varlen_prefill_tcgen05_pages_of_128_keys():
    """Pages of 128 keys: pass 1 of the tcgen05 kernel falls back to 128-key tiles."""
    from oracle import zipage_oracle as O
    from zipage_b200 import _lib
    from zipage_b200.layers.attention import varlen_prefill_attention
    dev = torch.device("cuda:0")
    Hq, Hkv, D, bs = 4, 2, 128, 128
    g = torch.Generator().manual_seed(31)
    lens_k = [520, 128, 77, 1000]
    lens_q = [520, 3, 77, 200]
    cuk = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    cuq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    P = sum((n + bs - 1) // bs for n in lens_k) + 1
    kc = torch.randn(P, bs, Hkv, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(P, bs, Hkv, D, generator=g).to(torch.bfloat16)
    width = max((n + bs - 1) // bs for n in lens_k)
    table = torch.full((len(lens_k), width), -1, dtype=torch.int32)
    perm = torch.randperm(P, generator=g)
    pos = 0
    for b, lk in enumerate(lens_k):
        npg = (lk + bs - 1) // bs
        table[b, :npg] = perm[pos:pos + npg].to(torch.int32)
        pos += npg
    q = torch.randn(int(cuq[-1]), Hq, D, generator=g).to(torch.bfloat16)
    ref = O.varlen_prefill_attention(q, kc, vc, cuq, cuk, block_table=table).float()
    out = varlen_prefill_attention(q.to(dev), kc.to(dev), vc.to(dev), max(lens_q), cuq.to(dev), max(lens_k),
                                   cuk.to(dev), block_table=table.to(dev), impl="tcgen05").float().cpu()
    torch.cuda.synchronize()
    assert _lib.device_error() == 0
    assert (out - ref).abs().max() <= 2e-2 * ref.abs().max()
