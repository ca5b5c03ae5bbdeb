"""Pin of the two attention rows against the library the reference calls.

The reference's decode and prefill attention are flash-attn calls
(zipage/layers/attention.py:79-103: flash_attn_varlen_func and flash_attn_with_kvcache); flash-attn
is a third-party dependency that is not part of the reference tree, so the CPU oracle for these
two rows is a restatement of softmax attention.  Where the installed flash-attn runs on the GPU at
hand, this file compares this library's kernels with it directly, on the reference's call shapes:
bf16 / fp16, 32 query / 8 KV heads of 128, pages of 256 keys, compressed tables of 9 pages.
Tolerance 2e-2 relative to the largest output (the bf16 tolerance of the path).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

BS = 256


def _flash():
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    try:
        import flash_attn
        from flash_attn import flash_attn_varlen_func, flash_attn_with_kvcache
    except Exception as e:  # not installed, or built for another torch
        pytest.skip(f"flash-attn cannot be imported here: {type(e).__name__}: {e}")
    # one tiny call decides whether its kernels run on this GPU
    try:
        q = torch.randn(1, 1, 8, 128, device="cuda", dtype=torch.bfloat16)
        kc = torch.randn(2, BS, 2, 128, device="cuda", dtype=torch.bfloat16)
        flash_attn_with_kvcache(q, kc, kc, cache_seqlens=torch.tensor([300], dtype=torch.int32, device="cuda"),
                                block_table=torch.tensor([[0, 1]], dtype=torch.int32, device="cuda"), causal=True)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"flash-attn {flash_attn.__version__} does not run on this GPU: {type(e).__name__}: {e}")
    return flash_attn_varlen_func, flash_attn_with_kvcache


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_decode_matches_flash_attn_with_kvcache(dtype):
    from zipage_b200.layers.attention import paged_decode_attention
    _, with_kvcache = _flash()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(3)
    B, Hq, Hkv, D, NB = 48, 32, 8, 128, 9
    P = B * NB + 5
    kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    table = torch.randperm(P, generator=g)[: B * NB].view(B, NB).to(torch.int32).to(dev)
    lens = torch.randint(8 * BS + 1, NB * BS + 1, (B,), generator=g).to(torch.int32)
    lens[0], lens[1], lens[2] = 1, BS, NB * BS          # one token, one full page, a full table
    table[0, 1:] = -1                                    # the reference pads short tables with -1
    lens = lens.to(dev)
    q = torch.randn(B, 1, Hq, D, generator=g).to(dtype).to(dev)
    scale = D ** -0.5
    want = with_kvcache(q, kc, vc, cache_seqlens=lens, block_table=table.clamp_min(0), softmax_scale=scale,
                        causal=True).float()
    got = paged_decode_attention(q, kc, vc, lens, table, scale).float()
    torch.cuda.synchronize()
    err = (got - want).abs().max().item() / want.abs().max().item()
    print(f"paged decode vs flash_attn_with_kvcache ({dtype}): max rel err {err:.2e}")
    assert err <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_varlen_prefill_matches_flash_attn_varlen_func(dtype):
    from zipage_b200.layers.attention import varlen_prefill_attention
    varlen, _ = _flash()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(5)
    Hq, Hkv, D = 32, 8, 128
    lens = [700, 1, 256, 1300, 45]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    tot = sum(lens)
    q = torch.randn(tot, Hq, D, generator=g).to(dtype).to(dev)
    k = torch.randn(tot, Hkv, D, generator=g).to(dtype).to(dev)
    v = torch.randn(tot, Hkv, D, generator=g).to(dtype).to(dev)
    scale = D ** -0.5
    want = varlen(q, k, v, max_seqlen_q=max(lens), cu_seqlens_q=cu, max_seqlen_k=max(lens), cu_seqlens_k=cu,
                  softmax_scale=scale, causal=True).float()
    for impl in ("tcgen05", "simt"):
        got = varlen_prefill_attention(q, k, v, max(lens), cu, max(lens), cu, scale, impl=impl).float()
        torch.cuda.synchronize()
        err = (got - want).abs().max().item() / want.abs().max().item()
        print(f"dense varlen prefill [{impl}] vs flash_attn_varlen_func ({dtype}): max rel err {err:.2e}")
        assert err <= 2e-2
    # prefix-cache form: keys from the pages (longer than the queries), bottom-right aligned causal mask
    NBs = 6
    klens = [1400, 300, 256 + 17]
    qlens = [120, 300, 17]
    B = len(klens)
    P = B * NBs + 2
    kc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    vc = torch.randn(P, BS, Hkv, D, generator=g).to(dtype).to(dev)
    table = torch.randperm(P, generator=g)[: B * NBs].view(B, NBs).to(torch.int32).to(dev)
    cuq = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev)
    cuk = torch.tensor([0] + list(torch.tensor(klens).cumsum(0)), dtype=torch.int32, device=dev)
    q2 = torch.randn(sum(qlens), Hq, D, generator=g).to(dtype).to(dev)
    want = varlen(q2, kc, vc, max_seqlen_q=max(qlens), cu_seqlens_q=cuq, max_seqlen_k=max(klens),
                  cu_seqlens_k=cuk, softmax_scale=scale, causal=True, block_table=table).float()
    got = varlen_prefill_attention(q2, kc, vc, max(qlens), cuq, max(klens), cuk, scale, block_table=table).float()
    torch.cuda.synchronize()
    err = (got - want).abs().max().item() / want.abs().max().item()
    print(f"paged varlen prefill vs flash_attn_varlen_func ({dtype}): max rel err {err:.2e}")
    assert err <= 2e-2
