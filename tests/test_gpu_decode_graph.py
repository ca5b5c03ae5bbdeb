"""The decode step replayed as a CUDA graph against the same step run launch by launch.

The graph's inputs are device state only (token counts, block tables, query ids); the number of
window-query rows written changes from step to step without a re-capture.
"""
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu

CFG = SimpleNamespace(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                      intermediate_size=1024, hidden_act="silu", rms_norm_eps=1e-6, vocab_size=1000,
                      num_hidden_layers=3, max_position_embeddings=4096, rope_theta=1e6)
QCL, BS = 32, 256


def _gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _model(dev):
    from zipage_b200.layers.qwen3_block import Qwen3Model
    torch.manual_seed(5)
    m = Qwen3Model(CFG)
    for p in m.parameters():
        if p.dim() == 1:   # norm weights near 1, as trained models have them
            p.data = 1.0 + 0.1 * torch.randn_like(p)
    return m.to(dev).to(torch.bfloat16).eval()


def _state(dev, n_seq, pages):
    """Sequences of 2-4 pages; some sit just below, some inside the observation window of their
    last page, one starts a fresh page in the second step."""
    g = torch.Generator().manual_seed(11)
    lens = [2, 3, 4, 2, 3][:n_seq]
    last = [BS - QCL - 1, BS - 3, 17, BS - 1, BS - QCL][:n_seq]   # tokens in the last page before the fed one
    perm = torch.randperm(pages, generator=g).tolist()
    tables, it = [], iter(perm)
    for n in lens:
        tables.append([next(it) for _ in range(n)])
    num_tokens = [(n - 1) * BS + l + 1 for n, l in zip(lens, last)]
    qids = [3, 0, -1, 5, 1][:n_seq]
    spare = [next(it) for _ in range(n_seq)]
    return tables, num_tokens, qids, spare


def _tensors(dev, tables, num_tokens, qids):
    w = max(len(t) for t in tables)
    return (torch.tensor([t + [-1] * (w - len(t)) for t in tables], dtype=torch.int32, device=dev),
            torch.tensor(num_tokens, dtype=torch.int32, device=dev),
            torch.tensor(qids, dtype=torch.int32, device=dev))


def _advance(tables, num_tokens, spare):
    """What the scheduler does between steps: one more token, a new page when the last is full."""
    for i in range(len(tables)):
        if num_tokens[i] % BS == 0:
            tables[i].append(spare[i])
        num_tokens[i] += 1


def _run_steps(runner, dev, kv, qc, snap, n_seq, steps, eager):
    kv.copy_(snap[0]); qc.copy_(snap[1])
    tables, num_tokens, qids, spare = _state(dev, n_seq, kv.shape[2])
    g = torch.Generator().manual_seed(3)
    outs = []
    for _ in range(steps):
        ids = torch.randint(0, CFG.vocab_size, (n_seq,), generator=g).to(dev)
        t, n, q = _tensors(dev, tables, num_tokens, qids)
        outs.append(runner.run(ids, n, t, q, eager=eager).clone())
        _advance(tables, num_tokens, spare)
    torch.cuda.synchronize()
    return outs, kv.clone(), qc.clone()


@pytest.mark.parametrize("n_seq", [5, 3])
def test_graph_replay_equals_eager_steps(n_seq):
    """n_seq = 5 fills no bucket exactly (8 is used), n_seq = 3 uses the bucket of 4: the padding
    rows must leave the caches untouched."""
    from zipage_b200 import _lib
    from zipage_b200.engine.decode_graph import DecodeGraphRunner
    dev = _gpu()
    model = _model(dev)
    pages = 24
    kv = (0.5 * torch.randn(2, CFG.num_hidden_layers, pages, BS, CFG.num_key_value_heads, CFG.head_dim,
                            device=dev)).to(torch.bfloat16)
    qc = torch.zeros(CFG.num_hidden_layers, 8, QCL, CFG.num_attention_heads, CFG.head_dim,
                     dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    snap = (kv.clone(), qc.clone())
    runner = DecodeGraphRunner(model, CFG.hidden_size, max_bs=8, max_num_blocks=6, query_cache_len=QCL,
                               device=dev)
    runner.capture()
    assert torch.equal(kv, snap[0]) and torch.equal(qc, snap[1]), "capture wrote to the caches"
    steps = 4
    eo, ekv, eqc = _run_steps(runner, dev, kv, qc, snap, n_seq, steps, eager=True)
    go, gkv, gqc = _run_steps(runner, dev, kv, qc, snap, n_seq, steps, eager=False)
    for a, b in zip(eo, go):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b)
    assert torch.equal(ekv, gkv) and torch.equal(eqc, gqc)
    assert not torch.equal(ekv, snap[0]) and not torch.equal(eqc, snap[1])
    # (the number of window rows written differs from step to step: a sequence enters its window
    # in the second step, two leave it when they start a new page)
    assert _lib.device_error() == 0


def test_eager_step_matches_fp32_model():
    """Wiring check of the blocks against the same network in plain fp32 torch over the gathered
    keys: positions, slots, context lengths and the window rows all enter the result."""
    from oracle import step_ops_oracle as S
    from zipage_b200.engine.decode_graph import DecodeGraphRunner
    dev = _gpu()
    model = _model(dev)
    pages, n_seq = 24, 5
    Hq, Hkv, D, L = CFG.num_attention_heads, CFG.num_key_value_heads, CFG.head_dim, CFG.num_hidden_layers
    kv = (0.5 * torch.randn(2, L, pages, BS, Hkv, D, device=dev)).to(torch.bfloat16)
    qc = torch.zeros(L, 8, QCL, Hq, D, dtype=torch.bfloat16, device=dev)
    model.bind_caches(kv, qc)
    kv0 = kv.clone()
    runner = DecodeGraphRunner(model, CFG.hidden_size, max_bs=8, max_num_blocks=6, query_cache_len=QCL, device=dev)
    tables, num_tokens, qids, _ = _state(dev, n_seq, pages)
    ids = torch.randint(0, CFG.vocab_size, (n_seq,), generator=torch.Generator().manual_seed(3)).to(dev)
    t, n, q = _tensors(dev, tables, num_tokens, qids)
    got = runner.run(ids, n, t, q, eager=True).float().cpu()

    sd = {k: v.float().cpu() for k, v in model.state_dict().items()}
    cos_sin = S.rope_cos_sin_cache(D, CFG.max_position_embeddings, CFG.rope_theta)
    kvc = kv0.float().cpu()
    pos = torch.tensor([x - 1 for x in num_tokens])

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + CFG.rms_norm_eps) * w

    h = sd["embed_tokens.weight"][ids.cpu()]
    res = None
    want_q_rows = {}
    for l in range(L):
        pre = f"layers.{l}."
        res = h if res is None else h + res
        x = norm(res, sd[pre + "input_layernorm.weight"])
        qkv = x @ sd[pre + "self_attn.qkv_proj.weight"].T
        qh = norm(qkv[:, : Hq * D].view(n_seq, Hq, D), sd[pre + "self_attn.q_norm.weight"])
        kh = norm(qkv[:, Hq * D: (Hq + Hkv) * D].view(n_seq, Hkv, D), sd[pre + "self_attn.k_norm.weight"])
        vh = qkv[:, (Hq + Hkv) * D:].view(n_seq, Hkv, D)
        cos, sin = cos_sin[pos].unsqueeze(1).chunk(2, dim=-1)
        qh, kh = S.apply_rotary_emb(qh, cos, sin), S.apply_rotary_emb(kh, cos, sin)
        o = torch.zeros(n_seq, Hq, D)
        for i in range(n_seq):
            nk = num_tokens[i] - 1
            keys = torch.cat([kvc[0, l, p] for p in tables[i]])[:nk]
            vals = torch.cat([kvc[1, l, p] for p in tables[i]])[:nk]
            keys, vals = torch.cat([keys, kh[i:i + 1]]), torch.cat([vals, vh[i:i + 1]])
            for hq in range(Hq):
                s = (keys[:, hq // (Hq // Hkv)] @ qh[i, hq]) * D ** -0.5
                o[i, hq] = torch.softmax(s, 0) @ vals[:, hq // (Hq // Hkv)]
        if l == 0:
            want_q_rows = {i: qh[i] for i in range(n_seq)}
        a = o.reshape(n_seq, Hq * D) @ sd[pre + "self_attn.o_proj.weight"].T
        res = a + res
        x = norm(res, sd[pre + "post_attention_layernorm.weight"])
        gu = x @ sd[pre + "mlp.gate_up_proj.weight"].T
        inter = CFG.intermediate_size
        h = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]) @ sd[pre + "mlp.down_proj.weight"].T
    want = norm(h + res, sd["norm.weight"])
    # bf16 activations through three layers against fp32: a few percent of the output scale
    err = (got - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item(), (err, want.abs().max().item())
    # the window rows of layer 0: sequences 1 and 3 are inside their window at this step
    for i, qid in enumerate(qids):
        last = num_tokens[i] - (len(tables[i]) - 1) * BS
        widx = last - (BS - QCL) - 1
        if qid != -1 and widx >= 0:
            row = qc[0, qid, widx].float().cpu()
            assert (row - want_q_rows[i]).abs().max() < 0.05 * want_q_rows[i].abs().max()
    assert int((qc[0].float().abs().sum(dim=(2, 3)) > 0).sum()) == sum(
        1 for i, qid in enumerate(qids)
        if qid != -1 and num_tokens[i] - (len(tables[i]) - 1) * BS > BS - QCL)
