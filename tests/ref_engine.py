"""Test / benchmark support: run the UNMODIFIED reference engine (zipage.ZipLLM from baseline/_ref)
on a synthetic Qwen3-shaped model, with or without this library bound at the reference's call sites.

    python tests/ref_engine.py --mode reference|kernels|full --out result.json [options]

Modes
  reference  the reference as it is: Triton kernels, flash-attn, torch.compile'd step ops
  kernels    zipage/engine/model_runner.py:19-27 import the compression kernels from zipage_b200.kernel
  full       `kernels` + the Attention layer (cache stores, prefill and decode attention) from
             zipage_b200.layers.attention, sharing the reference's Context module
  steps      `full` + RMSNorm and SiluAndMul of the decoder blocks from zipage_b200.layers.step_ops
              in place of the reference's torch.compile'd modules
  graph      `full` + the decode step as replayed CUDA graphs: the
             reference's scheduler, block manager, prefill, LM head and sampler stay; its decode
             forward (ModelRunner.run for decode batches) goes through DecodeGraphRunner over
             zipage_b200's Qwen3 blocks, which share the reference model's parameters and caches

There is no tokenizer or checkpoint offline, so the model directory is synthesised: a Qwen3
config.json, a word-level stub tokenizer (the engine only reads its eos / pad ids and decodes the
output), and seeded random safetensors in the checkpoint layout the reference's loader expects.
Prompts are uniform-random token ids.  `--greedy` replaces the sampler (an exponential race that is
not reproducible across implementations; zipage/layers/sampler.py:27-31) by argmax on both sides and
records the top-2 logit margin of every step; `--force FILE` additionally feeds the tokens of an
earlier run back (teacher forcing) while still recording this run's own argmax.

This file runs as a child process: the engine initialises torch.distributed and registers an exit
hook of its own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def make_model_dir(path: Path, layers, hidden, inter, hq, hkv, vocab, seed, device="cuda"):
    """config.json + stub tokenizer + seeded bf16 weights (one safetensors file per few layers)."""
    import torch
    from safetensors.torch import save_file
    path.mkdir(parents=True, exist_ok=True)
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden,
           "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": hq,
           "num_key_value_heads": hkv, "head_dim": 128, "hidden_act": "silu", "rms_norm_eps": 1e-6,
           "rope_theta": 1000000.0, "max_position_embeddings": 40960, "vocab_size": vocab,
           "tie_word_embeddings": False, "attention_bias": False, "torch_dtype": "bfloat16",
           "bos_token_id": 1, "eos_token_id": 1, "pad_token_id": 0}
    (path / "config.json").write_text(json.dumps(cfg))
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    words = {"<pad>": 0, "<eos>": 1}
    for i in range(2, vocab):
        words[f"t{i}"] = i
    tok = Tokenizer(WordLevel(words, unk_token="<pad>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(path / "tokenizer.json"))
    (path / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "pad_token": "<pad>",
         "unk_token": "<pad>", "model_max_length": 1000000}))
    (path / "special_tokens_map.json").write_text(json.dumps(
        {"eos_token": "<eos>", "pad_token": "<pad>", "unk_token": "<pad>"}))
    g = torch.Generator(device=device).manual_seed(seed)

    def rnd(*shape, std):
        return (torch.randn(*shape, generator=g, device=device) * std).to(torch.bfloat16).cpu()

    def ones(n):
        return (1.0 + 0.05 * torch.randn(n, generator=g, device=device)).to(torch.bfloat16).cpu()
    shard = {"model.embed_tokens.weight": rnd(vocab, hidden, std=1.0),
             "model.norm.weight": ones(hidden), "lm_head.weight": rnd(vocab, hidden, std=hidden ** -0.5)}
    n = 0
    for i in range(layers):
        p = f"model.layers.{i}."
        shard[p + "self_attn.q_proj.weight"] = rnd(hq * 128, hidden, std=hidden ** -0.5)
        shard[p + "self_attn.k_proj.weight"] = rnd(hkv * 128, hidden, std=hidden ** -0.5)
        shard[p + "self_attn.v_proj.weight"] = rnd(hkv * 128, hidden, std=hidden ** -0.5)
        shard[p + "self_attn.o_proj.weight"] = rnd(hidden, hq * 128, std=(hq * 128) ** -0.5)
        shard[p + "self_attn.q_norm.weight"] = ones(128)
        shard[p + "self_attn.k_norm.weight"] = ones(128)
        shard[p + "mlp.gate_proj.weight"] = rnd(inter, hidden, std=hidden ** -0.5)
        shard[p + "mlp.up_proj.weight"] = rnd(inter, hidden, std=hidden ** -0.5)
        shard[p + "mlp.down_proj.weight"] = rnd(hidden, inter, std=inter ** -0.5)
        shard[p + "input_layernorm.weight"] = ones(hidden)
        shard[p + "post_attention_layernorm.weight"] = ones(hidden)
        if (i + 1) % 4 == 0 or i == layers - 1:
            save_file(shard, str(path / f"model-{n:05d}.safetensors"))
            shard, n = {}, n + 1
    return path


def transformers_compat():
    """The reference reads `config.rope_theta` and spreads `config.rope_scaling` into its own rope
    initialiser (zipage/models/qwen3.py:129-130, zipage/layers/rotary_embedding.py:80-83), the
    layout of transformers 4.x.  transformers 5 moved both into `rope_parameters` (rope_theta reads
    None, rope_scaling holds {'rope_theta', 'rope_type'}), which makes the unmodified reference
    fail at start-up.  For a default (unscaled) rope the two attributes are put back the way the
    reference expects them; nothing of the reference is touched."""
    import zipage.config as zc
    real = zc.AutoConfig

    class _AutoConfig:
        @staticmethod
        def from_pretrained(*a, **k):
            c = real.from_pretrained(*a, **k)
            rp = dict(getattr(c, "rope_parameters", None) or {})
            if getattr(c, "rope_theta", None) is None and rp.get("rope_type", "default") == "default":
                c.rope_scaling = None
                c.rope_theta = rp.get("rope_theta", 1000000.0)
            return c
    zc.AutoConfig = _AutoConfig


def bind(mode):
    """Swap the reference's module-level names for this library's (INTEGRATION.md sections 1 and 3)."""
    if mode == "reference":
        return
    import zipage.engine.model_runner as mr
    from zipage_b200 import kernel as K
    for n in ["compress_kv", "compress_score", "attention_score", "raw_redudancy_score",
              "lightning_redudancy_score", "global_score", "window_mask", "topk_mask"]:
        setattr(mr, n, getattr(K, n))
    if mode in ("full", "steps", "graph", "native"):
        import zipage.layers.attention as ref_att
        import zipage.models.qwen3 as ref_qwen3
        import zipage.utils.context as ref_ctx
        import zipage_b200.layers.attention as our_att
        # The runner and the layer share one Context.  The reference runner fills the reference's
        # module; the graph runner of mode `graph` fills this library's: whichever holds a step.
        import zipage_b200.utils.context as our_ctx

        def shared_context():
            c = our_ctx.get_context()
            if c.is_prefill or c.context_lens is not None or c.slot_mapping is not None:
                return c
            return ref_ctx.get_context()
        our_att.get_context = shared_context
        ref_qwen3.Attention = our_att.Attention
        ref_att.Attention = our_att.Attention
    if mode == "steps":
        import zipage.models.qwen3 as ref_qwen3
        from zipage_b200.layers import step_ops
        ref_qwen3.RMSNorm = step_ops.RMSNorm
        ref_qwen3.SiluAndMul = step_ops.SiluAndMul


def bind_graph_decode(llm, max_bs, max_model_len, qcl):
    """ModelRunner.run for decode batches through DecodeGraphRunner (the reference's own graph
    branch, zipage/engine/model_runner.py:709-724, raises ValueError).  The blocks are
    zipage_b200.layers.qwen3_block.Qwen3Model with the reference model's parameter tensors (no
    copy) and the runner's caches."""
    import torch
    import zipage.engine.model_runner as mr
    from zipage_b200.engine.decode_graph import DecodeGraphRunner
    from zipage_b200.layers.qwen3_block import Qwen3Model
    runner = llm.model_runner
    hf = runner.config.hf_config
    inner = runner.model.model
    with torch.device("meta"):
        ours = Qwen3Model(hf)
    for name, p in inner.named_parameters():
        mod = ours
        *path, attr = name.split(".")
        for part in path:
            mod = getattr(mod, part)
        setattr(mod, attr, p)
    ours.eval()
    ours.bind_caches(runner.kv_cache, runner.query_cache)
    with torch.cuda.stream(runner.run_stream):
        dg = DecodeGraphRunner(ours, hf.hidden_size, max_bs=max_bs,
                               max_num_blocks=(max_model_len + 255) // 256 + 1, query_cache_len=qcl,
                               device="cuda")
        dg.capture()
    torch.cuda.synchronize()
    orig_run = mr.ModelRunner.run
    from zipage_b200.engine import scheduler as own
    native = isinstance(llm.scheduler, own.Scheduler)
    width = (max_model_len + 255) // 256 + 1
    if native:   # the scheduler fills pinned arrays for the whole batch in one call
        staged = {"input_ids": torch.empty(max_bs, dtype=torch.int32).pin_memory(),
                  "num_tokens": torch.empty(max_bs, dtype=torch.int32).pin_memory(),
                  "query_ids": torch.empty(max_bs, dtype=torch.int32).pin_memory(),
                  "block_tables": torch.empty(max_bs, width, dtype=torch.int32).pin_memory()}
        views = {k: v.numpy() for k, v in staged.items()}

    def run(self, seqs, is_prefill):
        if is_prefill or len(seqs) > max_bs:
            return orig_run(self, seqs, is_prefill)
        with torch.cuda.stream(self.run_stream), torch.inference_mode():
            pin = lambda data, dt: torch.tensor(data, dtype=dt, pin_memory=True).cuda(non_blocking=True)
            if native:
                n = len(seqs)
                d = llm.scheduler.decode_inputs(llm.scheduler._handles_of(seqs), table_width=width, out=views)
                ids = staged["input_ids"][:n].cuda(non_blocking=True)
                ntok = staged["num_tokens"][:n].cuda(non_blocking=True)
                qids = staged["query_ids"][:n].cuda(non_blocking=True)
                tables = staged["block_tables"][:n, :d["widest"]].cuda(non_blocking=True)
            else:
                ids = pin([s.last_token for s in seqs], torch.int64)
                ntok = pin([len(s) for s in seqs], torch.int32)
                qids = pin([s.query_id for s in seqs], torch.int32)
                tables = self.prepare_block_tables(seqs)
            past, temps = self.prepare_sample(seqs)
            hidden = dg.run(ids, ntok, tables, qids)
            logits = self.model.compute_logits(hidden)
            return self.sampler(logits, temps, past).tolist()
    mr.ModelRunner.run = run
    return dg


def bind_native_scheduler():
    """The engine's Scheduler / Sequence replaced by this library's native ones (same constructor
    argument, calls and attributes): zipage/engine/zipage_engine.py:12-13 imports the names the
    engine uses, so binding them there before ZipLLM is built is the whole swap."""
    import zipage.engine.zipage_engine as ze
    from zipage_b200.engine import scheduler as own
    ze.Scheduler = own.Scheduler
    ze.Sequence = own.Sequence


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="reference", choices=["reference", "kernels", "full", "steps", "graph", "native"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--model-dir", default="/tmp/zp_synth_model")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=8)
    ap.add_argument("--hkv", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--requests", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=600)
    ap.add_argument("--prompt-len-max", type=int, default=0, help="if > prompt-len: uniform in [min, max]")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--budget", type=int, default=2, help="max_cache_blocks_per_seq")
    ap.add_argument("--qcl", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--greedy", action="store_true")
    ap.add_argument("--force", default="")
    ap.add_argument("--lightning", action="store_true")
    ap.add_argument("--exact", action="store_true")
    ap.add_argument("--global-score", action="store_true")
    ap.add_argument("--pooling", action="store_true")
    ap.add_argument("--async-compress", action="store_true")
    ap.add_argument("--prefix-cache", action="store_true")
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--port", type=int, default=2391)
    ap.add_argument("--gpu-mem", type=float, default=0.85)
    ap.add_argument("--warmup-requests", type=int, default=0,
                    help="an untimed generate() of that many requests first (Triton / Inductor compile, "
                         "allocator warm-up); the time records are cleared after it")
    args = ap.parse_args()

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(REF))
    import torch
    md = Path(args.model_dir)
    tag = f"{args.layers}-{args.hidden}-{args.inter}-{args.hq}-{args.hkv}-{args.vocab}-{args.seed}"
    if not (md / "tag").exists() or (md / "tag").read_text() != tag:
        if md.exists():
            import shutil
            shutil.rmtree(md)
        make_model_dir(md, args.layers, args.hidden, args.inter, args.hq, args.hkv, args.vocab, args.seed)
        (md / "tag").write_text(tag)

    transformers_compat()
    bind(args.mode)
    if args.mode == "native":
        bind_native_scheduler()
    import zipage.layers.sampler as ref_sampler
    from zipage.llm import ZipLLM
    from zipage.sampling_params import SamplingParams

    steps = []          # per sampler call: own argmax, top-2 margin, logit spread
    forced = json.loads(Path(args.force).read_text())["steps"] if args.force else None
    if args.greedy:
        def forward(self, logits, temperatures, past_tokens=None):
            lf = logits.float()
            top = lf.topk(2, dim=-1)
            own = top.indices[:, 0]
            steps.append({"tokens": own.tolist(),
                          "margin": (top.values[:, 0] - top.values[:, 1]).tolist(),
                          "spread": (lf.max(dim=-1).values - lf.min(dim=-1).values).tolist()})
            if forced is not None:
                return torch.tensor(forced[len(steps) - 1]["tokens"], device=logits.device)
            return own
        ref_sampler.Sampler.forward = forward

    llm = ZipLLM(str(md), port=args.port, max_num_seqs=args.max_num_seqs, max_model_len=args.max_model_len,
                 max_num_batched_tokens=max(32768, args.max_model_len), gpu_memory_utilization=args.gpu_mem,
                 max_cache_blocks_per_seq=args.budget, query_cache_len=args.qcl,
                 use_redudancy=args.lightning or args.exact, lightning_redudancy=args.lightning,
                 redudancy_lambda=0.5, use_global_score=args.global_score, enable_pooling=args.pooling,
                 enable_async_compress=args.async_compress, enable_prefix_cache=args.prefix_cache)
    if args.mode in ("graph", "native"):
        bind_graph_decode(llm, min(args.max_num_seqs, max(args.requests, args.warmup_requests, 16)),
                          args.max_model_len, args.qcl)
    g = torch.Generator().manual_seed(args.seed + 1)
    prompts = []
    for _ in range(args.requests):
        n = args.prompt_len if args.prompt_len_max <= args.prompt_len else \
            int(torch.randint(args.prompt_len, args.prompt_len_max + 1, (1,), generator=g))
        prompts.append(torch.randint(2, args.vocab, (n,), generator=g).tolist())
    sp = SamplingParams(temperature=args.temperature, max_tokens=args.max_tokens, ignore_eos=True)
    if args.warmup_requests > 0:
        # long enough to cross one compression: prompt of budget+1 full pages minus a few tokens
        wl = (args.budget + 1) * 256 - 4
        wp = [torch.randint(2, args.vocab, (wl,), generator=g).tolist() for _ in range(args.warmup_requests)]
        llm.generate(wp, SamplingParams(temperature=args.temperature, max_tokens=8, ignore_eos=True), use_tqdm=True)
        llm.time_record.clear()
        llm.model_runner.time_record.clear()
        steps.clear()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp, use_tqdm=True)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    tr = dict(llm.time_record)
    gen = sum(len(o["token_ids"]) for o in outs)
    decode_tokens = gen - len(outs)   # the first token of every request comes out of the prefill step
    decode_s = tr.get("decode_sum", 0.0) + tr.get("compress_sum", 0.0)
    res = {"mode": args.mode, "requests": len(prompts), "generated_tokens": gen, "wall_s": wall,
           "engine_time_record": {k: float(v) for k, v in tr.items()},
           "runner_time_record": {k: float(v) for k, v in llm.model_runner.time_record.items()},
           "decode_tokens": decode_tokens,
           "decode_tok_per_s": decode_tokens / decode_s if decode_s > 0 else None,
           "decode_tok_per_s_excluding_compress": decode_tokens / tr["decode_sum"] if tr.get("decode_sum") else None,
           "prefill_tok_per_s": sum(len(p) for p in prompts) / tr["prefill_sum"] if tr.get("prefill_sum") else None,
           "max_concurrency": int(llm.model_runner.config.max_concurrency),
           "num_kvcache_blocks": int(llm.model_runner.config.num_kvcache_blocks),
           "tokens": [o["token_ids"] for o in outs], "steps": steps}
    Path(args.out).write_text(json.dumps(res))
    print(json.dumps({k: v for k, v in res.items() if k not in ("tokens", "steps")}))


if __name__ == "__main__":
    main()
