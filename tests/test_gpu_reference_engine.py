"""Greedy decode through the reference ENGINE: 256 steps across a compression, token by token.

The unmodified reference engine (zipage.ZipLLM.generate from baseline/_ref: scheduler, block
manager, model runner, Qwen3 model) runs a seeded random-init Qwen3-shaped model several times on
the same uniform-random prompts, with argmax in place of its sampler (the reference's sampler is
an exponential race that no two implementations reproduce, and its SamplingParams refuses
temperature 0):
  reference  as it is (Triton kernels, flash-attn), free running;
  kernels    with zipage_b200.kernel bound at the import sites of model_runner.py;
  full       with the Attention layer (cache stores, prefill and decode attention) bound as well;
  graph      with, on top of that, the decode forward replayed as CUDA graphs over this library's
             decoder blocks (device-built step state, fused q/k norm + rope + cache stores);
  native     with, on top of that, the engine's Scheduler / Sequence replaced by the native host
             control plane (the runner's decode inputs come from one array call).
A random-init model has near-flat logits, so two correct bf16 implementations that differ in the
last bit of one attention output — or that keep a different one of two keys tied at the top-k cut
— diverge for good at the first near-tie of the arg-max; a free-running comparison then says
nothing about the steps after it.  The bound runs are therefore teacher-forced on the reference's
tokens (same caches, same positions, same compressions at the same steps) while their own arg-max
is recorded at every step.  Checked for every bound run:
  * the own arg-max equals the reference's token at EVERY step whose top-2 logit margin (in the
    reference run) exceeds 2e-2 of the logit spread — the bf16 tolerance of the path;
  * the number of steps below that margin, the number of differing tokens and the length of the
    identical prefix of every sequence (how far a free run would have agreed) are printed.
Skipped with the reason when the reference, Triton or flash-attn is not usable on the machine.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ref_binding as RB

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
STEPS = 256


def _run(mode, out, extra=()):
    cmd = [sys.executable, str(ROOT / "tests" / "ref_engine.py"), "--mode", mode, "--out", str(out),
           "--greedy", "--lightning", "--pooling", "--requests", "4", "--prompt-len", "600",
           "--max-tokens", str(STEPS), "--budget", "2", "--qcl", "16", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if r.returncode != 0:
        tail = (r.stdout[-1500:] + r.stderr[-3000:])
        if mode == "reference":
            pytest.skip("the reference engine does not start on this machine: " + tail[-600:])
        raise AssertionError(f"engine run [{mode}] failed:\n{tail}")
    return json.loads(Path(out).read_text())


def test_greedy_256_steps_through_the_reference_engine(tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    ok, why = RB.reference_available()
    if not ok:
        pytest.skip(why)
    ref = _run("reference", tmp_path / "ref.json")
    assert all(len(t) == STEPS for t in ref["tokens"])
    # every sequence was compressed on the way (600-token prompt, budget of 2 pages: at length 769)
    assert ref["engine_time_record"].get("compress_sum", 0) > 0
    n_req = len(ref["tokens"])

    def compare(run, label):
        assert run["tokens"] == ref["tokens"]          # teacher forcing fed the reference's tokens back
        assert len(run["steps"]) == len(ref["steps"])
        total = mism = near = unexplained = 0
        prefix = [None] * n_req
        count = [0] * n_req
        for a, b in zip(ref["steps"], run["steps"]):
            assert len(a["tokens"]) == n_req        # one prefill batch, then every decode step holds all requests
            for i, (ta, tb, m, s) in enumerate(zip(a["tokens"], b["tokens"], a["margin"], a["spread"])):
                total += 1
                near += m <= 2e-2 * s
                if ta != tb:
                    mism += 1
                    unexplained += m > 2e-2 * s
                    if prefix[i] is None:
                        prefix[i] = count[i]
                count[i] += 1
        prefix = [STEPS if p is None else p for p in prefix]
        print(f"{label}: {total} sampled tokens, own arg-max differs on {mism}, {unexplained} of them at a margin "
              f"above 2e-2 of the logit spread ({near} steps are below it); identical prefix per sequence {prefix} "
              f"of {STEPS}")
        assert unexplained == 0
        assert mism <= 0.05 * total
        return prefix

    forced = ("--force", str(tmp_path / "ref.json"))
    ker = _run("kernels", tmp_path / "ker.json", forced)
    prefix = compare(ker, "compression kernels bound")
    # before the first compression (step 169 of the 600-token prompts) nothing of this library has run
    assert min(prefix) >= 169
    full = _run("full", tmp_path / "full.json", forced)
    compare(full, "compression kernels and attention layer bound")
    graph = _run("graph", tmp_path / "graph.json", forced)
    compare(graph, "decode step as CUDA graphs over this library's blocks")
    native = _run("native", tmp_path / "native.json", forced)
    compare(native, "the same with the native scheduler and page manager in place of the engine's")
    # same requests, same tokens fed back: the native scheduler took the same decisions
    assert native["engine_time_record"].get("compress_reqs") == graph["engine_time_record"].get("compress_reqs")
