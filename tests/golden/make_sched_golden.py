"""Writes tests/golden/sched_traces.json: the UNMODIFIED reference Scheduler / BlockManager /
Sequence (zipage/engine/scheduler.py, block_manager.py, sequence.py) driven through the seeded
scenarios of tests/sched_trace.py, one state checksum per step, folded into a running CRC that is
stored every 25 steps.  Also a few known answers of BlockManager.compute_hash.

usage: python tests/golden/make_sched_golden.py <reference source tree or installed copy>
"""
import json
import random
import sys
import zlib
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))


def fold(trace, every=25):
    """(number of steps, running CRC after every `every` steps and at the end, raised?)"""
    raised = bool(trace) and trace[-1] == "raised"
    steps = trace[:-1] if raised else trace
    run, marks = 0, []
    for i, c in enumerate(steps):
        run = zlib.crc32(c.to_bytes(4, "little"), run)
        if (i + 1) % every == 0:
            marks.append(run)
    marks.append(run)
    return {"steps": len(steps), "marks": marks, "raised": raised}


def main(ref_root):
    sys.path[:0] = [ref_root, str(Path(ref_root) / "third_party")]
    from zipage.engine.block_manager import BlockManager
    from zipage.engine.scheduler import Scheduler
    from zipage.engine.sequence import Sequence
    from zipage.sampling_params import SamplingParams
    import sched_trace as T

    out = {"traces": {}, "hashes": []}
    for name in T.SCENARIOS:
        out["traces"][name] = fold(T.run_trace(Scheduler, Sequence, SamplingParams, name, seed=0, max_steps=3000))
        print(name, out["traces"][name]["steps"], "steps")
    rng = random.Random(11)
    for n, with_prefix in [(256, False), (256, True), (1, False), (3, True), (31, False), (40, True), (512, True)]:
        toks = [rng.randrange(152000) for _ in range(n)]
        prefix = rng.getrandbits(64) if with_prefix else -1
        out["hashes"].append({"tokens": toks, "prefix": prefix, "hash": BlockManager.compute_hash(toks, prefix)})
    (HERE / "sched_traces.json").write_text(json.dumps(out))
    print("wrote", HERE / "sched_traces.json")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1])
