"""A device-side timeline of the kernels of one step: where a decoding step's time goes between its kernels.

A decoding step is a chain of dependent kernels launched as programmatic dependents: each does what does not
depend on its predecessor (weights, earlier keys) before it waits for it.  Host-side timers and profilers that
serialise kernels cannot see that overlap.  In the "timeline" build of the kernels (`csrc/build.py` FLAVORS,
`csrc/launch.cuh`) every block stamps the device's global timer when it starts, when its wait for the preceding
kernel returns and when it ends; block 0 can leave up to five more marks.  This module points the kernels at a
buffer, runs steps and turns the records into a table:

    python -m machserve_b200.timeline --shape qwen2.5-0.5b --batch 8 --context 2048 [--layers 4]
    python -m machserve_b200.timeline --model DIR --batch 4 --context 300

The reference has two counterparts: per-layer event triples behind MACH_STEP_PROFILE
(crates/mach-model/src/batched.rs:197-266 of gqf2008/machserve) and clock stamps inside its small-row kernels behind
a nullable pointer (crates/mach-model/src/kernels.rs:2671-2694); this is the second kind.

Only kernels that carry the hooks appear (the small-row products and the decoding attention: the kernels of a
decoding step of up to 16 rows).  The plain build has no hooks and pays nothing for them.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
from collections import defaultdict
from typing import Dict, List

# the files whose kernels carry hooks: each has a setter `ms_timeline_set_<unit>` in the timeline build
UNITS = ("gemm_small_m", "attention_decode_cluster", "attention_decode_cluster_rope")
# kernel ids as the hooks give them: 100 + 10 * epilogue + row scaling for the products, 200 for the attention
NAMES = {100: "product -> bfloat16", 101: "product / rms -> bfloat16", 110: "product -> float32", 111: "product / rms -> float32",
         120: "gate/up, SiLU-mul", 121: "gate/up / rms, SiLU-mul", 130: "product + residual, row sums", 200: "decoding attention"}
RECORD_WORDS, MAX_RECORDS = 10, 4096


class Timeline:
    """The buffer the kernels write to, and its reading.  Needs `ops.use_flavor("timeline")` before the first kernel call."""

    def __init__(self, device="cuda:0"):
        import torch

        from . import ops

        self.torch = torch
        lib = ops.lib()
        self.buf = torch.zeros(1 + MAX_RECORDS * RECORD_WORDS, dtype=torch.int64, device=device)
        for unit in UNITS:
            fn = getattr(lib, f"ms_timeline_set_{unit}", None)
            if fn is None:
                raise RuntimeError("this build of the kernels has no timeline hooks: call ops.use_flavor('timeline') first")
            if fn(ctypes.c_void_p(self.buf.data_ptr())) != 0:
                raise RuntimeError(f"could not hand the timeline buffer to {unit}")
        self.reset()

    def reset(self) -> None:
        rec = self.buf[1:].view(MAX_RECORDS, RECORD_WORDS)
        rec[:, 0] = 0
        rec[:, 1:4] = -1  # all ones: the largest unsigned value, for the minima the blocks take
        rec[:, 4:] = 0
        self.buf[0] = 0
        self.torch.cuda.synchronize()

    def records(self) -> List[Dict]:
        """One record per launch since `reset`, in launch order; times in microseconds from the first start."""
        self.torch.cuda.synchronize()
        n = min(int(self.buf[0].item()), MAX_RECORDS)
        raw = self.buf[1:].view(MAX_RECORDS, RECORD_WORDS)[:n].cpu().tolist()
        if not raw:
            return []
        t0 = raw[0][1]
        out, prev_end = [], None
        for r in raw:
            start, waited, first_end, last_end = ((x - t0) / 1000.0 for x in r[1:5])
            out.append({"id": int(r[0]), "kernel": NAMES.get(int(r[0]), str(int(r[0]))), "start": start, "wait_returned": waited,
                        "first_end": first_end, "last_end": last_end,
                        "hand_over": None if prev_end is None else waited - prev_end,  # predecessor's end -> this wait's return
                        "after_wait": last_end - waited, "marks": [x / 1000.0 for x in r[5:10]]})
            prev_end = last_end
        return out


def summarize(records: List[Dict]) -> str:
    if not records:
        return "no records (did the step run kernels that carry hooks?)"
    lines = [f"{len(records)} launches; from the first start to the last end {records[-1]['last_end']:.1f} us",
             f"{'kernel':34s} {'launches':>8s} {'early start':>12s} {'hand-over':>10s} {'after wait':>11s}   marks of block 0 after its wait (us)"]
    agg = defaultdict(list)
    for r in records[1:]:
        agg[r["kernel"]].append(r)
    for name, rs in agg.items():
        mean = lambda f: sum(f(r) for r in rs) / len(rs)
        marks = [mean(lambda r, i=i: r["marks"][i]) for i in range(5)]
        lines.append(f"{name:34s} {len(rs):8d} {mean(lambda r: r['wait_returned'] - r['start']):12.2f} {mean(lambda r: r['hand_over']):10.2f} "
                     f"{mean(lambda r: r['after_wait']):11.2f}   " + " ".join(f"{m:.2f}" for m in marks if m > 0))
    lines.append("early start: how long before its wait returned the kernel's first block was running (its weights and keys on their way);")
    lines.append("hand-over: from the end of the kernel before to the return of this kernel's wait; after wait: from there to its last block's end.")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None, help="a model folder; else random weights of --shape")
    ap.add_argument("--shape", default="qwen2.5-0.5b")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--json", action="store_true", help="print the records as JSON lines instead of the table")
    a = ap.parse_args(argv)

    import numpy as np
    import torch

    from . import ops

    ops.use_flavor("timeline")
    from .config import config_from_json, load_config
    from .engine import ModelRunner, StepEntry

    max_seq = a.context + 64
    kw = dict(dtype="bf16", page_size=64, num_pages=a.batch * (-(-max_seq // 64)) + 8, max_requests=a.batch,
              max_step_tokens=max(2048, a.context) + a.batch, max_seq_len=max_seq)
    if a.model:
        runner = ModelRunner.from_model_dir(a.model, **kw)
        vocab = load_config(a.model).model_spec().vocab_size
    else:
        sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parent.parent))
        import bench

        raw = dict(bench.SHAPES[a.shape])
        if a.layers:
            raw["num_hidden_layers"] = a.layers
        runner = ModelRunner.from_random(config_from_json(raw), seed=0, on_device=True, **kw)
        vocab = raw["vocab_size"]
    rng = np.random.default_rng(0)
    for r in range(a.batch):
        toks = rng.integers(0, vocab, size=a.context)
        for at in range(0, a.context, 2048):
            runner.step([StepEntry(r, toks[at : at + 2048].tolist(), [])])
    tl = Timeline(runner.device)
    step = lambda: runner.step([StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in range(a.batch)])
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    tl.reset()
    step()
    recs = tl.records()
    if a.json:
        for r in recs:
            print(json.dumps(r))
    else:
        print(f"one decoding step, batch {a.batch}, {a.context}-token contexts")
        print(summarize(recs))
    return 0


if __name__ == "__main__":
    sys.exit(main())
