"""The command line: `mach generate | replay | random | bench | timeline`.

The reference is configured by environment variables of its server
(crates/mach-server/src/main.rs:7-37 of gqf2008/machserve); the options here carry
their names and meanings: --capacity (MACH_CAPACITY, 64), --prefill-rows
(MACH_PREFILL_ROWS, 512), --dtype (MACH_DTYPE: f32, or bf16 where it has f16),
--tpp (MACH_TPP, tokens per page, 64), --max-seq (MACH_MAX_SEQ).  Sampling options
are the fields of its SamplingParams.  The library itself reads no environment, except for where to find
nvcc (NVCC, CUDA_HOME) and where to put the built kernels when the tree cannot be written
(MACHSERVE_B200_BUILD_DIR), both in csrc/build.py.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "float32"])
    p.add_argument("--capacity", type=int, default=64, help="most requests running at a time")
    p.add_argument("--prefill-rows", type=int, default=512, help="most prompt tokens per step")
    p.add_argument("--tpp", type=int, default=64, help="tokens per cache page")
    p.add_argument("--max-seq", type=int, default=None, help="context limit (default: the model's, at most 8192)")
    p.add_argument("--num-pages", type=int, default=None, help="pages per cache group (default: capacity x max-seq)")


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(a) -> int:
    from .engine import Engine
    from .sampling import SamplingParams

    eng = Engine(a.model, a.dtype, a.capacity, a.prefill_rows, a.tpp, a.max_seq, a.num_pages)
    print(json.dumps({"memory": eng.runner.memory_plan()}), file=sys.stderr)
    params = SamplingParams(a.temperature, a.top_k, a.top_p, a.seed, a.presence_penalty, a.frequency_penalty, a.top_logprobs)
    eos = a.eos if a.eos is not None else getattr(eng.config, "eos_token_id", None)
    t0 = time.time()
    ids = [eng.add(_ids(p), a.max_new, None if a.ignore_eos else eos, [_ids(s) for s in a.stop], None, params)
           for p in a.prompt_ids]
    while not eng.all_done():
        eng.step()
    dt = time.time() - t0
    for sid in ids:
        rec = {"id": sid, "tokens": eng.generated(sid), "finish_reason": eng.finish_reason(sid)}
        if a.top_logprobs:
            rec["logprobs"] = [round(x, 5) for x in eng.generated_logprobs(sid)]
            rec["top_logprobs"] = [[(t, round(lp, 5)) for t, lp in tops] for tops in eng.generated_top_logprobs(sid)]
        print(json.dumps(rec))
    print(json.dumps({"seconds": round(dt, 4), **eng.counters}), file=sys.stderr)
    return 0


def cmd_replay(a) -> int:
    import os

    from .engine.replay import make_replay_runner, replay_record

    os.makedirs(a.out, exist_ok=True)
    runner = make_replay_runner(a.model, a.dtype, a.max_tokens, a.page_size)
    src = open(a.trace) if a.trace != "-" else sys.stdin
    for line in src:
        if not line.strip():
            continue
        rec = json.loads(line)
        out = replay_record(runner, rec)
        if out is not None:
            out.tofile(os.path.join(a.out, f"{rec['step']}.f32"))
        print(f"done {rec['step']}", flush=True)
    return 0


def cmd_random(a) -> int:
    import torch

    from .config import config_from_json
    from .weights import write_random_model

    cfg = config_from_json(json.load(open(a.config)))
    dtype = torch.float32 if a.dtype in ("f32", "float32") else torch.bfloat16
    out = write_random_model(cfg, a.out, a.seed, dtype, a.weight_std, a.bias_std, a.norm_std)
    print(out)
    return 0


def cmd_bench(a) -> int:
    """Decode and prefill throughput of a shape with random weights, or of a model folder: the repository's bench.py
    with its options under this command's names."""
    import os
    import runpy
    from pathlib import Path

    batches = [int(b) for b in a.batch.split(",") if b.strip()]
    argv = ["bench.py", "--batch", str(batches[0]), "--points", ",".join(str(b) for b in batches[1:]), "--context", str(a.ctx),
            "--prefill", str(a.prefill), "--steps", str(a.steps), "--warmup", str(a.warmup), "--only", "headline",
            "--dtype", "f32" if a.fp32 else a.dtype]
    if os.path.isdir(a.target):
        argv += ["--model", a.target]
    else:
        argv += ["--shape", a.target.lower()]
    if a.layers:
        argv += ["--layers", str(a.layers)]
    sys.argv = argv
    runpy.run_path(str(Path(__file__).resolve().parent.parent / "bench.py"), run_name="__main__")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["timeline"]:  # its options are the timeline program's own (argparse would not pass "--shape ..." on)
        from . import timeline

        return timeline.main(argv[1:])
    ap = argparse.ArgumentParser(prog="mach", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="continue prompts given as token ids")
    g.add_argument("model", help="folder with config.json and model.safetensors")
    g.add_argument("--prompt-ids", action="append", required=True, help='token ids, e.g. "1,2,3"; may be repeated')
    g.add_argument("--max-new", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--top-logprobs", type=int, default=0, help="report the N (at most 20) most probable tokens beside each generated one")
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--eos", type=int, default=None, help="default: the model's eos_token_id")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--stop", action="append", default=[], help="a stop sequence of token ids; may be repeated")
    _engine_options(g)
    g.set_defaults(fn=cmd_generate)

    r = sub.add_parser("replay", help="feed a trace of steps through the model and write logits (see bin/trace_run)")
    r.add_argument("model")
    r.add_argument("trace", help="file of JSON lines, or - for standard input")
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--max-tokens", type=int, required=True)
    r.add_argument("--page-size", type=int, default=16)
    r.set_defaults(fn=cmd_replay)

    w = sub.add_parser("random", help="write a model folder with random weights from a config.json and a seed")
    w.add_argument("config", help="a config.json")
    w.add_argument("--out", required=True)
    w.add_argument("--seed", type=int, default=0)
    w.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "float32"])
    w.add_argument("--weight-std", type=float, default=0.02)
    w.add_argument("--bias-std", type=float, default=0.02)
    w.add_argument("--norm-std", type=float, default=0.05)
    w.set_defaults(fn=cmd_random)

    b = sub.add_parser("bench", help="decode and prefill throughput of a shape (random weights) or of a model folder")
    b.add_argument("target", help="qwen2.5-0.5b, qwen2.5-1.5b, qwen2.5-7b, or a folder with config.json and model.safetensors")
    b.add_argument("--batch", default="8,1,64", help="batch sizes, comma separated; the first is the headline")
    b.add_argument("--ctx", type=int, default=2048, help="tokens every request holds when decoding is timed")
    b.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prompt")
    b.add_argument("--fp32", action="store_true", help="the true 32-bit path")
    b.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "float32"])
    b.add_argument("--steps", type=int, default=50)
    b.add_argument("--warmup", type=int, default=5)
    b.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in the output)")
    b.set_defaults(fn=cmd_bench)

    t = sub.add_parser("timeline", help="device-side timeline of one decoding step (python -m machserve_b200.timeline)")
    t.add_argument("rest", nargs=argparse.REMAINDER)
    t.set_defaults(fn=lambda a: __import__("machserve_b200.timeline", fromlist=["main"]).main(a.rest))

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
