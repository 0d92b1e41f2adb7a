#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen2.5 layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 2048] [--layers L]
                    [--shape qwen2.5-0.5b | --model DIR] [--dtype bf16|f32] [--only headline,fp32,...]

Prints ONE JSON line.  A step is one decode step of `batch` requests that each hold
`context` tokens: the model, the sampler and the copy of the sampled tokens to pinned host
memory.  `value` is decoded tokens per second timed on the device with CUDA events around
K such steps after W warm-up steps (the next step's tokens are taken from the sampler's
output on the device); the block of K steps is timed three times and the median block is
reported, with the spread beside it.  `logits_only` is the same without sampler and copy.
`e2e` is the same through the Python entry point (`Engine.step`: host token ids in
through pinned memory, sampled token ids read by the host, every step).  `prefill` is one
request of 2,048 tokens in one step.  `roofline` relates the bytes a decode step has to
read (every weight once, and the cache of the live requests) to the measured copy
bandwidth.  Every step reads about a gigabyte of weights, far more than the 126 MB of L2,
so nothing needs flushing between steps.

Beside the headline the default run measures, under keys of their own:

* `fp32`: the true 32-bit path at the same sizes (decode at the headline batch, prefill);
* `serving_1p5b`: Qwen2.5-1.5B sizes, 64 requests with prompts of 128 to 2,048 tokens and
  256 new tokens each, through `Engine` with continuous batching (generated and prompt
  tokens per second, time to first token, preemptions);
* `mixed_7b`: Qwen2.5-7B sizes, one step of eight 512-row portions of 4,096-token prompts
  (3,584 earlier tokens in the cache) beside 56 decoding rows at 1,024-token contexts.

This engine runs on one GPU: for --gpus > 1 it says so and exits with 2.

    python bench.py --kernel attention_prefill

times the prompt attention kernel alone (2,048, 4,096 and 8,192 tokens) and prints a line of its own;
`--kernel gemm [--shape ...] [--prefill ROWS]` the four products of a layer with their fused epilogues beside the
library's.  `--profile decode|prefill|mixed` brackets that timed region with cudaProfilerStart/Stop, for a profiler
started with --profile-from-start off (the commands are in profiles/).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

_COMMON = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
SHAPES = {
    "qwen2.5-0.5b": dict(_COMMON, vocab_size=151936, hidden_size=896, num_hidden_layers=24, num_attention_heads=14,
                         num_key_value_heads=2, intermediate_size=4864, tie_word_embeddings=True),
    "qwen2.5-1.5b": dict(_COMMON, vocab_size=151936, hidden_size=1536, num_hidden_layers=28, num_attention_heads=12,
                         num_key_value_heads=2, intermediate_size=8960, tie_word_embeddings=True),
    "qwen2.5-7b": dict(_COMMON, vocab_size=152064, hidden_size=3584, num_hidden_layers=28, num_attention_heads=28,
                       num_key_value_heads=4, intermediate_size=18944, tie_word_embeddings=False),
}
QWEN25_05B = SHAPES["qwen2.5-0.5b"]
# the reference's own figure for decode at batch 8 (RX 7900 XTX, float32 weights, short context)
PUBLISHED_DECODE_B8 = 626.0
PAGE = 64


def peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        super().__init__(daemon=True)
        self.samples, self.stop_flag, self.proc = [], False, None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                if self.stop_flag:
                    break
                self.samples.append([x.strip() for x in line.split(",")])
        except OSError:
            pass

    def stop(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        rows = [s for s in self.samples if len(s) == 6 and s[0].isdigit()]
        if rows:
            out["sm_mhz"] = statistics.median(int(r[0]) for r in rows)
            out["sm_max_mhz"] = int(rows[0][1])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            out["reasons"] = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in rows)]
        return out


# ----------------------------------------------------------------- what a step has to read and to compute


def sizes(raw):
    d, i, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    hq, hkv = raw["num_attention_heads"], raw["num_key_value_heads"]
    return d, i, v, hq, hkv, raw.get("head_dim", d // hq)


def weight_bytes(raw, layers, elt=2):
    """Every weight a step reads once: the layers, the final norm and the head (a tied table is read by the head)."""
    d, i, v, hq, hkv, hd = sizes(raw)
    per_layer = d * (hq + 2 * hkv) * hd + (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * i + 2 * d
    return elt * (layers * per_layer + v * d + d)


def kv_bytes_per_token(raw, layers, elt=2):
    _, _, _, _, hkv, hd = sizes(raw)
    return elt * layers * 2 * hkv * hd


def decode_bytes(raw, layers, batch, context, elt=2):
    """Bytes one decode step has to read: every weight once, and the cache of the live requests."""
    return weight_bytes(raw, layers, elt) + kv_bytes_per_token(raw, layers, elt) * context * batch


def step_flops(raw, layers, rows, attended_keys, head_rows):
    """Multiply-adds x 2 of a step: `rows` token rows through the layers' matrices, `attended_keys` (query, key)
    pairs through the attention of every head, `head_rows` rows through the vocabulary head."""
    d, i, v, hq, hkv, hd = sizes(raw)
    matmul = 2 * rows * layers * (d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * i)
    return matmul + 2 * 2 * attended_keys * hd * hq * layers + 2 * head_rows * v * d


def prefill_flops(raw, layers, tokens):
    return step_flops(raw, layers, tokens, tokens * (tokens + 1) // 2, 1)


def config_block(raw, layers, **more):
    d, i, v, hq, hkv, hd = sizes(raw)
    return {"layers": layers, "layers_of_configuration": raw["num_hidden_layers"], "hidden_size": d, "heads": hq,
            "kv_heads": hkv, "head_dim": hd, "intermediate_size": i, "vocab_size": v,
            "tied_embeddings": bool(raw["tie_word_embeddings"]), "page_size": PAGE, **more}


def free_device_memory():
    """After the caller has dropped its runner: gives the device memory back before the next workload is built."""
    import torch

    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------- one kernel alone


def time_gemm_pair_tc(torch, ops, a, pk) -> int:
    """The four products of a layer at `--prefill` rows: the repository's tcgen05 product with its fused epilogues (a
    pair of SMs per tile; the engine uses its gated form for the feed-forward from 1,024 rows on and the library for
    the other products above 16 rows) beside the library's."""
    raw = SHAPES[a.shape]
    h, inter = raw["hidden_size"], raw["intermediate_size"]
    hd = raw.get("head_dim", h // raw["num_attention_heads"])
    qkv = (raw["num_attention_heads"] + 2 * raw["num_key_value_heads"]) * hd
    m, dev = a.prefill, "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, s=0.05: (torch.randn(*shape, device=dev, generator=g) * s).to(torch.bfloat16)
    x, xi = rnd(m, h, s=0.5), rnd(m, inter, s=0.5)
    w_qkv, w_o, w_gu, w_d = rnd(qkv, h), rnd(h, h), rnd(2 * inter, h), rnd(h, inter, s=0.02)
    res = torch.randn(m, h, device=dev, generator=g)
    nb = ops.gemm_pair_tc_stats_blocks(m, h)
    stats, copy = torch.ones(m, nb, device=dev), torch.empty(m, h, dtype=torch.bfloat16, device=dev)
    o_qkv, o_h = torch.empty(m, qkv, dtype=torch.bfloat16, device=dev), torch.empty(m, h, dtype=torch.bfloat16, device=dev)
    o_gu, o_i = torch.empty(m, 2 * inter, dtype=torch.bfloat16, device=dev), torch.empty(m, inter, dtype=torch.bfloat16, device=dev)

    def us(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (2 * reps) * 1000

    if a.profile:  # one launch each of the gated product, the same product plain and the library's, for a profiler
        for _ in range(3):
            ops.gemm_pair_tc_silu_mul(x, w_gu, o_i)
            ops.gemm_pair_tc(x, w_gu, o_gu)
            torch.mm(x, w_gu.T, out=o_gu)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        ops.gemm_pair_tc_silu_mul(x, w_gu, o_i)
        ops.gemm_pair_tc(x, w_gu, o_gu)
        torch.mm(x, w_gu.T, out=o_gu)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        assert ops.gemm_tc_status() == 0
        print(json.dumps({"kernel": "gemm_pair_tc", "shape": a.shape, "rows": m, "profiled": ["gate_up_silu_mul", "gate_up_plain", "library"]}))
        return 0
    out = {}
    for name, own, lib, flops in (
        ("qkv_norm_folded", lambda: ops.gemm_pair_tc(x, w_qkv, o_qkv, stats, nb, 1e-6), lambda: torch.mm(x, w_qkv.T, out=o_qkv), 2 * m * h * qkv),
        ("o_residual_add", lambda: ops.gemm_pair_tc_resadd(x, w_o, res, stats, copy), lambda: torch.mm(x, w_o.T, out=o_h), 2 * m * h * h),
        ("gate_up_silu_mul", lambda: ops.gemm_pair_tc_silu_mul(x, w_gu, o_i, stats, nb, 1e-6), lambda: torch.mm(x, w_gu.T, out=o_gu), 4 * m * h * inter),
        ("down_residual_add", lambda: ops.gemm_pair_tc_resadd(xi, w_d, res, stats, copy), lambda: torch.mm(xi, w_d.T, out=o_h), 2 * m * h * inter)):
        t_own, t_lib = us(own), us(lib)
        out[name] = {"own_us": round(t_own, 1), "own_tflops": round(flops / t_own / 1e6), "library_us": round(t_lib, 1),
                     "library_tflops": round(flops / t_lib / 1e6)}
    assert ops.gemm_tc_status() == 0
    print(json.dumps({"kernel": "gemm_pair_tc", "shape": a.shape, "rows": m, "dtype": "bf16", "products": out,
                      "note": "own: with the epilogue named; library: the plain product alone", "peaks": pk["source"]}))
    return 0


def time_attention_prefill(torch, ops, a, pk) -> int:
    """The prompt attention kernel alone: one sequence of 2,048, 4,096 and 8,192 tokens attending to itself through
    the paged cache, replayed as a CUDA graph of ten launches; CUDA events around the replays."""
    raw = SHAPES[a.shape]
    _, _, _, hq, hkv, hd = sizes(raw)
    page = PAGE
    dev, res = "cuda:0", {}
    for n in (512, 2048, 4096, 8192):
        torch.manual_seed(n)
        pages = n // page + 1
        kp = torch.randn((pages, hkv, page, hd), device=dev).to(torch.bfloat16)
        vp = torch.randn_like(kp)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        q = torch.randn((n, hq * hd), device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        pos = torch.arange(n, dtype=torch.int32, device=dev)
        slot = torch.zeros(n, dtype=torch.int32, device=dev)
        t0 = torch.arange(0, n, 128, dtype=torch.int32, device=dev)
        tn = torch.full_like(t0, 128)
        tiles = t0.numel()
        splits, alone, run_tiles = ops.attention_prefill_tc_plan(tiles, hq, hkv, hd, n, tiles * (tiles + 1) // 2)  # the engine's own choice
        words = ops.attention_prefill_tc_scratch_words(t0.numel(), hq, hd, splits)
        scratch = torch.zeros(words, dtype=torch.float32, device=dev) if words else None
        counters = torch.zeros(t0.numel() * hq, dtype=torch.int32, device=dev) if words else None
        def run():
            ops.attention_prefill_tc(q, kp, vp, out, t0, tn, t0.numel(), pos, slot, table, hq, hkv, hd, None, hd ** -0.5,
                                     splits, scratch, counters, alone=alone, run_tiles=run_tiles)
        for _ in range(max(a.warmup, 3)):
            run()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(10):
                run()
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(1, a.steps // 10)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / (10 * reps) * 1000
        flops = 4 * hq * hd * n * (n + 1) / 2
        res[str(n)] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3),
                       "key_splits": splits, "key_tiles_a_run": run_tiles, "heads_per_block": 1 if alone or hd == 64 else 2}
    assert ops.gemm_tc_status() == 0
    print(json.dumps({"kernel": "attention_prefill_tc", "heads": hq, "kv_heads": hkv, "head_dim": hd, "page_size": page,
                      "dtype": "bf16", "tokens": res, "peaks": pk["source"]}))
    return 0


# --------------------------------------------------------------------------- decode and prefill of one model


class DecodeBench:
    """A runner of one shape with helpers that fill contexts and time decode steps and a prefill."""

    def __init__(self, a, raw, layers, dtype, max_batch, max_seq, load_dir=None):
        import numpy as np
        import torch

        from machserve_b200 import ModelRunner
        from machserve_b200.config import config_from_json
        from machserve_b200.sampling.sampler import Sampler

        self.a, self.raw, self.layers, self.dtype = a, raw, layers, dtype
        self.torch, self.np = torch, np
        pages = max_batch * (-(-max_seq // PAGE)) + 8
        kw = dict(dtype=dtype, page_size=PAGE, num_pages=pages, max_requests=max_batch,
                  max_step_tokens=2048 + max_batch, max_seq_len=max_seq)
        if load_dir:
            self.runner = ModelRunner.from_model_dir(load_dir, **kw)
        else:
            cfg = dict(raw)
            cfg["num_hidden_layers"] = layers
            self.runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, **kw)
        self.sampler = Sampler(max_batch, self.runner.device)
        self.rng = np.random.default_rng(0)
        self.vocab = raw["vocab_size"]

    def release_all(self):
        for r in list(self.runner.cache.requests):
            self.runner.release(r)

    def fill(self, batch, context):
        from machserve_b200 import StepEntry

        self.release_all()
        for r in range(batch):
            toks = self.rng.integers(0, self.vocab, size=context)
            for at in range(0, context, 2048):
                self.runner.step([StepEntry(r, toks[at : at + 2048].tolist(), [])])
        self.torch.cuda.synchronize()

    def time_decode(self, batch, context, steps, warmup, blocks=3, sampled=True, profile=False):
        """ms per step of `blocks` blocks of `steps` decode steps (sorted), and the launches of one block.
        With `sampled`, a step is the model, the sampler and the copy of the tokens to pinned host memory, and the
        next step takes its tokens from the sampler's output on the device; without, the model alone."""
        from machserve_b200 import SamplingParams, StepEntry, ops

        torch, runner, sampler = self.torch, self.runner, self.sampler
        self.fill(batch, context)
        greedy, states = [SamplingParams()] * batch, [1] * batch
        toks = self.rng.integers(0, self.vocab, size=batch)
        first = [True]

        def one():
            if not sampled:
                runner.step([StepEntry(r, [int(toks[r])], [0]) for r in range(batch)])
                return
            if first[0]:
                entries = [StepEntry(r, [int(toks[r])], [0]) for r in range(batch)]
                first[0] = False
            else:
                entries = [StepEntry(r, [0], [0], from_sampled=r) for r in range(batch)]
            logits = runner.step(entries, sampled=sampler.tokens_on_device)
            sampler.launch(logits, greedy, states)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        times, launches = [], 0
        for b in range(blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = ops.launches()
            if profile and b == 0:
                torch.cuda.profiler.start()  # a profiler started with --profile-from-start off sees these steps only
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            if profile and b == 0:
                torch.cuda.profiler.stop()
            times.append(e0.elapsed_time(e1) / steps)
            launches = ops.launches() - l0
        return sorted(times), launches

    def time_prefill(self, tokens, warmup, reps=5, profile=False):
        """Median ms of one request of `tokens` tokens in one step, logits at its last token, sampled."""
        from machserve_b200 import SamplingParams, StepEntry

        torch, runner = self.torch, self.runner
        self.release_all()
        times = []
        for it in range(warmup + reps):
            toks = self.rng.integers(0, self.vocab, size=tokens).tolist()
            torch.cuda.synchronize()
            last = it == warmup + reps - 1
            if profile and last:
                torch.cuda.profiler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            logits = runner.step([StepEntry("p", toks, [tokens - 1])])
            self.sampler.launch(logits, [SamplingParams()], [1])
            e1.record()
            torch.cuda.synchronize()
            if profile and last:
                torch.cuda.profiler.stop()
            runner.release("p")
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def time_e2e(self, batch, context, steps, warmup):
        """Tokens per second through `Engine.step`: host ids in, sampled ids read by the host, every step."""
        from machserve_b200 import Engine, SamplingParams

        torch, runner = self.torch, self.runner
        self.release_all()
        eng = Engine(runner=runner, prefill_rows=2048)
        # (a request decodes while the prompts behind it are still read, one prompt a step: none may finish before the end)
        for _ in range(batch):
            eng.add(self.rng.integers(0, self.vocab, size=context).tolist(), steps + warmup + batch + 8, params=SamplingParams())
        while any(s.computed < len(s.prompt) for s in eng.scheduler.running) or eng.scheduler.waiting:
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d0, d2h0 = runner.h2d_bytes + eng.sampler.h2d_bytes, eng.sampler.d2h_bytes
        t0 = time.perf_counter()
        made = 0
        for _ in range(steps):
            made += len(eng.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        # counted from the tensors that were copied: the step's index arrays (token ids among them) and changed
        # block-table rows from pinned memory to the device; the sampled tokens and log-probabilities back
        out = {"value": round(made / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round((runner.h2d_bytes + eng.sampler.h2d_bytes - h2d0) / steps, 1),
               "d2h_bytes_per_step": round((eng.sampler.d2h_bytes - d2h0) / steps, 1)}
        while not eng.all_done():
            eng.step()
        return out


# ------------------------------------------------------------------------------------ the other workloads


def workload_fp32(a, pk, raw, layers):
    """The true 32-bit path at the headline's sizes: decode at the headline batch and a prefill of 2,048 tokens."""
    steps = max(10, a.steps // 2)
    b = DecodeBench(a, raw, layers, "f32", a.batch, a.context + 4 * (steps + a.warmup) + a.batch + 64)
    times, launches = b.time_decode(a.batch, a.context, steps, a.warmup)
    ms = times[len(times) // 2]
    nbytes = decode_bytes(raw, layers, a.batch, a.context + a.warmup + steps * 3 // 2, elt=4)
    pms = b.time_prefill(2048, 1, reps=3)
    out = {"dtype": "fp32", "global_batch": a.batch, "seq_len": a.context, "steps": steps,
           "decode_tokens_per_s": round(a.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
           "ms_min": round(times[0], 4), "ms_max": round(times[-1], 4), "gpu_launches_per_step": launches // steps,
           "hbm_gbs": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4),
           "prefill_tokens": 2048, "prefill_ms": round(pms, 3), "prefill_tokens_per_s": round(2048e3 / pms, 1),
           "prefill_tflops": round(prefill_flops(raw, layers, 2048) / pms / 1e9, 2),
           "matrix_products": "float32 multiply-adds on the CUDA cores, no reduced-precision mode"}
    b.release_all()
    del b
    free_device_memory()
    return out


def workload_serving(a, pk):
    """Qwen2.5-1.5B sizes: 64 requests, prompts of 128 to 2,048 tokens (seeded), 256 new tokens each, through `Engine`
    with its default budget of prompt tokens per step.  All requests arrive at time zero.  Three loads of other prompt
    lengths and token ids run untimed first, as a server that has been up for a while: they load the kernels and
    capture the graphs of the step sizes that keep coming (the timed load's own steps have not been seen before)."""
    import numpy as np
    import torch

    from machserve_b200 import Engine, ModelRunner, SamplingParams
    from machserve_b200.config import config_from_json

    raw = SHAPES["qwen2.5-1.5b"]
    layers = a.layers_serving or raw["num_hidden_layers"]
    cfg = dict(raw)
    cfg["num_hidden_layers"] = layers
    n_req, new, lo, hi, prefill_rows = 64, 256, 128, 2048, 512
    max_seq = hi + new
    runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, dtype="bf16", page_size=PAGE,
                                     num_pages=n_req * (-(-max_seq // PAGE)), max_requests=n_req,
                                     max_step_tokens=n_req + prefill_rows, max_seq_len=max_seq)
    wb, kvb = weight_bytes(raw, layers), kv_bytes_per_token(raw, layers)

    def run(seed, lengths_seed=1):
        lengths = [int(x) for x in np.random.default_rng(lengths_seed).integers(lo, hi + 1, size=n_req)]
        eng = Engine(runner=runner, prefill_rows=prefill_rows)
        ids_rng = np.random.default_rng(seed)
        plans = []
        schedule = eng.scheduler.schedule

        def recording():
            plan = schedule()
            plans.append([(e.start, e.count, e.samples) for e in plan.entries])
            return plan

        eng.scheduler.schedule = recording
        prompts = [ids_rng.integers(0, raw["vocab_size"], size=n).tolist() for n in lengths]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sids = [eng.add(p, new, params=SamplingParams()) for p in prompts]
        first, steps = {}, 0
        while not eng.all_done():
            out = eng.step()
            steps += 1
            now = time.perf_counter() - t0
            for sid, _ in out:
                if sid not in first:
                    first[sid] = (now, steps)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        made = sum(len(eng.generated(s)) for s in sids)
        for s in sids:
            eng.ack(s)
        return wall, made, first, steps, plans, eng.counters, lengths

    for warm in range(3):
        run(2, 100 + warm)
    wall, made, first, steps, plans, counters, lengths = run(3)
    runner.check_device_status()
    # what the steps as planned have to read and to compute: the slower of the two bounds, step by step
    floor = 0.0
    for plan in plans:
        if not plan:
            continue
        rows = sum(c for _, c, _ in plan)
        keys = sum(c * s + c * (c + 1) // 2 for s, c, _ in plan)
        nbytes = wb + kvb * sum(s + c for s, c, _ in plan)
        flops = step_flops(raw, layers, rows, keys, sum(1 for _, _, w in plan if w))
        floor += max(nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
    ttft_ms = sorted(t * 1000 for t, _ in first.values())
    ttft_steps = sorted(s for _, s in first.values())
    p95 = lambda xs: xs[min(len(xs) - 1, int(round(0.95 * (len(xs) - 1))))]
    out = config_block(raw, layers, dtype="bf16", requests=n_req, prompt_tokens_min=lo, prompt_tokens_max=hi,
                       prompt_tokens_total=sum(lengths), new_tokens_each=new, capacity=n_req, prefill_rows=prefill_rows)
    out.update({
        "generated_tokens_per_s": round(made / wall, 1), "prompt_tokens_per_s": round(sum(lengths) / wall, 1),
        "generated_tokens": made, "wall_s": round(wall, 3), "engine_steps": steps, "preemptions": counters["preemptions"],
        "ttft_ms_median": round(statistics.median(ttft_ms), 1), "ttft_ms_p95": round(p95(ttft_ms), 1),
        "ttft_steps_median": statistics.median(ttft_steps), "ttft_steps_p95": p95(ttft_steps),
        "roofline_floor_s": round(floor, 4), "roofline_frac": round(floor / wall, 4),
        "graphs_of_decoding_steps": runner.graph_counts()["decode"], "graphs_of_other_steps": runner.graph_counts()["shapes"],
        "timing": "wall clock around the whole load through Engine.step, host ids in, sampled ids read by the host",
    })
    del runner
    free_device_memory()
    return out


def workload_mixed(a, pk):
    """Qwen2.5-7B sizes: ONE step of eight 512-row portions of 4,096-token prompts (the last portion of each: 3,584
    earlier tokens are in the cache) beside 56 decoding rows at 1,024-token contexts; the step's logits (64 rows)
    are sampled and the tokens read by the host inside the timed region.  Median of the repeats; between repeats
    the eight prompts are given back and brought to 3,584 tokens again."""
    import numpy as np
    import torch

    from machserve_b200 import ModelRunner, SamplingParams, StepEntry
    from machserve_b200.config import config_from_json
    from machserve_b200.sampling.sampler import Sampler

    raw = SHAPES["qwen2.5-7b"]
    layers = a.layers_mixed or raw["num_hidden_layers"]
    cfg = dict(raw)
    cfg["num_hidden_layers"] = layers
    n_dec, ctx, n_pf, prompt, portion, reps = 56, 1024, 8, 4096, 512, 5
    max_seq = prompt + 64
    pages = n_dec * (-(-(ctx + reps + 12) // PAGE)) + n_pf * (-(-prompt // PAGE)) + 8
    runner = ModelRunner.from_random(config_from_json(cfg), seed=0, on_device=True, dtype="bf16", page_size=PAGE,
                                     num_pages=pages, max_requests=n_dec + n_pf,
                                     max_step_tokens=n_pf * portion + n_dec, max_seq_len=max_seq)
    sampler = Sampler(n_dec + n_pf, runner.device)
    rng = np.random.default_rng(4)
    vocab = raw["vocab_size"]
    ids = lambda n: rng.integers(0, vocab, size=n).tolist()
    for at in range(0, n_dec, 4):  # the decoding requests' contexts, four prompts of 1,024 tokens per step
        runner.step([StepEntry(("d", r), ids(ctx), []) for r in range(at, min(at + 4, n_dec))])
    greedy, states = [SamplingParams()] * (n_dec + n_pf), [1] * (n_dec + n_pf)
    times, walls = [], []
    for rep in range(reps + 4):
        for r in range(n_pf):
            runner.release(("p", r))
        for at in range(0, prompt - portion, portion):
            runner.step([StepEntry(("p", r), ids(portion), []) for r in range(n_pf)])
        entries = [StepEntry(("p", r), ids(portion), [portion - 1]) for r in range(n_pf)]
        entries += [StepEntry(("d", r), ids(1), [0]) for r in range(n_dec)]
        torch.cuda.synchronize()
        bracket = a.profile == "mixed" and rep == reps + 3
        if bracket:
            torch.cuda.cudart().cudaProfilerStart()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        logits = runner.step(entries)
        toks, _ = sampler.sample(logits, greedy, states)
        e1.record()
        torch.cuda.synchronize()
        if bracket:
            torch.cuda.cudart().cudaProfilerStop()
        if rep >= 4:  # the first passes load kernels and size the scratch memory, the second captures the step
            walls.append((time.perf_counter() - t0) * 1000)
            times.append(e0.elapsed_time(e1))
        assert len(toks) == n_dec + n_pf
    runner.check_device_status()
    ms = statistics.median(times)
    rows = n_pf * portion + n_dec
    keys = n_pf * (portion * (prompt - portion) + portion * (portion + 1) // 2) + n_dec * (ctx + (reps + 4) // 2 + 1)
    flops = step_flops(raw, layers, rows, keys, n_dec + n_pf)
    nbytes = weight_bytes(raw, layers) + kv_bytes_per_token(raw, layers) * (n_pf * prompt + n_dec * ctx)
    out = config_block(raw, layers, dtype="bf16", prompt_portions=n_pf, portion_rows=portion, prompt_tokens=prompt,
                       earlier_tokens_in_cache=prompt - portion, decode_rows=n_dec, decode_context=ctx, rows=rows)
    out.update({
        "ms_per_step": round(ms, 3), "ms_min": round(min(times), 3), "ms_max": round(max(times), 3), "repeats": reps,
        "wall_ms_median": round(statistics.median(walls), 3), "rows_per_s": round(rows * 1000.0 / ms, 1),
        "tflops": round(flops / ms / 1e9, 1), "tensor_frac": round(flops / ms / 1e9 / pk["bf16_tflops"], 4),
        "hbm_gbs": round(nbytes / ms / 1e6, 1), "bound": "tensor",
        "timing": "CUDA events around runner.step + sampler + read of the 64 sampled tokens by the host",
    })
    del runner, sampler
    free_device_memory()
    return out


# ------------------------------------------------------------------------------------------------- main


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prompt")
    ap.add_argument("--points", default="1,64", help="further batch sizes for `points` (comma separated)")
    ap.add_argument("--shape", default="qwen2.5-0.5b", choices=sorted(SHAPES), help="layer sizes of the headline")
    ap.add_argument("--model", default=None, help="a model folder (config.json, model.safetensors) instead of a shape")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--layers-serving", type=int, default=None, help="the same for the serving_1p5b workload")
    ap.add_argument("--layers-mixed", type=int, default=None, help="the same for the mixed_7b workload")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "fp32", "float32"])
    ap.add_argument("--only", default="headline,fp32,serving_1p5b,mixed_7b",
                    help="which parts to run: headline, fp32, serving_1p5b, mixed_7b (comma separated)")
    ap.add_argument("--no-points", action="store_true", help="skip the further batch sizes and the prefill")
    ap.add_argument("--profile", default=None, choices=["decode", "prefill", "mixed"],
                    help="which timed region is bracketed by cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--kernel", default=None, choices=["attention_prefill", "gemm"],
                    help="time one kernel alone at the configuration's head sizes instead of the step, and print its own line")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "gqf2008/machserve is Rust + HIP (hiprtc, hipBLAS) for AMD GPUs: no Rust toolchain here, "
                          "no Python package to install, and no CUDA path in its tree"}))
        return 0
    if a.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    only = {x.strip() for x in a.only.split(",") if x.strip()}
    if a.profile:
        only = {"mixed_7b"} if a.profile == "mixed" else {"headline"}

    import torch

    from machserve_b200 import ops

    pk = peaks()
    if a.kernel == "gemm":
        return time_gemm_pair_tc(torch, ops, a, pk)
    if a.kernel == "attention_prefill":
        return time_attention_prefill(torch, ops, a, pk)
    if a.model:
        raw = json.load(open(os.path.join(a.model, "config.json")))
        raw.setdefault("num_key_value_heads", raw["num_attention_heads"])
        raw.setdefault("tie_word_embeddings", False)
        name = os.path.basename(os.path.normpath(a.model))
    else:
        raw, name = SHAPES[a.shape], {"qwen2.5-0.5b": "Qwen2.5-0.5B sizes", "qwen2.5-1.5b": "Qwen2.5-1.5B sizes",
                                      "qwen2.5-7b": "Qwen2.5-7B sizes"}[a.shape]
    full_layers = raw["num_hidden_layers"]
    layers = full_layers if a.model else (a.layers or full_layers)
    f32 = a.dtype in ("f32", "fp32", "float32")
    elt = 4 if f32 else 2
    points_b = [] if a.no_points else [int(x) for x in a.points.split(",") if x.strip()]

    line = {}
    if "headline" in only:
        max_batch = max([a.batch, *points_b])
        b = DecodeBench(a, raw, layers, a.dtype, max_batch, a.context + 4 * (a.steps + a.warmup) + max_batch + 64, load_dir=a.model)
        clocks = ClockSampler()
        clocks.start()
        times, launches = b.time_decode(a.batch, a.context, a.steps, a.warmup, profile=a.profile == "decode")
        clock_info = clocks.stop()
        ms_step = times[len(times) // 2]
        value = a.batch * 1000.0 / ms_step
        bare, _ = b.time_decode(a.batch, a.context, a.steps, a.warmup, blocks=1, sampled=False)
        e2e = b.time_e2e(a.batch, a.context, a.steps, a.warmup)
        points, points_e2e, prefill = {}, {}, None
        for pb in points_b:
            t, _ = b.time_decode(pb, a.context, a.steps, a.warmup)
            points[f"decode_b{pb}"] = round(pb * 1000.0 / t[len(t) // 2], 1)
            points_e2e[f"decode_b{pb}"] = b.time_e2e(pb, a.context, a.steps, a.warmup)["value"]
        if not a.no_points:
            pms = b.time_prefill(a.prefill, a.warmup, profile=a.profile == "prefill")
            prefill = {"value": round(a.prefill * 1000.0 / pms, 1), "tokens": a.prefill, "ms": round(pms, 3),
                       "frac": round(prefill_flops(raw, layers, a.prefill) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        b.runner.check_device_status()  # raises if a tensor-core kernel gave up one of its bounded waits
        b.release_all()
        del b
        free_device_memory()

        # the median block ran at contexts of about context + warmup + 1.5 * steps tokens
        nbytes = decode_bytes(raw, layers, a.batch, a.context + a.warmup + a.steps * 3 // 2, elt)
        achieved = nbytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": f"decode tokens/s ({name}, batch {a.batch}, {a.context}-token contexts)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / PUBLISHED_DECODE_B8, 2) if a.shape == "qwen2.5-0.5b" and not a.model else None,
            "dtype": "fp32" if f32 else "bf16",
            "data": "synthetic: seeded uniform random token ids, random-init weights N(0, 0.02) drawn on the device",
            "config": config_block(
                raw, layers, model=name, global_batch=a.batch, seq_len=a.context, parallelism="single GPU",
                l2="inputs larger than L2 (weights read every step)",
                timed="model + sampler + token copy to host, CUDA events, median of 3 blocks of K steps",
                baseline="reference decode batch 8 on RX 7900 XTX, f32: 626 tok/s", peaks=pk["source"]),
            "spread": {"blocks": len(times), "ms_min": round(times[0], 4), "ms_max": round(times[-1], 4)},
            "logits_only": {"value": round(a.batch * 1000.0 / bare[0], 1), "ms_per_step": round(bare[0], 4),
                            "what": "the model's step alone, no sampler and no copy of tokens"},
            "e2e": e2e, "gpu_launches": launches, "clocks": clock_info,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
        }
        if prefill:
            line["prefill"] = prefill
        if points:
            line["points"] = points
            line["points_e2e"] = points_e2e
    if "fp32" in only and not f32 and not a.model:
        line["fp32"] = workload_fp32(a, pk, raw, layers)
    if "serving_1p5b" in only:
        line["serving_1p5b"] = workload_serving(a, pk)
    if "mixed_7b" in only:
        line["mixed_7b"] = workload_mixed(a, pk)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
