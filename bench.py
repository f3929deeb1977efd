#!/usr/bin/env python3
"""Serving benchmark: decode and prefill throughput of GPT-2 medium on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests.  The default run has the layer
sizes of GPT-2 medium (24 x 1024, 16 heads of 64, inner 4096, vocabulary 50257) with
seeded random bfloat16 weights; each request has a 512-token random prompt and decodes
towards the context length of 1,024.  It prints ONE JSON line:

* ``value``: decoded tokens a second over exactly K steps, timed on the device with CUDA
  events (step function with device sampling, captured CUDA graph; token ids are
  synthetic, uploaded from pinned memory every step);
* ``e2e``: the same through the Python entry point (``LLMEngine.step``): host token ids
  in, sampled token ids out, every step, wall clock;
* ``prefill``: 2,048 prompt tokens (2 x 1,024) in one step, with the fraction of the
  bfloat16 tensor peak its FLOPs reach;
* ``roofline``: bytes a decode step has to read (every weight once, the cache of the live
  requests) / time, against the HBM peak;
* ``points``: decode tokens a second at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the
fallback figures (6.65 TB/s, 1.59 PFLOP/s) of an earlier measurement on this pool.
Every step reads the 0.7 GB of weights, which is larger than the 126 MB L2, so no flush
is needed between timed steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    p = dict(FALLBACK_PEAKS)
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            if "hbm_gbs" in raw:
                p["hbm_gbs"] = float(raw["hbm_gbs"])
            if "bf16_tflops" in raw:
                p["bf16_tflops"] = float(raw["bf16_tflops"])
            if "bf16_tflops_sustained" in raw:
                p["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            src = "measured"
        except (OSError, ValueError):
            pass
    return p, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def model_config(args):
    from hetero_serve_b200 import preset
    cfg = preset("gpt2-medium")
    full_layers = cfg["n_layer"]
    if args.layers:
        cfg["n_layer"] = args.layers
    cfg["eos_token_id"] = None
    return cfg, full_layers


def decode_bytes(model, cfg, batch, mean_ctx, itemsize):
    """Bytes one decode step must read: every weight it uses once (all but the position
    table, of which it reads `batch` rows) and the cache of the live requests."""
    weights = sum(t.numel() * t.element_size() for n, t in model.tensors.items()
                  if n != "wpe.weight")
    kv = batch * mean_ctx * model.kv_bytes_per_token(itemsize)
    return weights + kv


def prefill_flops(cfg, n_seqs, seq_len, n_logit_rows):
    E, I, L, V = cfg["n_embd"], cfg["n_inner"] or 4 * cfg["n_embd"], cfg["n_layer"], cfg["vocab_size"]
    T = n_seqs * seq_len
    linear = 2 * T * L * (E * 3 * E + E * E + 2 * E * I) + 2 * n_logit_rows * E * V
    # causal attention: q.k and p.v over (s+1) keys for query s
    attn = L * n_seqs * 2 * 2 * E * (seq_len * (seq_len + 1) // 2)
    return linear + attn


def time_decode(runner, torch, batch, prompt_len, steps, warmup, vocab, seed, tag):
    """Prefill `batch` requests, then time exactly `steps` decode steps on the device."""
    from hetero_serve_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    ids = [f"{tag}{i}" for i in range(batch)]
    prompts = torch.randint(0, vocab, (batch, prompt_len), generator=g).tolist()
    per_step = max(1, 2048 // prompt_len)
    for i in range(0, batch, per_step):
        runner.step([StepEntry(r, p) for r, p in zip(ids[i:i + per_step], prompts[i:i + per_step])],
                    check_status=False)
    toks = torch.randint(0, vocab, (warmup + steps, batch), generator=g).tolist()
    entries = [StepEntry(r, [0], want=[0]) for r in ids]

    def one(k):
        row = toks[k]
        for e, t in zip(entries, row):
            e.tokens = [t]
        return runner.step(entries, sample=True)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    launches0 = runner.kernel_launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        res = one(k)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    res.tokens_host()                       # reads the status word: a refused index raises
    launches = runner.kernel_launches - launches0
    ctx_first = prompt_len + warmup + 1
    mean_ctx = ctx_first + (steps - 1) / 2
    for r in ids:
        runner.close(r)
    return ms, launches, mean_ctx


def time_prefill(runner, torch, n_seqs, seq_len, vocab, seed, reps=5, warmup=3):
    from hetero_serve_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (n_seqs, seq_len), generator=g).tolist()
    times = []
    for it in range(warmup + reps):
        entries = [StepEntry(f"p{it}_{i}", p, want=[seq_len - 1]) for i, p in enumerate(prompts)]
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        runner.step(entries, sample=True, check_status=False)
        e.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(s.elapsed_time(e))
        for en in entries:
            runner.close(en.req_id)
    runner.check_status()
    return statistics.median(times)


def time_e2e(model_dir, torch, batch, prompt_len, steps, warmup, vocab, seed, num_blocks):
    """The same decode steps through the public entry point: LLMEngine.step(), which packs the
    step's host-side inputs into pinned memory and copies them to the device, and brings
    sampled ids back to the host, every call.  The engine pipelines: a call launches one step
    and reads the tokens of the step before it, so K calls are K launches and K reads."""
    from hetero_serve_b200 import EngineConfig, LLMEngine, Request
    eng = LLMEngine(model_dir, EngineConfig(
        dtype="bfloat16", num_blocks=num_blocks, max_batch=batch, max_prefill_tokens=2048,
        max_requests=batch, prefix_cache=False, cuda_graphs=True))
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (batch, prompt_len), generator=g).tolist()
    seqs = [eng.submit_nowait(Request(p, max_new_tokens=warmup + steps + 2, stop_at_eos=False))
            for p in prompts]
    while any(s.state != "running" for s in seqs):
        eng.step()
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert all(len(s.output_ids) + s.pending == 1 + warmup + steps for s in seqs)
    lay = eng.runner._layout(max(8, batch), batch, batch)
    h2d = lay.total * 4
    d2h = (batch + 1) * 4
    eng.run_until_done()
    return batch * steps / dt, h2d, d2h


def run_ours(args):
    import torch
    from hetero_serve_b200.engine import Runner, load_model
    from hetero_serve_b200.weights import write_model_dir

    if not torch.cuda.is_available():
        print(json.dumps({"impl": "ours", "error": "no CUDA device: this engine has no CPU path"}))
        return 1
    pk, pk_src = peaks()
    cfg, full_layers = model_config(args)
    batch, prompt_len, context = args.batch, args.prompt_len, args.context
    steps, warmup = args.steps, args.warmup
    if prompt_len + warmup + steps + 2 > context:
        steps = context - prompt_len - warmup - 2
    vocab = cfg["vocab_size"]
    with tempfile.TemporaryDirectory(prefix="hsb200-bench-") as d:
        write_model_dir(d, cfg, seed=0, dtype="bfloat16")
        model, _ = load_model(d, "bfloat16", "cuda:0")
        page = 16
        pages_per_req = context // page
        runner = Runner(model, num_pages=64 * pages_per_req + 8, page_size=page, max_requests=64,
                        dtype=torch.bfloat16, device="cuda:0", prefix_cache=False,
                        cuda_graphs=True)
        # correctness gate: the step function must agree with itself across cuts before
        # anything is timed (full comparisons with the plain model live in tests/)
        from hetero_serve_b200.engine import StepEntry
        g = torch.Generator().manual_seed(99)
        probe = torch.randint(0, vocab, (48,), generator=g).tolist()
        a = runner.step([StepEntry("gate_a", probe, want=[47])]).logits.clone()
        runner.step([StepEntry("gate_b", probe[:31])])
        b = runner.step([StepEntry("gate_b", probe[31:], want=[16])]).logits.clone()
        runner.close("gate_a"); runner.close("gate_b")
        if not torch.isfinite(a).all() or (a - b).abs().max() > 5e-2:
            print(json.dumps({"impl": "ours", "error": "correctness gate failed",
                              "max_diff": float((a - b).abs().max())}))
            return 1

        sampler = ClockSampler()
        sampler.start()
        ms, launches, mean_ctx = time_decode(runner, torch, batch, prompt_len, steps, warmup,
                                             vocab, 1, "d")
        clocks = sampler.stop()
        value = batch * steps / (ms / 1e3)
        nbytes = decode_bytes(model, cfg, batch, mean_ctx, 2)
        achieved = nbytes / (ms / steps / 1e3) / 1e9

        points = {}
        for b_ in (1, 64):
            k = min(steps, 128)
            ms_b, _, _ = time_decode(runner, torch, b_, prompt_len, k, warmup, vocab, 2 + b_, f"b{b_}_")
            points[f"decode_b{b_}"] = round(b_ * k / (ms_b / 1e3), 1)

        pre_ms = time_prefill(runner, torch, 2, 1024, vocab, 5)
        flops = prefill_flops(cfg, 2, 1024, 2)
        pre_frac = flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12)
        del runner
        torch.cuda.empty_cache()
        e2e_val, h2d, d2h = time_e2e(d, torch, batch, prompt_len, steps, warmup, vocab, 1,
                                     batch * pages_per_req + 8)

    line = {
        "metric": "decode tokens/s at batch 8, GPT-2 medium, 512-token prompts decoding to 1,024",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": "gpt2-medium (random weights, seed 0)", "n_layer": cfg["n_layer"],
            "n_layer_full": full_layers, "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
            "head_dim": cfg["n_embd"] // cfg["n_head"], "n_inner": cfg["n_inner"],
            "vocab_size": vocab, "n_positions": cfg["n_positions"], "global_batch": batch,
            "seq_len": context, "prompt_len": prompt_len, "kv_block_size": 16,
            "parallelism": "single GPU", "residual_stream": "fp32",
            "l2": "each step reads 0.7 GB of weights (> 126 MB L2); no flush needed",
            "peaks": pk_src,
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e_val, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(2048 / (pre_ms / 1e3), 1), "tokens": 2048,
                    "ms": round(pre_ms, 3), "frac": round(pre_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def run_one_step(args):
    """For profilers: build the model, warm up, then run ONE step (eager, no CUDA graph)
    between cudaProfilerStart and cudaProfilerStop, so that
    `ncu --profile-from-start off ... python bench.py --one-step decode` captures just it."""
    import torch
    from hetero_serve_b200.engine import Runner, StepEntry, load_model
    from hetero_serve_b200.weights import write_model_dir
    cfg, _ = model_config(args)
    vocab = cfg["vocab_size"]
    with tempfile.TemporaryDirectory(prefix="hsb200-bench-") as d:
        write_model_dir(d, cfg, seed=0, dtype="bfloat16")
        model, _ = load_model(d, "bfloat16", "cuda:0")
        runner = Runner(model, num_pages=args.batch * 64 + 136, page_size=16, max_requests=64,
                        dtype=torch.bfloat16, device="cuda:0", cuda_graphs=False)
        g = torch.Generator().manual_seed(0)
        if args.one_step == "decode":
            ids = [f"r{i}" for i in range(args.batch)]
            for r in ids:
                runner.step([StepEntry(r, torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist())])
            entries = [StepEntry(r, [5], want=[0]) for r in ids]
            for _ in range(3):
                runner.step(entries, sample=True)
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            runner.step(entries, sample=True)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            prompts = torch.randint(0, vocab, (2, 1024), generator=g).tolist()
            for it in range(3):
                entries = [StepEntry(f"w{it}_{i}", p, want=[1023]) for i, p in enumerate(prompts)]
                runner.step(entries, sample=True)
                for e in entries:
                    runner.close(e.req_id)
            entries = [StepEntry(f"p{i}", p, want=[1023]) for i, p in enumerate(prompts)]
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            runner.step(entries, sample=True)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        runner.check_status()
    print(json.dumps({"one_step": args.one_step, "n_layer": cfg["n_layer"], "batch": args.batch,
                      "kernel_launches_total": runner.kernel_launches}))
    return 0


def run_reference(args):
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "heteroserve")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "mneha05/hetero-serve has no setup.py or pyproject.toml: pip reports "
                          "'not installable', so there is no offline install to run"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable":
                      "baseline/_ref holds no runnable install of the reference"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", dest="prompt_len", type=int, default=512)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (0: all); both numbers "
                         "are named in `config`")
    ap.add_argument("--one-step", dest="one_step", default="", choices=["", "decode", "prefill"],
                    help="for profilers: run a single eager step between cudaProfilerStart/Stop")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.one_step:
        return run_one_step(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
