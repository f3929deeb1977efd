#!/usr/bin/env python3
"""Serving benchmark: decode and prefill throughput of GPT-2 medium on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workloads large,xl|none] [--kernels] [--dtype bfloat16|float32]

A "step" is one decode step of a batch of 8 requests.  The default run has the layer
sizes of GPT-2 medium (24 x 1024, 16 heads of 64, inner 4096, vocabulary 50257) with
seeded random bfloat16 weights; each request stands for a 512-token random prompt that
decodes towards the context length of 1,024.  Whatever K is, the K timed steps are spread
over that whole trajectory: it is cut into five windows of equal length, K/5 steps are
timed in the middle of each (requests are prefilled to the window's context, W warm-up
steps run, then the timed steps run up to three times and the median counts), and the
windows' times are added.  With the default K = 500 the windows join up and the run is
the trajectory itself.  It prints ONE JSON line:

* ``value``: decoded tokens a second over exactly K steps, timed on the device with CUDA
  events (step function with device sampling, captured CUDA graph; token ids are
  synthetic, uploaded from pinned memory every step);
* ``e2e``: the same windows through the Python entry point (``LLMEngine.step``): host
  token ids in, sampled token ids out, every step, wall clock;
* ``prefill``: 2,048 prompt tokens (2 x 1,024) in one step, with the fraction of the
  bfloat16 tensor peak its FLOPs reach;
* ``roofline``: bytes a decode step has to read (every weight once, the cache of the live
  requests) / time, against the HBM peak;
* ``points``: decode tokens a second at batch 1 and 64 over the same windows, the batch-8
  figure of every window, and the serving workloads of GPT-2 large (64 requests, a quarter
  sharing a 256-token prefix, portions of 512) and GPT-2 XL (128 concurrent requests, a
  pool that forces recompute-preemption) through ``LLMEngine``;
* ``kernels``: for the kernels a decode step and a prefill step spend their time in, the
  fraction of the HBM or tensor peak each reaches alone, cold L2 (``--kernels`` prints the
  table behind it; a kernel whose output is off its plain PyTorch twin is not timed).

Before anything is timed the engine's logits are compared with the plain implementation
(tests/plain_gpt2.py) on a two-layer model of the same widths: the last rows of a
2 x 1,024 prefill and of decode steps at batch 64.  A failed comparison ends the run.

``--impl reference`` runs mneha05/hetero-serve itself (baseline/_ref, unmodified) through
its own classes on the same windows and prints the same line with ``"impl": "reference"``.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the
fallback figures (6.65 TB/s, 1.59 PFLOP/s).  Every step reads the 0.7 GB of weights, which
is larger than the 126 MB L2, so no flush is needed between timed steps.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
N_WINDOWS = 5
METRIC = ("decode tokens/s at batch 8, GPT-2 medium, 512-token prompts decoding to 1,024 "
          "(K steps spread over the whole trajectory)")
MODEL_NAMES = {"gpt2": "GPT-2 small", "gpt2-medium": "GPT-2 medium", "gpt2-large": "GPT-2 large",
               "gpt2-xl": "GPT-2 XL"}


def metric_name(args):
    """The headline metric's name; other presets of the family (--model) say which they are."""
    name = MODEL_NAMES.get(args.model, args.model)
    return METRIC.replace("GPT-2 medium", name).replace("batch 8", f"batch {args.batch}")


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
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed.  The
    reported clock is the median of the samples taken while the GPU was busy (utilisation above
    zero); a program that leaves the GPU idle between small kernels, as the reference arm does,
    shows the idle clock in the others."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,utilization.gpu")

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
        sm, mx, busy, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            try:
                if len(parts) > 7 and float(parts[7]) > 0:
                    busy.append(sm[-1])
            except ValueError:
                pass
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        under_load = busy or sm
        return {"sm_mhz": statistics.median(under_load) if under_load else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "samples_busy": len(busy), "reasons": sorted(reasons)}


def decode_windows(prompt_len: int, context: int, steps: int, n_windows: int = N_WINDOWS):
    """Cut the decode trajectory prompt_len -> context into windows and place the timed steps
    in the middle of each: ``[(first, k, repeats)]`` where the first timed step of a window
    attends over ``first`` keys, ``k`` steps make one repeat, and up to three repeats follow
    one another while they fit the window.  The k of all windows add up to ``steps``.  A
    timed repeat starts behind a synchronisation, i.e. from an idle GPU, so it is kept at 16
    steps or more: few steps make fewer windows (one, around the trajectory's middle, below 32
    steps), and the mean context of the timed steps stays that of the whole trajectory."""
    n = max(1, min(n_windows, steps // 16, steps))
    per = (context - prompt_len) // n
    out = []
    for i in range(n):
        k = steps // n + (1 if i < steps % n else 0)
        lo = prompt_len + i * per
        room = min(context - 2, lo + per) - lo
        reps = max(1, min(3, room // k))
        out.append((lo + max(0, (room - reps * k) // 2), k, reps))
    return out


def max_steps(prompt_len: int, context: int, n_windows: int = N_WINDOWS) -> int:
    return n_windows * ((context - prompt_len) // n_windows - 2)


def windows_mean_context(windows) -> float:
    total = sum(k for _f, k, _r in windows)
    return sum(k * (first + (reps * k - 1) / 2) for first, k, reps in windows) / total


def model_config(args):
    from hetero_serve_b200.config import preset
    cfg = preset(args.model)
    full_layers = cfg["n_layer"]
    if args.layers:
        cfg["n_layer"] = args.layers
    cfg["eos_token_id"] = None
    return cfg, full_layers


def decode_bytes(model, batch, mean_ctx, itemsize):
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


def time_decode(runner, torch, batch, windows, warmup, vocab, seed, tag):
    """Times the windows of a decode trajectory on the device.  Returns (ms over the K counted
    steps, kernel launches in them, ms per step of each window)."""
    from hetero_serve_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    total_ms = 0.0
    launches = 0
    per_window = []
    for wi, (first, k, reps) in enumerate(windows):
        ids = [f"{tag}{wi}_{i}" for i in range(batch)]
        # One-time costs stay out of the timed steps: the engine gives a step shape its second
        # CUDA graph (metadata uploads that overlap the step before) once the shape has come
        # back `hot_shape_uses` times, so the first window's prompts are that much shorter and
        # decode up to the window's start before the W warm-up steps.
        settle = 0
        if wi == 0:
            settle = max(0, getattr(runner, "hot_shape_uses", 0) + 3 - warmup)
            settle = min(settle, max(0, first - warmup - 1 - 64))
        plen = first - warmup - 1 - settle
        prompts = torch.randint(0, vocab, (batch, plen), generator=g).tolist()
        per_step = max(1, 2048 // plen)
        for i in range(0, batch, per_step):
            runner.step([StepEntry(r, p) for r, p in zip(ids[i:i + per_step],
                                                         prompts[i:i + per_step])],
                        check_status=False)
        toks = torch.randint(0, vocab, (warmup + reps * k, batch), generator=g).tolist()
        entries = [StepEntry(r, [0], want=[0]) for r in ids]

        def one(j):
            for e, t in zip(entries, toks[j]):
                e.tokens = [t]
            return runner.step(entries, sample=True)

        for j in range(settle):
            one(j % len(toks))
        for j in range(warmup):
            one(j)
        times = []
        for r in range(reps):
            torch.cuda.synchronize()
            l0 = runner.kernel_launches
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for j in range(warmup + r * k, warmup + (r + 1) * k):
                res = one(j)
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
            if r == 0:
                launches += runner.kernel_launches - l0
        res.tokens_host()                   # reads the status word: a refused index raises
        med = statistics.median(times)
        total_ms += med
        per_window.append(med / k)
        for r in ids:
            runner.close(r)
    return total_ms, launches, per_window


def time_prefill(runner, torch, n_seqs, seq_len, vocab, seed, reps=5, warmup=3, chain=4):
    """Milliseconds of one prefill step of n_seqs whole prompts: `chain` such steps (other
    requests, other pages) launched back to back between two events, divided by `chain`, so
    that the host's preparation of a step runs while the device works on the one before, as
    it does in serving and in the decode windows; the median of `reps` such chains.  Also
    returned: the same for a single step launched on an idle device (host preparation
    included)."""
    from hetero_serve_b200.engine import StepEntry
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (n_seqs, seq_len), generator=g).tolist()
    out = {}
    for n in (chain, 1):
        times = []
        for it in range(warmup + reps):
            steps = [[StepEntry(f"p{n}_{it}_{c}_{i}", p, want=[seq_len - 1])
                      for i, p in enumerate(prompts)] for c in range(n)]
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for entries in steps:
                runner.step(entries, sample=True, check_status=False)
            e.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(s.elapsed_time(e) / n)
            for entries in steps:
                for en in entries:
                    runner.close(en.req_id)
        out[n] = statistics.median(times)
    runner.check_status()
    return out[chain], out[1]


def time_e2e(model_dir, torch, batch, windows, warmup, vocab, seed, num_blocks, dtype,
             fused_decode=False):
    """The same windows through the public entry point: LLMEngine.step(), which packs the
    step's host-side inputs into pinned memory and copies them to the device, and brings
    sampled ids back to the host, every call.  The engine pipelines: a call launches one step
    and reads the tokens of the step before it, so k calls are k launches and k reads."""
    from hetero_serve_b200 import EngineConfig, LLMEngine, Request
    eng = LLMEngine(model_dir, EngineConfig(
        dtype=dtype, num_blocks=num_blocks, max_batch=batch, max_prefill_tokens=2048,
        max_requests=batch, prefix_cache=False, cuda_graphs=True, fused_decode=fused_decode))
    g = torch.Generator().manual_seed(seed)
    total = 0.0
    for wi, (first, k, reps) in enumerate(windows):
        settle = 0                          # as in time_decode: one-time costs before the window
        if wi == 0:
            settle = max(0, getattr(eng.runner, "hot_shape_uses", 0) + 3 - warmup)
            settle = min(settle, max(0, first - warmup - 1 - 64))
        plen = first - warmup - 1 - settle
        prompts = torch.randint(0, vocab, (batch, plen), generator=g).tolist()
        seqs = [eng.submit_nowait(Request(p, max_new_tokens=settle + warmup + reps * k + 2,
                                          stop_at_eos=False)) for p in prompts]
        while any(s.state != "running" for s in seqs):
            eng.step()
        for _ in range(settle + warmup):
            eng.step()
        times = []
        for _ in range(reps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(k):
                eng.step()
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
        assert all(len(s.output_ids) + s.pending == 1 + settle + warmup + reps * k for s in seqs)
        total += statistics.median(times)
        eng.run_until_done()
    lay = eng.runner._layout(max(8, batch), batch, batch)
    steps = sum(k for _f, k, _r in windows)
    return batch * steps / total, lay.total * 4, (batch + 1) * 4


# ---------------------------------------------------------------------------------------
# the gate: engine against the plain implementation, at the widths that are timed
# ---------------------------------------------------------------------------------------

def correctness_gate(torch, cfg, dtype):
    """Logits of the engine against tests/plain_gpt2.py (float32 arithmetic on the CPU, the
    matrices rounded as the engine stores them) on a two-layer model of the timed widths:
    the last rows of a 2 x 1,024 prefill, and of a decode step at batch 64 with contexts
    near the end of the table (four of the 64 requests are compared).  Returns the largest
    difference and the tolerance."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_gpt2
    from hetero_serve_b200.engine import Runner, StepEntry, load_model
    from hetero_serve_b200.weights import read_safetensors, write_model_dir
    small = dict(cfg, n_layer=2)
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tol = 6e-2 if dtype == "bfloat16" else 2e-3
    vocab = small["vocab_size"]
    with tempfile.TemporaryDirectory(prefix="hsb200-gate-") as d:
        write_model_dir(d, small, seed=7, dtype=dtype)
        raw = read_safetensors(os.path.join(d, "model.safetensors"))
        plain = plain_gpt2.prepare_weights(raw, dtype=torch.float32,
                                           round_to=tdt if dtype == "bfloat16" else None)
        model, _ = load_model(d, dtype, "cuda:0")
        runner = Runner(model, num_pages=64 * 64 + 8, page_size=16, max_requests=64, dtype=tdt,
                        device="cuda:0", cuda_graphs=(dtype == "bfloat16"))
        g = torch.Generator().manual_seed(99)
        worst = 0.0
        # prefill 2 x 1,024
        prompts = torch.randint(0, vocab, (2, 1024), generator=g).tolist()
        got = runner.step([StepEntry(f"g{i}", p, want=[1023]) for i, p in enumerate(prompts)]
                          ).logits.float().cpu()
        for i, p in enumerate(prompts):
            want = plain_gpt2.forward(small, plain, p, dtype=torch.float32, rows=[1023])[0]
            worst = max(worst, float((got[i] - want).abs().max()))
            runner.close(f"g{i}")
        # decode at batch 64: contexts 900..1,020, checked on four requests
        lens = [900 + (i * 37) % 120 for i in range(64)]
        seqs = [torch.randint(0, vocab, (n + 2,), generator=g).tolist() for n in lens]
        for i0 in range(0, 64, 2):
            runner.step([StepEntry(f"d{i}", seqs[i][:lens[i]]) for i in (i0, i0 + 1)])
        for j in range(2):
            res = runner.step([StepEntry(f"d{i}", [seqs[i][lens[i] + j]], want=[0])
                               for i in range(64)])
        got = res.logits.float().cpu()
        for i in (0, 21, 42, 63):
            n = lens[i] + 2
            want = plain_gpt2.forward(small, plain, seqs[i][:n], dtype=torch.float32,
                                      rows=[n - 1])[0]
            worst = max(worst, float((got[i] - want).abs().max()))
        finite = bool(torch.isfinite(got).all())
        del runner, model
        torch.cuda.empty_cache()
    return (worst if finite else float("inf")), tol


# ---------------------------------------------------------------------------------------
# serving workloads of GPT-2 large and XL through the Python entry point
# ---------------------------------------------------------------------------------------

WORKLOADS = {
    # 64 requests, prompt lengths uniform in [32, 768], a quarter sharing a 256-token prefix,
    # 128 new tokens each, prompt portions of 512
    "large": dict(preset="gpt2-large", n_requests=64, prompt_lo=32, prompt_hi=768,
                  shared_frac=0.25, shared_len=256, new_tokens=128, chunk=512, max_batch=64,
                  num_blocks=64 * 57, prefix_cache=True),
    # 128 concurrent requests, prompt lengths uniform in [64, 1024), 256 new tokens capped at
    # 1,024 positions, a pool of 3,072 pages (49,152 tokens; the requests grow towards about
    # 100,000) so that decoding runs out of pages and preempts
    "xl": dict(preset="gpt2-xl", n_requests=128, prompt_lo=64, prompt_hi=1023,
               shared_frac=0.0, shared_len=0, new_tokens=256, chunk=512, max_batch=128,
               num_blocks=3072, prefix_cache=True),
}


def run_workload(torch, name, dtype, policy, layers=0):
    """One serving workload through LLMEngine: every request submitted at once, run until all
    have finished.  Returns flat figures (tokens a second, latencies, preemptions, prefix
    hits)."""
    from hetero_serve_b200 import EngineConfig, LLMEngine, Request
    from hetero_serve_b200.config import preset
    w = WORKLOADS[name]
    cfg = preset(w["preset"])
    full = cfg["n_layer"]
    if layers:
        cfg["n_layer"] = layers
    cfg["eos_token_id"] = None
    vocab = cfg["vocab_size"]
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(w["prompt_lo"], w["prompt_hi"] + 1, (w["n_requests"],), generator=g).tolist()

    def make_prompts():
        shared = torch.randint(0, vocab, (max(1, w["shared_len"]),), generator=g).tolist()
        prompts = []
        for i, n in enumerate(lens):
            p = torch.randint(0, vocab, (n,), generator=g).tolist()
            if w["shared_frac"] and i % round(1 / w["shared_frac"]) == 0 and n > w["shared_len"]:
                p[:w["shared_len"]] = shared
            prompts.append(p)
        return prompts

    eng = LLMEngine.random(cfg, seed=0, config=EngineConfig(
        dtype=dtype, num_blocks=w["num_blocks"], max_batch=w["max_batch"],
        max_prefill_tokens=w["chunk"], max_requests=w["max_batch"], policy=policy,
        prefix_cache=w["prefix_cache"], cuda_graphs=True))
    # The workload runs twice with the same lengths and other token ids: the first pass
    # captures the CUDA graph of every step shape, the second is timed.  No page of the first
    # pass matches a prompt of the second.
    for timed in (False, True):
        prompts = make_prompts()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i, p in enumerate(prompts):
            eng.submit_nowait(Request(p, max_new_tokens=w["new_tokens"], stop_at_eos=False,
                                      seed=i))
        records = eng.run_until_done()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if not timed:
            before = eng.state_message()
    s = eng.summarise(records, wall)
    st = eng.state_message()
    out = {
        "tok_s": round(s["throughput_tok_s"], 1), "wall_s": round(wall, 3),
        "generated": sum(r.generated_tokens for r in records),
        "ttft_p50_ms": round(s["ttft_p50"] * 1e3, 2), "ttft_p95_ms": round(s["ttft_p95"] * 1e3, 2),
        "tpot_p50_ms": round(s["tpot_p50"] * 1e3, 3),
        "preemptions": s["preemptions"], "prefix_hit_tokens": s["prefill_tokens_saved"],
        "steps": st["steps"] - before["steps"], "n_layer": cfg["n_layer"], "n_layer_full": full,
    }
    del eng
    torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------

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
    steps = min(args.steps, max_steps(prompt_len, context))
    warmup = min(args.warmup, 64)
    windows = decode_windows(prompt_len, context, steps)
    vocab = cfg["vocab_size"]
    dtype = args.dtype
    itemsize = 2 if dtype == "bfloat16" else 4
    tdt = torch.bfloat16 if dtype == "bfloat16" else torch.float32

    worst, tol = correctness_gate(torch, cfg, dtype)
    if not worst <= tol:
        print(json.dumps({"impl": "ours", "error": "correctness gate failed: the engine's "
                          "logits are off the plain implementation's", "max_diff": worst,
                          "tolerance": tol}))
        return 1

    with tempfile.TemporaryDirectory(prefix="hsb200-bench-") as d:
        write_model_dir(d, cfg, seed=0, dtype=dtype)
        model, _ = load_model(d, dtype, "cuda:0")
        page = 16
        pages_per_req = context // page
        runner = Runner(model, num_pages=64 * pages_per_req + 8, page_size=page, max_requests=64,
                        dtype=tdt, device="cuda:0", prefix_cache=False, cuda_graphs=True,
                        fused_decode=args.fused_decode)
        sampler = ClockSampler()
        sampler.start()
        ms, launches, per_window = time_decode(runner, torch, batch, windows, warmup, vocab, 1, "d")
        clocks = sampler.stop()
        value = batch * steps / (ms / 1e3)
        mean_ctx = windows_mean_context(windows)
        nbytes = decode_bytes(model, batch, mean_ctx, itemsize)
        achieved = nbytes / (ms / steps / 1e3) / 1e9

        points = {}
        for (first, _k, _r), t in zip(windows, per_window):
            points[f"decode_b{batch}_ctx{first}"] = round(batch / (t / 1e3), 1)
        for b_ in (1, 64):
            ms_b, _, _ = time_decode(runner, torch, b_, windows, warmup, vocab, 2 + b_, f"b{b_}_")
            points[f"decode_b{b_}"] = round(b_ * steps / (ms_b / 1e3), 1)
            nb = decode_bytes(model, b_, mean_ctx, itemsize)
            points[f"decode_b{b_}_hbm_frac"] = round(nb / (ms_b / steps / 1e3) / 1e9 / pk["hbm_gbs"], 4)

        pre_ms, pre_single_ms = time_prefill(runner, torch, 2, 1024, vocab, 5)
        flops = prefill_flops(cfg, 2, 1024, 2)
        if dtype == "bfloat16":
            pre_peak, pre_peak_of = pk["bf16_tflops"], "bf16 tensor, " + pk_src
        else:
            # the 32-bit path runs on the CUDA cores: 128 FMA lanes an SM at the highest clock
            props = torch.cuda.get_device_properties(0)
            pre_peak = props.multi_processor_count * 128 * 2 * props.clock_rate * 1e3 / 1e12
            pre_peak_of = "fp32 CUDA cores, nominal"
        pre_frac = flops / (pre_ms / 1e3) / (pre_peak * 1e12)
        del runner
        torch.cuda.empty_cache()
        e2e_val, h2d, d2h = time_e2e(d, torch, batch, windows, warmup, vocab, 1,
                                     batch * pages_per_req + 8, dtype, args.fused_decode)
        kernels = None
        if not args.no_kernels:
            from hetero_serve_b200.kernels import microbench
            kernels = microbench.fractions(model, cfg, pk, dtype=dtype)
        del model
        torch.cuda.empty_cache()

    for name in [w for w in args.workloads.split(",") if w and w != "none"]:
        for policy in ("prefill_first", "mixed"):
            r = run_workload(torch, name, dtype, policy, layers=args.workload_layers)
            short = "pf" if policy == "prefill_first" else "mixed"
            for k, v in r.items():
                if k in ("tok_s", "ttft_p50_ms", "ttft_p95_ms", "tpot_p50_ms", "preemptions",
                         "prefix_hit_tokens", "n_layer"):
                    points[f"{name}_{short}_{k}"] = v

    line = {
        "metric": metric_name(args),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms / steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dtype == "bfloat16" else "fp32",
        "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"{args.model} (random weights, seed 0)", "n_layer": cfg["n_layer"],
            "n_layer_full": full_layers, "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
            "head_dim": cfg["n_embd"] // cfg["n_head"], "n_inner": cfg["n_inner"],
            "vocab_size": vocab, "n_positions": cfg["n_positions"], "global_batch": batch,
            "seq_len": context, "prompt_len": prompt_len, "kv_block_size": 16,
            "parallelism": "single GPU", "residual_stream": "fp32",
            "windows": "x".join(str(f) for f, _k, _r in windows),
            "mean_context": round(mean_ctx, 1), "fused_decode": bool(args.fused_decode),
            "l2": "each step reads 0.7 GB of weights (> 126 MB L2); no flush needed",
            "peaks": pk_src,
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e_val, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(2048 / (pre_ms / 1e3), 1), "tokens": 2048,
                    "ms": round(pre_ms, 3), "frac": round(pre_frac, 4),
                    "steps_back_to_back": 4, "single_step_ms": round(pre_single_ms, 3),
                    "peak_tflops": round(pre_peak, 1), "peak_of": pre_peak_of},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "gate": {"max_diff": round(worst, 5), "tolerance": tol},
    }
    if kernels is not None:
        line["kernels"] = kernels
    print(json.dumps(line))
    return 0


def run_kernels(args):
    """Per-kernel table: time alone with a cold L2, bytes or FLOPs, fraction of the peak."""
    import torch
    from hetero_serve_b200.engine import load_model
    from hetero_serve_b200.kernels import microbench
    from hetero_serve_b200.weights import write_model_dir
    pk, pk_src = peaks()
    cfg, _ = model_config(args)
    cfg["n_layer"] = args.layers or 2
    with tempfile.TemporaryDirectory(prefix="hsb200-bench-") as d:
        write_model_dir(d, cfg, seed=0, dtype=args.dtype)
        model, _ = load_model(d, args.dtype, "cuda:0")
        rows = microbench.table(model, cfg, pk, dtype=args.dtype, batches=(1, 8, 64),
                                context=args.kernel_context)
    for r in rows:
        print(json.dumps(r))
    print(json.dumps({"peaks": pk_src, "hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"]}))
    return 0


def run_phase_marks(args):
    """`HETERO_SERVE_PHASE_MARKS=1 python bench.py --phase-marks [--batch B]`: one JSON line per
    launch of the later layers of the chain (see kernels/microbench.py:phase_marks)."""
    from hetero_serve_b200.kernels import microbench
    cfg, _ = model_config(args)
    rows = microbench.phase_marks(cfg, rows=args.batch)
    if not rows:
        print(json.dumps({"phase_marks": "unavailable: build the library with "
                                         "HETERO_SERVE_PHASE_MARKS=1"}))
        return 0
    for r in rows:
        print(json.dumps(r))
    shares = microbench.attention_phase_marks(cfg)
    if shares:
        print(json.dumps(shares))
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
        tdt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
        write_model_dir(d, cfg, seed=0, dtype=args.dtype)
        model, _ = load_model(d, args.dtype, "cuda:0")
        runner = Runner(model, num_pages=args.batch * 64 + 136, page_size=16, max_requests=64,
                        dtype=tdt, device="cuda:0", cuda_graphs=False,
                        fused_decode=args.fused_decode)
        g = torch.Generator().manual_seed(0)
        if args.one_step == "decode":
            ids = [f"r{i}" for i in range(args.batch)]
            for r in ids:
                runner.step([StepEntry(r, torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist())])
            entries = [StepEntry(r, [5], want=[0], temperature=args.temperature, top_k=args.top_k,
                                 seed=i) for i, r in enumerate(ids)]
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


def reference_root() -> str | None:
    """Where the unmodified copy of the reference lives: baseline/_ref (git-ignored).  When it
    is missing and the reference's checkout is on this machine, it is copied there."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref, "heteroserve")):
        return ref
    src = os.environ.get("HETEROSERVE_SOURCE", "/root/reference")
    if os.path.isdir(os.path.join(src, "heteroserve")):
        os.makedirs(ref, exist_ok=True)
        shutil.copytree(os.path.join(src, "heteroserve"), os.path.join(ref, "heteroserve"))
        return ref
    return None


def run_reference(args):
    if args.model != "gpt2-medium":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference arm is set up for the headline's gpt2-medium only"}))
        return 0
    ref = reference_root()
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "no copy of mneha05/hetero-serve under baseline/_ref and no checkout "
                          "to copy from"}))
        return 0
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except Exception as exc:                                    # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable":
                          f"cannot import the reference: {type(exc).__name__}: {exc}"}))
        return 0
    pk, pk_src = peaks()
    sizes = dict(n_layer=args.layers or 24, n_head=16, n_embd=1024, vocab_size=50257, n_ctx=1024)
    batch, prompt_len, context = args.batch, args.prompt_len, args.context
    steps = min(args.steps, max_steps(prompt_len, context))
    warmup = min(args.warmup, 64)
    windows = decode_windows(prompt_len, context, steps)
    sampler = ClockSampler()
    sampler.start()
    try:
        r = reference_arm.run(ref, sizes=sizes, batch=batch, windows=windows, warmup=warmup,
                              point_batches=(1, 64), prefill_shape=(2, 1024), page=16,
                              num_blocks=64 * (context // 16) + 8)
    except Exception as exc:                                    # noqa: BLE001
        sampler.stop()
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference failed while running: {type(exc).__name__}: "
                          f"{str(exc).splitlines()[-1][:300] if str(exc) else ''}"}))
        return 0
    clocks = sampler.stop()
    if "unavailable" in r:
        print(json.dumps({"impl": "reference", "unavailable": r["unavailable"]}))
        return 0
    cfg = dict(n_embd=1024, n_inner=4096, n_layer=sizes["n_layer"], vocab_size=50257)
    flops = prefill_flops(cfg, 2, 1024, 2)
    pre_ms = r["prefill_ms"]
    max_blocks = context // 16
    line = {
        "metric": METRIC, "value": round(r["value"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(r["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"float32": "fp32", "float16": "fp16"}[r["dtype"]], "data": "synthetic",
        "impl": "reference", "same_config": sizes["n_layer"] == 24,
        "config": {
            "model": "gpt2-medium (the reference's synthetic_gpt2, seed 0)",
            "n_layer": sizes["n_layer"], "n_layer_full": 24, "n_embd": 1024, "n_head": 16,
            "head_dim": 64, "n_inner": 4096, "vocab_size": 50257, "n_positions": 1024,
            "global_batch": batch, "seq_len": context, "prompt_len": prompt_len,
            "kv_block_size": 16, "parallelism": "single GPU", "kv_dtype": r["kv_dtype"],
            "windows": "x".join(str(f) for f, _k, _r in windows),
            "kernel_backend": r["kernel_backend"], "prefill_attention": r["prefill_attention"],
            "peaks": pk_src,
        },
        "clocks": clocks,
        "e2e": {"value": round(r["e2e"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": batch * (8 + 8 + 4 + 8) + batch * max_blocks * 4,
                "d2h_bytes_per_step": batch * 50257 * 4},
        "gpu_launches": 0,
        "prefill": {"value": round(2048 / (pre_ms / 1e3), 1), "tokens": 2048,
                    "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "points": r["points"],
        "by_dtype": r["dtypes"],
        "kernel_backend": r["kernel_backend"], "kernel_build_error": r["kernel_build_error"],
        "kernel_build_s": r["kernel_build_s"],
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="gpt2-medium",
                    help="preset of the architecture to time (this engine's arm; default: the "
                         "headline's gpt2-medium)")
    ap.add_argument("--prompt-len", dest="prompt_len", type=int, default=512)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit path (CUDA cores only)")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (0: all); both numbers "
                         "are named in `config`")
    ap.add_argument("--workloads", default="large,xl",
                    help="serving workloads run through LLMEngine after the timed steps "
                         "(comma-separated: large, xl; 'none' skips them)")
    ap.add_argument("--workload-layers", dest="workload_layers", type=int, default=0,
                    help="fewer layers for the workloads (0: all)")
    ap.add_argument("--fused-decode", dest="fused_decode", action="store_true",
                    help="decode steps of up to 16 tokens as one persistent kernel (off by "
                         "default: it measures slower than the layer-by-layer path)")
    ap.add_argument("--no-kernels", dest="no_kernels", action="store_true",
                    help="skip the per-kernel roofline fractions")
    ap.add_argument("--kernel-context", dest="kernel_context", type=int, default=768,
                    help="context length of the decode attention in the --kernels table")
    ap.add_argument("--kernels", action="store_true",
                    help="print the per-kernel table (one JSON object a kernel) and exit")
    ap.add_argument("--temperature", type=float, default=0.0,
                    help="with --one-step decode: sample with this temperature (0: greedy)")
    ap.add_argument("--top-k", dest="top_k", type=int, default=0,
                    help="with --one-step decode: restrict sampling to the k largest")
    ap.add_argument("--phase-marks", dest="phase_marks", action="store_true",
                    help="print the few-row linears' own time marks inside a CUDA graph (needs a "
                         "library built with HETERO_SERVE_PHASE_MARKS=1) and exit")
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
    if args.kernels:
        return run_kernels(args)
    if args.phase_marks:
        return run_phase_marks(args)
    if args.one_step:
        return run_one_step(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
