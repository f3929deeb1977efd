"""The reference arm of bench.py: mneha05/hetero-serve itself, unmodified, driven
through its own public classes for the workload bench.py measures.

Nothing of hetero_serve_b200 is imported here.  The stock path on a CUDA device is

* ``synthetic_gpt2(ModelConfig(...))``           heteroserve/model/weights.py:103-142
* ``TorchEngine(weights, cfg, "cuda:0", dtype)`` heteroserve/model/torch_engine.py:28-70
* ``TorchBlockAllocator(KVConfig, cfg, device)`` heteroserve/kv/torch_blocks.py:30-48
* ``allocate`` / ``grow``                        heteroserve/kv/blocks.py:168-209
* ``prefill_paged``                              heteroserve/model/torch_engine.py:257-321
* ``decode_batch_paged``                         heteroserve/model/torch_engine.py:195-253
* ``sample_token`` on the returned host logits   heteroserve/worker/worker.py:43-50

used in the order the reference's worker uses them (worker.py:599-703).  Its attention
kernels are compiled by the reference at first use (``load_inline``); when that fails it
falls back to its own torch attention and records why — ``kernel_backend`` in the output
says which ran.
"""

from __future__ import annotations

import os
import statistics
import sys
import time


def _import_reference(ref_root: str):
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    import numpy as np
    import torch
    from heteroserve.config import KVConfig, ModelConfig
    from heteroserve.kv.torch_blocks import TorchBlockAllocator
    from heteroserve.model import paged_attn
    from heteroserve.model.torch_engine import TorchEngine
    from heteroserve.model.weights import synthetic_gpt2
    from heteroserve.worker.worker import sample_token
    return dict(np=np, torch=torch, KVConfig=KVConfig, ModelConfig=ModelConfig,
                TorchBlockAllocator=TorchBlockAllocator, paged_attn=paged_attn,
                TorchEngine=TorchEngine, synthetic_gpt2=synthetic_gpt2,
                sample_token=sample_token)


class _Seq:
    def __init__(self, prompt, block_ids):
        self.prompt = prompt
        self.block_ids = block_ids
        self.out: list[int] = []
        self.n_kv = 0
        self.seed = 0


def _start(R, engine, alloc, prompts):
    """Admission and prefill as the worker does them: allocate the prompt's blocks, one
    prefill call per sequence, first token from its logits (worker.py:378-416, 599-657)."""
    np = R["np"]
    seqs = []
    for p in prompts:
        a = alloc.allocate(p)
        s = _Seq(p, list(a.block_ids))
        logits = engine.prefill_paged(np.asarray(p, dtype=np.int64), 0, s.block_ids, alloc)
        s.n_kv = len(p)
        s.out.append(R["sample_token"](logits, 0.0, 0, np.random.default_rng(s.seed)))
        seqs.append(s)
    return seqs


def _decode_step(R, engine, alloc, seqs):
    """One decode step as the worker's ``_decode`` (worker.py:659-703)."""
    np = R["np"]
    for s in seqs:
        alloc.grow(s.block_ids, s.n_kv + 1)
    ctx = [s.prompt + s.out for s in seqs]
    toks = np.array([c[s.n_kv] for c, s in zip(ctx, seqs)], dtype=np.int64)
    pos = np.array([s.n_kv for s in seqs], dtype=np.int64)
    logits = engine.decode_batch_paged(toks, pos, [s.block_ids for s in seqs], pos, alloc)
    for i, s in enumerate(seqs):
        s.n_kv += 1
        rng = np.random.default_rng(s.seed + s.n_kv)
        s.out.append(R["sample_token"](logits[i], 0.0, 0, rng))
    return logits


def _decode_windows(R, engine, alloc, batch, windows, warmup, vocab, seed):
    """Times the windows of a decode trajectory; returns (device ms, wall s, steps, finite)."""
    np, torch = R["np"], R["torch"]
    rng = np.random.default_rng(seed)
    dev_ms = wall = 0.0
    steps = 0
    finite = True
    for first, k, reps in windows:
        prompts = rng.integers(0, vocab, (batch, first - warmup - 1)).tolist()
        seqs = _start(R, engine, alloc, prompts)
        for _ in range(warmup):
            _decode_step(R, engine, alloc, seqs)
        d_ms, w_s = [], []
        for _ in range(reps):
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            a.record()
            for _ in range(k):
                logits = _decode_step(R, engine, alloc, seqs)
            b.record()
            torch.cuda.synchronize()
            w_s.append(time.perf_counter() - t0)
            d_ms.append(a.elapsed_time(b))
        finite = finite and bool(np.isfinite(logits).all())
        dev_ms += statistics.median(d_ms)
        wall += statistics.median(w_s)
        steps += k
        for s in seqs:
            alloc.free_sequence(s.block_ids)
    return dev_ms, wall, steps, finite


def _prefill(R, engine, alloc, n_seqs, seq_len, vocab, seed, reps=3, warm=1):
    np, torch = R["np"], R["torch"]
    rng = np.random.default_rng(seed)
    prompts = rng.integers(0, vocab, (n_seqs, seq_len)).tolist()
    times = []
    for it in range(warm + reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        held = []
        for p in prompts:
            a = alloc.allocate(p)
            engine.prefill_paged(np.asarray(p, dtype=np.int64), 0, list(a.block_ids), alloc)
            held.append(a.block_ids)
        torch.cuda.synchronize()
        if it >= warm:
            times.append((time.perf_counter() - t0) * 1e3)
        for b in held:
            alloc.free_sequence(b)
    return statistics.median(times)


def run(ref_root: str, *, sizes: dict, batch: int, windows, warmup: int, point_batches,
        prefill_shape, page: int, num_blocks: int) -> dict:
    """Runs the reference on ``cuda:0``; returns the fields bench.py prints.  ``sizes`` holds
    n_layer, n_head, n_embd, vocab_size and n_ctx; ``windows`` is bench.py's list of
    ``(first context, steps, repeats)``."""
    # build artefacts of the reference's kernels stay beside the copy of the reference
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(ref_root, ".torch_extensions"))
    R = _import_reference(ref_root)
    torch = R["torch"]
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device: the reference's paged path needs one"}
    cfg = R["ModelConfig"](n_layer=sizes["n_layer"], n_head=sizes["n_head"],
                           n_embd=sizes["n_embd"], vocab_size=sizes["vocab_size"],
                           n_ctx=sizes["n_ctx"])
    t0 = time.perf_counter()
    backend = R["paged_attn"].which_backend()        # compiles the decode kernel
    build_error = R["paged_attn"].build_error()
    build_s = time.perf_counter() - t0
    weights = R["synthetic_gpt2"](cfg, seed=0)
    vocab = cfg.vocab_size
    out: dict = {"kernel_backend": backend, "kernel_build_error": build_error,
                 "kernel_build_s": round(build_s, 1), "kv_dtype": "float16", "dtypes": {}}
    best = None
    for dtype in ("float32", "float16"):
        engine = R["TorchEngine"](weights, cfg, "cuda:0", dtype=dtype)
        alloc = R["TorchBlockAllocator"](R["KVConfig"](block_size=page, num_blocks=num_blocks),
                                         cfg, "cuda:0")
        dev_ms, wall, steps, finite = _decode_windows(R, engine, alloc, batch, windows, warmup,
                                                      vocab, 1)
        rec = {"value": batch * steps / (dev_ms / 1e3), "ms_per_step": dev_ms / steps,
               "e2e": batch * steps / wall, "steps": steps, "finite_logits": finite}
        out["dtypes"][dtype] = {k: (round(v, 4) if isinstance(v, float) else v)
                                for k, v in rec.items()}
        if best is None or rec["e2e"] > best[1]["e2e"]:
            best = (dtype, rec, engine, alloc)
        else:
            del engine, alloc
        torch.cuda.empty_cache()
    dtype, rec, engine, alloc = best
    out.update(dtype=dtype, value=rec["value"], ms_per_step=rec["ms_per_step"],
               e2e=rec["e2e"], steps=rec["steps"])
    points = {}
    for b in point_batches:
        d_ms, _w, st, _f = _decode_windows(R, engine, alloc, b, windows, warmup, vocab, 2 + b)
        points[f"decode_b{b}"] = round(b * st / (d_ms / 1e3), 1)
    out["points"] = points
    n_seqs, seq_len = prefill_shape
    out["prefill_ms"] = _prefill(R, engine, alloc, n_seqs, seq_len, vocab, 5)
    # which prefill attention the reference chose (torch_engine.py:279-284)
    try:
        from heteroserve.model import paged_attn_wmma
        out["prefill_attention"] = ("wmma" if paged_attn_wmma.supports(
            alloc.block_size, cfg.head_dim, alloc.torch_dtype) else "scalar or torch")
    except Exception as exc:                       # noqa: BLE001
        out["prefill_attention"] = f"unknown ({type(exc).__name__})"
    return out
