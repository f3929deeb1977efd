"""Each kernel of a decode step and of a prefill step alone, at the step's shapes, against its
roofline — in the manner of the reference's kernel benchmark (scripts/bench_kernel.py:61-221:
time each kernel, print GB/s against a peak, and refuse to time a kernel whose output is off
its torch reference, :193-201).

How a kernel is timed.  Its weights (or cache pages) are allocated in as many copies as it
takes to exceed twice the L2 (126 MB), one launch per copy is captured into a CUDA graph, and
the graph is replayed: every launch reads operands no earlier launch left in the L2, as in a
real step, where the layers' weights stream through once.  Small activations stay in the L2,
as they do in a step.  The time of a launch is the graph's time divided by its launches
(device time, CUDA events, median of the replays) and so includes the gap between
back-to-back launches, which is part of what a kernel costs in a step.

Rooflines: kernels that stream weights or cache pages are held against the HBM peak with the
bytes they must read (weights once, the live requests' pages, large activations), the
contractions of a prefill step against the bfloat16 tensor peak with their FLOPs.  Before a
kernel is timed its output is compared with plain PyTorch arithmetic in float32 on the same
operands; if it is off, the row carries the difference and no time.
"""

from __future__ import annotations

import math
import statistics

import torch

from .ops import AttentionGeometry, CudaOps

L2_BYTES = 126 * 2 ** 20
GATE_TOL = {torch.bfloat16: 4e-2, torch.float32: 2e-3}


def _copies(nbytes: int, lo: int = 2, hi: int = 160) -> int:
    return max(lo, min(hi, math.ceil(2 * L2_BYTES / max(1, nbytes))))


def _time_graph(launch, n: int, replays: int = 7) -> float:
    """Microseconds per launch: ``launch(i)`` for i in range(n) captured once, replayed."""
    for i in range(min(n, 3)):
        launch(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / n)
    return statistics.median(times)


def _act(v, act):
    if act == "gelu_tanh":
        return torch.nn.functional.gelu(v, approximate="tanh")
    if act == "gelu_erf":
        return torch.nn.functional.gelu(v)
    return v


def _layernorm(x, g, b, eps):
    mu = x.mean(-1, keepdim=True)
    c = x - mu
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * g + b


class _Bench:
    def __init__(self, cfg, peaks, dtype, device):
        self.cfg, self.peaks = cfg, peaks
        self.dt = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.item = 2 if self.dt == torch.bfloat16 else 4
        self.dev = torch.device(device)
        self.ops = CudaOps(self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.ops.status = self.status
        self.E, self.H = cfg["n_embd"], cfg["n_head"]
        self.D = self.E // self.H
        self.I = cfg["n_inner"] or 4 * self.E
        self.V = cfg["vocab_size"]
        self.eps = cfg.get("layer_norm_epsilon", 1e-5)
        self.gen = torch.Generator(device=self.dev).manual_seed(0)
        self.rows: list[dict] = []

    def rand(self, *shape, scale=1.0, dtype=None):
        t = torch.randn(*shape, device=self.dev, generator=self.gen) * scale
        return t.to(dtype or self.dt)

    def record(self, step, kernel, us, gate, *, nbytes=0, flops=0, bound):
        row = {"step": step, "kernel": kernel, "gate_max_diff": round(gate, 5)}
        if us is None:
            row["refused"] = "output is off the plain reference: not timed"
        else:
            row["us"] = round(us, 2)
            if bound == "hbm":
                ach = nbytes / (us * 1e-6) / 1e9
                row.update(bound="hbm", bytes=int(nbytes), achieved_gbs=round(ach, 1),
                           frac=round(ach / self.peaks["hbm_gbs"], 4))
            else:
                ach = flops / (us * 1e-6) / 1e12
                row.update(bound="tensor", flops=int(flops), achieved_tflops=round(ach, 1),
                           frac=round(ach / self.peaks["bf16_tflops"], 4))
        self.rows.append(row)

    def gate_ok(self, got, want) -> tuple[bool, float]:
        diff = float((got.float() - want.float()).abs().max())
        ok = math.isfinite(diff) and diff <= GATE_TOL[self.dt] * max(1.0, float(want.abs().max()))
        return ok, diff

    # -- linears ------------------------------------------------------------------------
    def linear(self, step, kernel, M, N, K, *, act="none", norm=False, residual=False,
               out_dtype=None, bound="hbm"):
        ops = self.ops
        out_dtype = out_dtype or (torch.float32 if residual else self.dt)
        n = _copies(N * K * self.item) if bound == "hbm" else 4
        w = self.rand(n, N, K, scale=K ** -0.5)
        bias = self.rand(N, dtype=torch.float32)
        out = torch.zeros(M, N, device=self.dev, dtype=out_dtype)
        res0 = self.rand(M, N, dtype=torch.float32) if residual else None
        if norm:
            x = self.rand(M, K, dtype=torch.float32) * 3 + 1
            g, b = self.rand(K, dtype=torch.float32), self.rand(K, dtype=torch.float32)
            h = torch.empty(M, K, device=self.dev, dtype=self.dt)
            a_ref = _layernorm(x, g, b, self.eps).to(self.dt).float()

            def launch(i):
                ops.norm_linear(out, h, x, g, b, self.eps, w[i % n], bias, act)
        else:
            a = self.rand(M, K)
            a_ref = a.float()

            def launch(i):
                if residual:
                    ops.linear(out, a, w[i % n], bias, act=act, residual=out)
                else:
                    ops.linear(out, a, w[i % n], bias, act=act)
        if residual:
            out.copy_(res0)
        launch(0)
        want = _act(a_ref @ w[0].float().T + bias, act)
        if residual:
            want = want + res0
        ok, diff = self.gate_ok(out, want)
        us = _time_graph(launch, n) if ok else None
        act_bytes = M * K * (4 if norm else self.item) + M * N * out.element_size() * (2 if residual else 1)
        self.record(step, kernel, us, diff, nbytes=N * K * self.item + act_bytes,
                    flops=2 * M * N * K, bound=bound)

    # -- attention ----------------------------------------------------------------------
    def _cache(self, lens, new, n_entries):
        """Pools [entries, pages, 2, H, 16, D] with random keys and values for the cached
        positions, a block table, and the step's qkv rows."""
        PS, H, D = 16, self.H, self.D
        pages_per = [-(-n // PS) for n in lens]
        n_pages = sum(pages_per) + 1
        max_pages = max(pages_per) + 1
        table = torch.full((len(lens), max_pages), -1, dtype=torch.int32)
        at = 0
        for r, k in enumerate(pages_per):
            table[r, :k] = torch.arange(at, at + k, dtype=torch.int32)
            at += k
        pool = self.rand(n_entries, n_pages, 2, H, PS, D)
        T = sum(new)
        qkv = self.rand(T, 3 * self.E)
        pos, req = [], []
        for r, (n, k) in enumerate(zip(lens, new)):
            pos += list(range(n - k, n))
            req += [r] * k
        geom = AttentionGeometry(H, H, D, PS, n_pages, max_pages, 0, self.E, 2 * self.E, 3 * self.E)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.dev)   # noqa: E731
        host = [(f"r{r}", r, n - k, k) for r, (n, k) in enumerate(zip(lens, new))]
        return geom, qkv, pool, table.to(self.dev), i32(pos), i32(req), host

    def _attention_reference(self, qkv, pool, table, lens, new, geom, scale):
        H, D, PS = geom.n_heads, geom.head_dim, geom.page_size
        out, t = [], 0
        for r, (n, k) in enumerate(zip(lens, new)):
            pos = torch.arange(n, device=self.dev)
            pages = table[r, pos // PS].long()
            keys = pool[pages, 0, :, pos % PS, :].float()
            vals = pool[pages, 1, :, pos % PS, :].float()
            q = qkv[t:t + k, :H * D].view(k, H, D).float()
            s = torch.einsum("qhd,nhd->hqn", q, keys) * scale
            qpos = torch.arange(n - k, n, device=self.dev)
            s = s.masked_fill((pos[None, :] > qpos[:, None])[None], float("-inf"))
            out.append(torch.einsum("hqn,nhd->qhd", torch.softmax(s, -1), vals).reshape(k, H * D))
            t += k
        return torch.cat(out)

    def attention(self, step, kernel, lens, new, bound):
        ops = self.ops
        kv_bytes = sum(lens) * 2 * self.E * self.item
        n = _copies(kv_bytes, hi=48) if bound == "hbm" else 2
        geom, qkv, pool, table, pos, req, host = self._cache(lens, new, n)
        T = qkv.shape[0]
        plan = ops.make_plan(host, T, 16) if self.dt == torch.bfloat16 else None
        out = torch.zeros(T, self.E, device=self.dev, dtype=self.dt)
        scale = 1.0 / math.sqrt(self.D)

        def launch(i):
            ops.attention_append(out, qkv, pool[i % n], table, pos, req, geom, scale, self.status,
                                 plan, True)
        launch(0)
        want = self._attention_reference(qkv, pool[0], table, lens, new, geom, scale)
        ok, diff = self.gate_ok(out, want)
        us = _time_graph(launch, n) if ok else None
        flops = sum(4 * self.E * (k * (n_ - k) + k * (k + 1) // 2) for n_, k in zip(lens, new))
        self.record(step, kernel, us, diff, nbytes=kv_bytes + T * 4 * self.E * self.item,
                    flops=flops, bound=bound)

    # -- the rest -----------------------------------------------------------------------
    def layernorm(self, step, kernel, M):
        x = self.rand(4, M, self.E, dtype=torch.float32) * 3 + 1
        g, b = self.rand(self.E, dtype=torch.float32), self.rand(self.E, dtype=torch.float32)
        out = torch.empty(M, self.E, device=self.dev, dtype=self.dt)

        def launch(i):
            self.ops.layernorm(out, x[i % 4], g, b, self.eps)
        launch(0)
        ok, diff = self.gate_ok(out, _layernorm(x[0], g, b, self.eps))
        us = _time_graph(launch, 8) if ok else None
        self.record(step, kernel, us, diff, nbytes=M * self.E * (4 + self.item), bound="hbm")

    def head_and_sample(self, step, B):
        ops = self.ops
        n = _copies(self.V * self.E * self.item, hi=4)
        w = self.rand(n, self.V, self.E, scale=self.E ** -0.5)
        hf = self.rand(B, self.E)
        logits = torch.empty(B, self.V, device=self.dev, dtype=torch.float32)

        def launch(i):
            ops.linear(logits, hf, w[i % n])
        launch(0)
        ok, diff = self.gate_ok(logits, hf.float() @ w[0].float().T)
        us = _time_graph(launch, n) if ok else None
        self.record(step, "head", us, diff, nbytes=self.V * self.E * self.item + B * self.V * 4,
                    flops=2 * B * self.V * self.E, bound="hbm")
        tokens = torch.empty(B + 1, dtype=torch.int32, device=self.dev)
        zeros = torch.zeros(B, dtype=torch.int32, device=self.dev)
        temp = torch.zeros(B, dtype=torch.float32, device=self.dev)

        def sample(i):
            ops.sample(tokens, logits, temp, zeros, zeros, zeros, zeros)
        sample(0)
        same = bool((tokens[:B].long() == logits.argmax(-1)).all())
        us = _time_graph(sample, 8) if same else None
        self.record(step, "sample (greedy)", us, 0.0 if same else float("inf"),
                    nbytes=B * self.V * 4, bound="hbm")


def table(model, cfg, peaks, dtype="bfloat16", batches=(8,), context=768, device="cuda:0"):
    """Rows (dictionaries) for the kernels of a decode step at each batch size and of a prefill
    step of 2 x 1,024 tokens.  ``model`` is not used for its weights (operands are allocated
    here, in copies); it is accepted so that callers pass what they have."""
    b = _Bench(cfg, peaks, dtype, device)
    E, I = b.E, b.I
    fast = b.dt == torch.bfloat16
    for B in batches:
        s = f"decode_b{B}"
        b.linear(s, "layernorm + qkv", B, 3 * E, E, norm=fast)
        b.attention(s, "attention (+ append)", [context] * B, [1] * B, "hbm")
        b.linear(s, "attention out + residual", B, E, E, residual=True)
        b.linear(s, "layernorm + fc + gelu", B, I, E, act="gelu_tanh", norm=fast)
        b.linear(s, "mlp out + residual", B, E, I, residual=True)
        b.head_and_sample(s, B)
    s, T = "prefill_2048", 2048
    bound = "tensor" if fast else "hbm"
    b.layernorm(s, "layernorm", T)
    b.linear(s, "qkv", T, 3 * E, E, bound=bound)
    b.attention(s, "attention (+ append)", [1024, 1024], [1024, 1024], bound)
    b.linear(s, "attention out + residual", T, E, E, residual=True, bound=bound)
    b.linear(s, "fc + gelu", T, I, E, act="gelu_tanh", bound=bound)
    b.linear(s, "mlp out + residual", T, E, I, residual=True, bound=bound)
    return b.rows


def fractions(model, cfg, peaks, dtype="bfloat16", device="cuda:0") -> dict:
    """Flat ``{"step.kernel": fraction of its peak}`` for a decode step at batch 8 and a
    prefill step (a kernel that failed its comparison carries ``None``)."""
    return {f"{r['step']}.{r['kernel']}": r.get("frac") for r in
            table(model, cfg, peaks, dtype, batches=(8,), device=device)}


def phase_marks(cfg, rows: int = 8, layers: int = 8, device: str = "cuda:0") -> list[dict]:
    """The four few-row linears of a decode layer (LayerNorm + QKV, attention out + residual,
    LayerNorm + fc + GELU, MLP out + residual) chained ``layers`` times in one CUDA graph with
    programmatic dependent launch, weights rotating through DRAM, and the kernel's own time
    marks read back: for every launch of the later layers, when its LAST CTA passed the
    dependency wait, had its activations staged, had issued its MMAs and had finished, in ns
    after the last CTA of the launch before.  Needs a library built with phase marks
    (``HETERO_SERVE_PHASE_MARKS=1``); the product build has none and returns an empty list."""
    import ctypes

    from .ops import CudaOps
    ops = CudaOps(device)
    if not hasattr(ops.lib, "hs_set_timing_buffer"):
        return []
    ops.lib.hs_set_timing_buffer.argtypes = [ctypes.c_void_p]
    E = cfg["n_embd"]
    inner = cfg.get("n_inner") or 4 * E
    slots = 512
    bufs = torch.zeros(layers * 4, slots * 8, dtype=torch.int64, device=device)
    ws = [dict(qkv=torch.randn(3 * E, E, device=device).bfloat16(),
               o=torch.randn(E, E, device=device).bfloat16(),
               fc=torch.randn(inner, E, device=device).bfloat16(),
               p2=torch.randn(E, inner, device=device).bfloat16()) for _ in range(layers)]
    x = torch.randn(rows, E, device=device)
    g, b = torch.randn(E, device=device), torch.randn(E, device=device)
    h = torch.empty(rows, E, device=device, dtype=torch.bfloat16)
    qkv = torch.empty(rows, 3 * E, device=device, dtype=torch.bfloat16)
    att = torch.randn(rows, E, device=device).bfloat16()
    mid = torch.empty(rows, inner, device=device, dtype=torch.bfloat16)
    bq, bo, bf = (torch.randn(n, device=device) for n in (3 * E, E, inner))

    def layer(i, armed):
        w = ws[i]

        def arm(k):
            ops.lib.hs_set_timing_buffer(bufs[i * 4 + k].data_ptr() if armed else None)
        arm(0); ops.norm_linear(qkv, h, x, g, b, 1e-5, w["qkv"], bq)
        arm(1); ops.linear(x, att, w["o"], bo, residual=x)
        arm(2); ops.norm_linear(mid, h, x, g, b, 1e-5, w["fc"], bf, act="gelu_tanh")
        arm(3); ops.linear(x, mid, w["p2"], bo, residual=x)

    for i in range(layers):
        layer(i, False)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(layers):
            layer(i, True)
    ops.lib.hs_set_timing_buffer(None)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    marks = bufs.view(layers * 4, slots, 8).cpu()
    names = ["layernorm + qkv", "attention out + residual", "layernorm + fc + gelu",
             "mlp out + residual"]
    out, prev_end = [], None
    for j in range(layers * 4):
        t = marks[j]
        t = t[t[:, 0] > 0]
        if t.shape[0] == 0:
            return []                                   # built without marks
        first = int(t[:, 0].min())                      # the first CTA to start (may be negative:
        wait, staged, mma, end = (int(t[:, k].max()) for k in (1, 2, 3, 4))   # it overlaps)
        if prev_end is not None and j >= 8:             # the first two layers warm up
            out.append({"kernel": names[j % 4], "ctas": int(t.shape[0]),
                        "first_start_ns": first - prev_end, "wait_over_ns": wait - prev_end, "staged_ns": staged - wait,
                        "mma_ns": mma - staged, "end_ns": end - mma, "total_ns": end - prev_end})
        prev_end = end
    return out


def attention_phase_marks(cfg, n_seqs: int = 2, seq_len: int = 1024, device: str = "cuda:0") -> dict:
    """The prompt attention on tcgen05 over `n_seqs` whole prompts of `seq_len` tokens with the
    kernel's own cycle counters on (a library built with ``HETERO_SERVE_PHASE_MARKS=1``): what
    one softmax thread of every CTA spends in each phase of its loop, as mean cycles per CTA and
    as shares.  Empty when the library has no counters or the head size is not the kernel's."""
    import ctypes

    b = _Bench(cfg, {"hbm_gbs": 1.0, "bf16_tflops": 1.0}, "bfloat16", device)
    ops = b.ops
    if not hasattr(ops.lib, "hs_set_timing_buffer") or b.D != 64:
        return {}
    ops.lib.hs_set_timing_buffer.argtypes = [ctypes.c_void_p]
    lens = [seq_len] * n_seqs
    geom, qkv, pool, table, pos, req, host = b._cache(lens, lens, 1)
    T = qkv.shape[0]
    plan = ops.make_plan(host, T, 16)
    out = torch.zeros(T, b.E, device=b.dev, dtype=b.dt)
    scale = 1.0 / math.sqrt(b.D)
    for _ in range(3):
        ops.attention_append(out, qkv, pool[0], table, pos, req, geom, scale, b.status, plan, True)
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(b.dev).multi_processor_count
    buf = torch.zeros(sms * 8, dtype=torch.int64, device=b.dev)
    ops.lib.hs_set_timing_buffer(buf.data_ptr())
    ops.attention(out, qkv, pool[0], table, pos, req, geom, scale, b.status, plan)
    torch.cuda.synchronize()
    ops.lib.hs_set_timing_buffer(None)
    t = buf.view(sms, 8).cpu().double()
    total = float(t.sum(1).mean())
    if total <= 0:
        return {}
    names = ["wait for S", "row maximum", "exponentials", "wait for P V, add O_tile", "write P",
             "loop", "last O_tile and output", "wait for an item's first S"]
    return {"kernel": "attention_prefill_tc", "tokens": T, "cycles_per_cta": round(total),
            "shares": {n: round(float(t[:, i].mean()) / total, 4) for i, n in enumerate(names)}}
