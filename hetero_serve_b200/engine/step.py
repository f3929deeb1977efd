"""The step function: one forward pass over a batch of (request, its next tokens).

A batch is flat and ragged.  Each entry brings the next tokens of one request — a
portion of its prompt, cut anywhere, or a single decoded token — and the places among
them whose logits are wanted.  :meth:`Runner.step` runs exactly these tokens, as one
batch, against the pages earlier steps left in the cache, and returns the logits at
the wanted places (and, on request, tokens sampled from them on the device).

The reference has four entry points instead (``prefill``, ``decode_batch``,
``prefill_paged``, ``decode_batch_paged``, heteroserve/model/torch_engine.py:94-321) and
never mixes a prompt portion with decoded tokens in one pass
(heteroserve/worker/worker.py:580-591); the order inside a layer is the same
(torch_engine.py:297-317).

Host to device traffic per step is ONE copy of a packed int32 block (token ids,
positions, the request of each token, block tables, wanted rows, sampling
parameters); device to host is one small copy of the sampled tokens and the status
word, or nothing at all when the caller only wants device logits.  With
``cuda_graphs`` the kernels of a step are captured once per size class and replayed.
"""

from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, GroupSpec, OutOfPages
from ..kernels.ops import size_class

STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a position outside the table",
               4: "a page number outside the pool", 8: "a kernel pipeline timed out"}


class StepError(RuntimeError):
    pass


# As the first token of an entry: "the token the device sampled for this request last", which
# the step reads from device memory.  It lets a decode step be launched before the host has
# read the previous step's tokens.
FROM_DEVICE = -1
HOT_SHAPE_USES = 32     # steps of one shape before it gets a second metadata block and graph


@dataclass
class StepEntry:
    """The next tokens of one request, and which of their logits are wanted."""

    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # used only when the step samples on the device
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 0


@dataclass
class StepResult:
    logits: torch.Tensor | None          # [n_wanted, vocab] float32 on the device
    tokens: torch.Tensor | None          # [n_wanted] int32 on the device (if sampled)
    rows: list[tuple[Hashable, int]]     # (request, index among its tokens) per wanted row
    n_tokens: int = 0
    _with_status: torch.Tensor | None = None
    _runner: "Runner | None" = None
    _host: torch.Tensor | None = None
    _copied: "torch.cuda.Event | None" = None
    _block: int | None = None            # the metadata block of a step whose copies use side streams

    def start_fetch(self) -> None:
        """Enqueue the device-to-host copy of the sampled tokens (and the status word) behind
        the step, without waiting for it.  Must be called before the next step is launched: the
        device buffer is reused."""
        if self._with_status is None or self._host is not None:
            return
        self._host, self._copied = self._runner._fetch(self._with_status, self._block)

    def tokens_host(self) -> list[int]:
        """The sampled tokens as Python ints: one device-to-host copy that also brings the
        kernels' status word, which is checked."""
        if self._with_status is None:
            return []
        self.start_fetch()
        if self._copied is not None:
            self._copied.synchronize()
        n = self.tokens.shape[0]
        host = self._host.tolist()          # [bucketed rows..., status word]
        if host[-1]:
            self._runner.raise_status(host[-1])
        return host[:n]


@dataclass
class CacheView:
    """What a mixer sees of the cache for one layer call."""

    pool: torch.Tensor           # [pages, 2, kv_heads, page_size, head_dim]
    table: torch.Tensor          # [requests, max_pages] int32: this batch's block tables
    page_size: int
    num_pages: int
    writes: bool
    group: int


class Layout:
    """Offsets of the sections of the packed int32 metadata block for one size class."""

    def __init__(self, T: int, R: int, W: int, max_pages: Sequence[int], plan_ints: int):
        self.T, self.R, self.W = T, R, W
        self.max_pages = tuple(max_pages)
        off = 0

        def take(n):
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4          # keep every section 16-byte aligned
            return start

        self.tok_ids, self.tok_pos, self.tok_req = take(T), take(T), take(T)
        self.req_start, self.req_len, self.req_ctx, self.req_slot = (take(R), take(R), take(R),
                                                                     take(R))
        self.logit_rows = take(W)
        self.samp_temp, self.samp_topk = take(W), take(W)
        self.samp_seed_lo, self.samp_seed_hi, self.samp_pos = take(W), take(W), take(W)
        self.samp_slot = take(W)
        self.tables = [take(R * mp) for mp in self.max_pages]
        self.plan = take(plan_ints)
        self.plan_ints = plan_ints
        self.total = off


class StepContext:
    """Everything a part may touch while a step runs."""

    def __init__(self, runner: "Runner", layout: Layout, meta: torch.Tensor):
        self.runner = runner
        self.ops = runner.ops
        self.dtype = runner.dtype
        self.device = runner.device
        self.status = runner.status
        self.layout = layout
        self.meta = meta
        L = layout
        self.n_rows, self.n_requests, self.n_logit_rows = L.T, L.R, L.W
        self.tok_ids = meta[L.tok_ids:L.tok_ids + L.T]
        self.tok_pos = meta[L.tok_pos:L.tok_pos + L.T]
        self.tok_req = meta[L.tok_req:L.tok_req + L.T]
        self.req_start = meta[L.req_start:L.req_start + L.R]
        self.req_len = meta[L.req_len:L.req_len + L.R]
        self.req_ctx = meta[L.req_ctx:L.req_ctx + L.R]
        self.req_slot = meta[L.req_slot:L.req_slot + L.R]
        self.logit_rows = meta[L.logit_rows:L.logit_rows + L.W]
        self.samp_temp = meta[L.samp_temp:L.samp_temp + L.W].view(torch.float32)
        self.samp_topk = meta[L.samp_topk:L.samp_topk + L.W]
        self.samp_seed_lo = meta[L.samp_seed_lo:L.samp_seed_lo + L.W]
        self.samp_seed_hi = meta[L.samp_seed_hi:L.samp_seed_hi + L.W]
        self.samp_pos = meta[L.samp_pos:L.samp_pos + L.W]
        self.samp_slot = meta[L.samp_slot:L.samp_slot + L.W]
        self.feedback = runner.feedback
        self.tables = [meta[o:o + L.R * mp].view(L.R, mp)
                       for o, mp in zip(L.tables, L.max_pages)]
        self.fused = runner.fused   # the whole-step decode kernel's plan for this model, if any
        self.fused_tokens = None   # greedy tokens a fused step left (with the status word)
        self.greedy_only = False   # no wanted row of this step samples with a temperature
        self.sampling = False      # the step chooses tokens (a head may then choose them itself)
        self.tokens_name = "sampled"   # the workspace buffer the step's tokens go to
        self.plan = None          # work lists for the specialised attention kernels, if any
        self.position = None      # the model's position encoding (set by Model.forward)
        self.call_index: int | None = None
        # host-side view of the batch for parts written in plain PyTorch
        self.host: list[tuple[Hashable, int, int, int]] = []   # (req, slot, start, n)

    def buffer(self, name: str, shape, dtype) -> torch.Tensor:
        """A temporary tensor that lives until the next step (never allocated twice for the
        same use and size class)."""
        return self.runner.workspace.get(name, shape, dtype)

    def cache_view(self, call) -> CacheView:
        model, rn = self.runner.model, self.runner
        gi, k = model.entry_location[call.cache]
        pool = rn.storage.entry_pool(gi, k)
        return CacheView(pool=pool, table=self.tables[gi], page_size=rn.manager.page_size,
                         num_pages=pool.shape[0], writes=call.writes_cache, group=gi)

    def state(self) -> torch.Tensor:
        """State tensor ``[slots, ...]`` of the mixer running now; rows are indexed with
        ``req_slot``."""
        return self.runner.storage.states[self.call_index]


class Workspace:
    """Temporary buffers by (name, dtype): one flat allocation each, grown when a larger
    shape is asked for.  Outgrown allocations are kept, since captured graphs may still
    point into them."""

    def __init__(self, device):
        self.device = device
        self._flat: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []

    def get(self, name, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        flat = self._flat.get(key)
        if flat is None or flat.numel() < n:
            if flat is not None:
                self._retired.append(flat)
            flat = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
        return flat[:n].view(*shape)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


def _bucket(n: int, lo: int) -> int:
    b = lo
    while b < n:
        b *= 2
    return b


class Runner:
    """Owns the model, the cache and the kernels, and runs steps."""

    def __init__(self, model, *, num_pages: int, page_size: int, max_requests: int,
                 dtype: torch.dtype, device, ops=None, prefix_cache: bool = False,
                 cuda_graphs: bool = False, fused_decode: bool = False):
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        if ops is None:
            from ..kernels.ops import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.model = model
        self.dtype = dtype
        if model.dtype != dtype:
            raise StepError("the model was bound with another dtype than the runner's")
        self.manager = CacheManager(
            [GroupSpec(window=g.window) for g in model.cache_groups], num_pages, page_size,
            max_requests, prefix_cache=prefix_cache, has_state=bool(model.state_shapes))
        self.storage = CacheStorage(model, self.manager, dtype, self.device)
        self.manager.on_open = self._clear_slot
        # The whole-step decode kernel is opt-in: on this model family it measured slower than
        # the layer-by-layer path (its phases are serial instruction chains on nine warps an SM).
        self.fused = None
        if self.device.type == "cuda" and (fused_decode or getattr(self.ops, "fused_decode_on", False)):
            from ..parts.fused import plan_fused_decode
            self.ops.fused_decode_on = True
            self.fused = plan_fused_decode(model, self.ops, self.storage, page_size)
        self.workspace = Workspace(self.device)
        self.max_positions = model.spec.max_positions
        self.max_pages = [self.manager.pages_for(self.max_positions) for _ in model.cache_groups]
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the token each request sampled last, by state slot: what FROM_DEVICE reads
        self.feedback = torch.zeros(max(1, max_requests), dtype=torch.int32, device=self.device)
        self._fetch_ring: list[torch.Tensor] = []
        self._fetch_next = 0
        if hasattr(ops, "status"):
            ops.status = self.status       # kernels that take no status argument report here
        self.cuda = self.device.type == "cuda"
        self.use_graphs = bool(cuda_graphs and self.cuda)
        self._graphs: dict[tuple, "_Captured"] = {}
        self._host_meta: dict[tuple[int, int], torch.Tensor] = {}
        self._dev_meta: dict[tuple, torch.Tensor] = {}
        self._layouts: dict[tuple, Layout] = {}
        # With CUDA graphs, the metadata of a step whose shape keeps coming back is uploaded on
        # a side stream into one of two device blocks (from one of two pinned blocks) that
        # alternate from step to step, so that the upload of step i + 1 runs while step i
        # computes: between two graphs the GPU then idles 2-3 us instead of 11-15 us (the copy,
        # and the launch behind it).  Such a shape has a captured graph per block.
        self._parity = 0
        self.hot_shape_uses = HOT_SHAPE_USES
        self._shape_uses: dict[tuple, int] = {}   # steps run per shape (a graph's key, less the block)
        self._copy_stream = (torch.cuda.Stream(device=self.device)
                             if self.use_graphs and self.model.capturable else None)
        self._copy_done = [None, None]     # the upload from this pinned block has run
        self._block_free = [None, None]    # the last step that read this device block has ended
        # the sampled tokens of such a step come back on a side stream too (a copy between two
        # graphs on the step's stream kept the GPU idle for 9-19 us); each block has a tokens
        # buffer of its own, free again once its last fetch has run
        self._fetch_stream = (torch.cuda.Stream(device=self.device)
                              if self._copy_stream is not None else None)
        self._tokens_free = [None, None]
        self.steps_run = 0
        self.kernel_launches = 0      # kernels of this package launched by steps so far

    # -- requests ---------------------------------------------------------------
    def open(self, req_id, token_ids=None):
        """Start a request (state slot; prefix pages if ``token_ids`` is given and prefix
        reuse is on).  Returns how many leading tokens are already cached."""
        return self.manager.open(req_id, token_ids).cached_tokens

    def _clear_slot(self, slot: int) -> None:
        """Every request starts on zeroed state, whoever opened it (this runner, the scheduler
        at admission or after a preemption): the manager calls this for each slot it hands
        out."""
        for st in self.storage.states.values():
            st[slot].zero_()

    def close(self, req_id) -> None:
        self.manager.close(req_id)

    # -- the step -----------------------------------------------------------------
    def _layout(self, T, R, W) -> Layout:
        key = (T, R, W)
        lay = self._layouts.get(key)
        if lay is None:
            plan_ints = 0
            if hasattr(self.ops, "attention_plan_ints"):
                plan_ints = self.ops.attention_plan_ints(T, R)
            lay = Layout(T, R, W, self.max_pages, plan_ints)
            self._layouts[key] = lay
        return lay

    def _host_buffer(self, n: int, parity: int = 0) -> torch.Tensor:
        size = _bucket(n, 1024)
        buf = self._host_meta.get((size, parity))
        if buf is None:
            buf = torch.zeros(size, dtype=torch.int32)
            if self.cuda:
                buf = buf.pin_memory()
            self._host_meta[(size, parity)] = buf
        return buf

    def step(self, entries: Sequence[StepEntry], sample: bool = False,
             check_status: bool = True) -> StepResult:
        """Run one batch.  The kernels are launched on the current stream of the runner's own
        device, which is made current for the duration if another one is."""
        if not entries:
            return StepResult(None, None, [], 0)
        if self.cuda and torch.cuda.current_device() != self.device.index:
            with torch.cuda.device(self.device):
                return self._step(entries, sample, check_status)
        return self._step(entries, sample, check_status)

    def _step(self, entries, sample, check_status) -> StepResult:
        mgr = self.manager
        # ---- host side: validate, reserve pages, lay the batch out ----------------
        seen = set()
        starts = []
        n_tok = n_want = 0
        vocab = self.model.spec.vocab_size
        token_arrays: list[np.ndarray] = []
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            toks = np.asarray(e.tokens, dtype=np.int64)     # once: checked here, packed below
            token_arrays.append(toks)
            known = toks[1:] if int(toks[0]) == FROM_DEVICE else toks
            if known.size and not (0 <= int(known.min()) and int(known.max()) < vocab):
                raise StepError(f"request {e.req_id!r}: token id outside [0, {vocab})")
            start = mgr.length(e.req_id) if e.req_id in mgr else 0
            if start + n > self.max_positions:
                raise StepError(f"request {e.req_id!r}: {start + n} positions exceed the "
                                f"model's {self.max_positions}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.req_id!r}: wanted place {w} outside its "
                                    f"{n} tokens")
            starts.append(start)
            n_tok += n
            n_want += len(e.want)
        # Nothing above changed anything.  Requests the cache does not know are opened here and
        # pages are reserved entry by entry; if one cannot be had, what this step took so far
        # is given back, so that a refused step leaves the cache as it found it.
        taken: list[tuple[Hashable, list[int] | None]] = []     # (request, table lengths | opened)
        try:
            for e, start in zip(entries, starts):
                if e.req_id not in mgr:
                    self.open(e.req_id)
                    taken.append((e.req_id, None))
                else:
                    taken.append((e.req_id, mgr.table_lengths(e.req_id)))
                mgr.reserve(e.req_id, start + len(e.tokens))
        except OutOfPages:
            for req_id, lengths in taken:
                if lengths is None:
                    mgr.close(req_id)
                else:
                    mgr.unreserve(req_id, lengths)
            raise

        if self.use_graphs:
            T, R = max(8, size_class(n_tok)), size_class(len(entries))
            W = size_class(n_want) if n_want else 0
        else:
            T, R, W = n_tok, len(entries), n_want
        lay = self._layout(T, R, W)
        # The second block (and the second graph of a shape) is for shapes that keep coming
        # back, such as a decode batch of a fixed size: capturing a graph costs what a
        # thousand overlapped uploads save, so a shape earns it with use.
        shape = (T, R, W, bool(sample))
        uses = self._shape_uses.get(shape, 0) + 1
        self._shape_uses[shape] = uses
        hot = self._copy_stream is not None and uses > self.hot_shape_uses
        parity = self._parity if hot else 0
        self._parity ^= 1
        host = self._host_buffer(lay.total, parity)
        if self._copy_done[parity] is not None:
            self._copy_done[parity].synchronize()   # the last upload from this block has run
        hm = host.numpy()
        hm[lay.tok_req:lay.tok_req + T] = -1
        hm[lay.tok_ids:lay.tok_ids + T] = 0
        hm[lay.tok_pos:lay.tok_pos + T] = 0
        if W:
            hm[lay.logit_rows:lay.logit_rows + W] = 0
            hm[lay.samp_temp:lay.samp_temp + W] = 0
            hm[lay.samp_topk:lay.samp_topk + W] = 0
            hm[lay.samp_pos:lay.samp_pos + W] = 0
            hm[lay.samp_slot:lay.samp_slot + W] = -1
        for gi, mp in enumerate(lay.max_pages):
            hm[lay.tables[gi]:lay.tables[gi] + R * mp] = -1
        hm[lay.req_len:lay.req_len + R] = 0
        hm[lay.req_ctx:lay.req_ctx + R] = 0
        hm[lay.req_start:lay.req_start + R] = 0
        hm[lay.req_slot:lay.req_slot + R] = 0
        temps = hm[lay.samp_temp:lay.samp_temp + W].view(np.float32) if W else None
        rows: list[tuple[Hashable, int]] = []
        host_batch = []
        t = w_i = 0
        for r, (e, start) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            toks = token_arrays[r]
            slot = mgr.slot(e.req_id)
            from_device = int(toks[0]) == FROM_DEVICE
            hm[lay.tok_ids + t:lay.tok_ids + t + n] = toks
            if from_device:
                hm[lay.tok_ids + t] = -(slot + 1)
            hm[lay.tok_pos + t:lay.tok_pos + t + n] = np.arange(start, start + n)
            hm[lay.tok_req + t:lay.tok_req + t + n] = r
            hm[lay.req_start + r] = t
            hm[lay.req_len + r] = n
            hm[lay.req_ctx + r] = start + n
            hm[lay.req_slot + r] = slot
            for gi, mp in enumerate(lay.max_pages):
                tab = mgr.table(e.req_id, gi)
                o = lay.tables[gi] + r * mp
                hm[o:o + len(tab)] = tab
            for w in e.want:
                hm[lay.logit_rows + w_i] = t + w
                temps[w_i] = e.temperature
                hm[lay.samp_topk + w_i] = e.top_k
                seed = int(e.seed) & 0xFFFFFFFFFFFFFFFF
                hm[lay.samp_seed_lo + w_i] = np.array(seed & 0xFFFFFFFF, dtype=np.uint32).view(np.int32)
                hm[lay.samp_seed_hi + w_i] = np.array(seed >> 32, dtype=np.uint32).view(np.int32)
                hm[lay.samp_pos + w_i] = start + w + 1     # position the new token will take
                if w == n - 1:                             # the request's next token
                    hm[lay.samp_slot + w_i] = slot
                rows.append((e.req_id, w))
                w_i += 1
            host_batch.append((e.req_id, slot, start, n))
            t += n
        plan_shape = None
        if lay.plan_ints:
            plan_shape = self.ops.plan_attention(hm[lay.plan:lay.plan + lay.plan_ints],
                                                 host_batch, T, R, mgr.page_size, self.use_graphs)

        # ---- device side -------------------------------------------------------------
        greedy = all(e.temperature <= 0.0 for e in entries)
        key = (T, R, W, bool(sample), plan_shape, greedy, parity)
        dev = self._dev_meta.get((T, R, W, parity))
        fresh = dev is None
        if fresh:
            dev = torch.zeros(lay.total, dtype=torch.int32, device=self.device)
            self._dev_meta[(T, R, W, parity)] = dev
        if not hot:
            # This copy is also what separates steps on the stream: it is not a kernel, so no
            # kernel of this step, however early programmatic dependent launch lets it start,
            # runs before every kernel of the step before has ended.  The decode attention
            # relies on it when it prefetches keys of earlier positions before its dependency
            # wait.  (With graphs the graph's boundary separates the steps.)
            dev.copy_(host[:lay.total], non_blocking=True)
            if self.cuda:
                if self._copy_done[parity] is None:
                    self._copy_done[parity] = torch.cuda.Event()
                self._copy_done[parity].record()
        else:
            main = torch.cuda.current_stream(self.device)
            if self._copy_done[parity] is None:
                self._copy_done[parity] = torch.cuda.Event()
            if main.query():
                # nothing is running: there is no step to overlap with, and a hand-over between
                # streams would only add its latency (30 us on a step that starts from idle)
                dev.copy_(host[:lay.total], non_blocking=True)
                self._copy_done[parity].record(main)
            else:
                side = self._copy_stream
                if fresh:
                    side.wait_stream(main)                         # the block has been zeroed
                if self._block_free[parity] is not None:
                    side.wait_event(self._block_free[parity])      # its last reader has ended
                with torch.cuda.stream(side):
                    dev.copy_(host[:lay.total], non_blocking=True)
                    self._copy_done[parity].record(side)
                main.wait_event(self._copy_done[parity])

        if self._fetch_stream is not None and self._tokens_free[parity] is not None:
            # the last fetch from the tokens buffer this step writes has run
            torch.cuda.current_stream(self.device).wait_event(self._tokens_free[parity])
        cap = self._graphs.get(key) if self.use_graphs else None
        if cap is not None:
            cap.ctx.host = host_batch
            cap.graph.replay()
            self.kernel_launches += cap.n_launches
            logits, tokens = cap.logits, cap.tokens
        else:
            ctx = StepContext(self, lay, dev)
            ctx.host = host_batch
            ctx.greedy_only = greedy
            ctx.tokens_name = "sampled" if parity == 0 else "sampled_b"
            if plan_shape is not None:
                from ..kernels.ops import AttentionPlan
                ctx.plan = AttentionPlan(dev[lay.plan:lay.plan + lay.plan_ints], T, *plan_shape)
            if self.use_graphs and self.model.capturable:
                # run once eagerly (loads kernels, sizes buffers), then capture and replay.  The
                # replay must see the same inputs as the eager run: all of them come from the
                # metadata block except the tokens kept on the device, which sampling
                # overwrites, and the per-request state of stateful mixers, which the eager run
                # has already advanced (the state tensors have fixed addresses, so a captured
                # step reads and writes them like any other)
                # (the shape's graph over the other metadata block, if there is one, has done
                # that already)
                ran_eagerly = self._graphs.get(key[:-1] + (parity ^ 1,)) is None
                if ran_eagerly:
                    kept = self.feedback.clone()
                    kept_state = {k: st.clone() for k, st in self.storage.states.items()}
                    self._forward(ctx, sample)
                    self.feedback.copy_(kept)
                    for k, st in kept_state.items():
                        self.storage.states[k].copy_(st)
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                # An object freed by the garbage collector in the middle of a capture (an
                # older runner's graphs, say) would invalidate it: hold the collector off
                # until the capture has ended.  (No collection beforehand: it takes 25-35 ms,
                # four times the rest of a capture.)
                gc_was_on = gc.isenabled()
                gc.disable()
                before = getattr(self.ops, "launches", 0)
                try:
                    with torch.cuda.graph(graph):
                        logits, tokens = self._forward(ctx, sample)
                finally:
                    if gc_was_on:
                        gc.enable()
                n_launch = getattr(self.ops, "launches", 0) - before
                self._graphs[key] = _Captured(graph, ctx, logits, tokens, n_launch)
                graph.replay()
                self.kernel_launches += (2 if ran_eagerly else 1) * n_launch
            else:
                before = getattr(self.ops, "launches", 0)
                logits, tokens = self._forward(ctx, sample)
                self.kernel_launches += getattr(self.ops, "launches", 0) - before

        if self._copy_stream is not None:
            if self._block_free[parity] is None:
                self._block_free[parity] = torch.cuda.Event()
            self._block_free[parity].record()
        for e, start in zip(entries, starts):
            mgr.commit(e.req_id, start + len(e.tokens))
        self.steps_run += 1
        if check_status and not sample:
            self.check_status()
        return StepResult(
            logits=None if logits is None else logits[:n_want],
            tokens=None if tokens is None else tokens[:n_want],
            rows=rows, n_tokens=n_tok,
            _with_status=None if tokens is None else tokens, _runner=self,
            _block=parity if hot else None)

    def _forward(self, ctx: StepContext, sample: bool):
        ctx.fused_tokens = None
        ctx.sampling = bool(sample)
        logits = self.model.forward(ctx)
        tokens = None
        if sample and logits is not None:
            # one extra element carries the status word, so that one copy brings both back
            W = ctx.n_logit_rows
            tokens = ctx.buffer(ctx.tokens_name, (W + 1,), torch.int32)
            if ctx.fused_tokens is not None and ctx.greedy_only:
                # the step ran as one kernel, which also chose the tokens (argmax, lowest
                # index on ties), kept them for the requests and stored the status word
                return logits, ctx.fused_tokens
            more = {}
            if getattr(self.ops, "takes_status_word", False):
                more["status_word"] = self.status          # stored to tokens[W] by the kernel
            self.ops.sample(tokens, logits, ctx.samp_temp, ctx.samp_topk, ctx.samp_seed_lo,
                            ctx.samp_seed_hi, ctx.samp_pos, feedback=self.feedback,
                            feedback_slot=ctx.samp_slot, **more)
            if not more:
                tokens[W:].copy_(self.status)
        return logits, tokens

    def _fetch(self, dev: torch.Tensor, block: int | None = None):
        """Start copying ``dev`` (int32) to pinned host memory behind the work enqueued so far;
        returns (host tensor, event).  Four buffers rotate: a result is to be read before four
        later ones have been fetched.  ``block``: the step ran over that metadata block with
        its copies on side streams; the fetch then leaves the step's stream free for the next
        graph."""
        n = dev.shape[0]
        if not self.cuda:
            return dev.clone(), None
        if len(self._fetch_ring) < 4:
            self._fetch_ring.append(torch.empty(1024, dtype=torch.int32).pin_memory())
        i = self._fetch_next % 4
        self._fetch_next += 1
        if self._fetch_ring[i].shape[0] < n:
            self._fetch_ring[i] = torch.empty(_bucket(n, 1024), dtype=torch.int32).pin_memory()
        host = self._fetch_ring[i][:n]
        ev = torch.cuda.Event()
        if block is None or self._fetch_stream is None:
            host.copy_(dev, non_blocking=True)
            ev.record()
        else:
            done = torch.cuda.Event()
            done.record()                                  # the step's work, on its own stream
            side = self._fetch_stream
            side.wait_event(done)
            with torch.cuda.stream(side):
                host.copy_(dev, non_blocking=True)
                ev.record(side)
            self._tokens_free[block] = ev
        return host, ev

    def check_status(self) -> None:
        """Read the status word the kernels OR their refusals into (synchronises)."""
        code = int(self.status.item())
        if code:
            self.raise_status(code)

    def raise_status(self, code: int) -> None:
        self.status.zero_()
        what = [msg for bit, msg in STATUS_BITS.items() if code & bit]
        raise StepError("a kernel refused an index: " + "; ".join(what))


@dataclass
class _Captured:
    graph: "torch.cuda.CUDAGraph"
    ctx: StepContext
    logits: torch.Tensor | None
    tokens: torch.Tensor | None
    n_launches: int = 0
