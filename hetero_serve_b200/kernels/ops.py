"""The kernel interface of the engine: thin, checked Python wrappers around the
``extern "C"`` entry points of the CUDA library.

Every operation writes into tensors the caller owns (nothing is allocated here),
runs on the current CUDA stream and raises :class:`KernelError` for a size or
type a kernel does not take.  There is no fallback: if the library cannot be
built or loaded, constructing :class:`CudaOps` fails.

``tests/plain_ops.py`` holds a plain PyTorch twin of each operation with the same
signature; the kernel tests compare the two.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass

import torch

from . import build as _build

ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


@dataclass(frozen=True)
class AttentionGeometry:
    """Sizes an attention layer hands to the cache and attention kernels."""

    n_heads: int
    n_kv_heads: int
    head_dim: int
    page_size: int
    num_pages: int
    max_pages: int          # row length of the block table
    q_off: int              # column of q / k / v in a row of the fused projection
    k_off: int
    v_off: int
    qkv_stride: int
    window: int = 0         # 0: every earlier key; w: the last w keys

    def page_elems(self) -> int:
        return 2 * self.n_kv_heads * self.page_size * self.head_dim


@dataclass
class AttentionPlan:
    """Work lists of one step for the specialised attention kernels, in device memory.

    ``data`` (int32): ``[0]`` number of single-query tokens, ``[1]`` number of 128-query
    tiles, ``[2]`` longest context among the single-query tokens, ``[3]`` unused; then per
    single-query token (``n_rows`` slots) its flat index, request row and position; then per
    tile (``tile_slots`` slots) the flat index of its first query, its number of queries, its
    request row and the position of its first query.
    ``decode_cap`` / ``tile_cap`` are the grid sizes the kernels are launched with (at
    least the counts; fixed per size class so that a captured graph stays valid)."""

    data: torch.Tensor
    n_rows: int
    decode_cap: int
    tile_cap: int
    single_new: bool = False     # every single-query token is the only new token of its request

    @property
    def tile_slots(self) -> int:
        return plan_tile_slots(self.n_rows)


def pack_weight_units(w: torch.Tensor) -> torch.Tensor:
    """A [features, k] bfloat16 matrix (k contiguous, k a multiple of 64) in the layout the
    persistent decode kernel streams: features padded with zero rows to a multiple of 16; tile j
    (rows 16 j .. 16 j + 15) is k / 64 boxes of [16 rows x 64 k] one behind the other, so that
    any run of boxes of a tile is contiguous; inside a box the 16-byte piece c of row r lies at
    piece c ^ (r & 7) of the row (the 128-byte XOR swizzle)."""
    n, k = w.shape
    if k % 64:
        raise KernelError(f"pack_weight_units: k = {k} is not a multiple of 64")
    n16 = -(-n // 16) * 16
    if n16 != n:
        w = torch.cat([w, w.new_zeros(n16 - n, k)])
    t = w.contiguous().view(n16 // 16, 16, k // 64, 8, 8)      # tile, row, box, piece, element
    out = torch.empty_like(t)
    for r in range(16):
        perm = [c ^ (r & 7) for c in range(8)]
        out[:, r] = t[:, r][:, :, perm]
    return out.permute(0, 2, 1, 3, 4).contiguous().view(-1)


@dataclass
class FusedTables:
    """Device records of a model for the persistent decode kernel (see ``fused_decode_build``)."""

    data: torch.Tensor            # uint8 on the device: layer records, then head and cache maps
    n_layers: int
    layer_bytes: int
    keep: list                    # the tensors the records point at

    @property
    def layers_ptr(self) -> int:
        return self.data.data_ptr()

    @property
    def tables_ptr(self) -> int:
        return self.data.data_ptr() + self.n_layers * self.layer_bytes


DECODE_MAX_NEW = 4        # requests bringing at most this many tokens use the decode kernel
PREFILL_TILE = 128


def _pow2(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


def size_class(n: int) -> int:
    """The size a count is rounded up to where shapes must repeat (captured graphs): powers of
    two up to 8, then four classes per doubling (10, 12, 14, 16, 20, 24, 28, 32, 40, 48, ...),
    so that padding stays below a quarter of the work."""
    if n <= 8:
        return _pow2(n)
    step = _pow2(n) // 8
    return -(-n // step) * step


def plan_tile_slots(n_rows: int) -> int:
    """Tile entries a plan holds: every tile a batch of n_rows tokens can have, rounded up to
    a power of two (grids are sized in powers of two when steps are captured)."""
    return _pow2(n_rows // PREFILL_TILE + n_rows // (DECODE_MAX_NEW + 1) + 1)


def plan_decode_ints(n_rows: int) -> int:
    """Ints of the single-query section: 3 per token, padded so that the tile section that
    follows is 16-byte aligned."""
    return (3 * n_rows + 3) // 4 * 4


_ERRORS = {-1: "unsupported size, type or option", -2: "bad argument"}

_lib = None


def load_library():
    """Build if needed and open the CUDA library (once per process)."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None
        _declare(_lib)
    return _lib


def _declare(lib) -> None:
    P, I, F = c_void_p, c_int, c_float
    sig = {
        "hs_embed": [P, P, P, P, P, P, I, I, I, I, I, P, I, P, P],
        "hs_layernorm": [P, P, P, P, P, I, I, F, I, P],
        "hs_linear_simt": [P, P, P, P, P, I, I, I, I, I, I, P],
        "hs_linear_tcgen05": [P, P, P, P, P, I, I, I, I, I, I, I, P, P, P, P],
        "hs_linear_tcgen05_scratch": [I, I, I, I, I, P, P],
        "hs_linear_skinny": [P, P, P, P, P, F, P, P, P, I, I, I, I, I, P, P, I, P],
        "hs_linear_skinny_scratch": [I, I, I, I, P, P],
        "hs_linear_skinny_argmax": [P, P, P, I, I, I, P, P, P, P, P, P, P, I, P],
        "hs_linear_skinny_argmax_scratch": [I, I, I, P],
        "hs_kv_append": [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "hs_attention_simt": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, I, P, P],
        "hs_attention_simt_grouped": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, F, I, I,
                                      P, P],
        "hs_attention_decode_append": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I,
                                       F, I, I, I, I, P, P, P, P, P],
        "hs_attention_decode_mma": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, I, I, I,
                                    P, P, P, P, P],
        "hs_attention_prefill": [P, P, P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, F, P, P],
        "hs_attention_prefill_tc": [P, P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, I, F, P, P],
        "hs_argmax": [P, P, I, I, P],
        "hs_sample": [P, P, P, P, P, P, P, I, I, P, P, P, P],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    LL = ctypes.c_longlong
    lib.hs_decode_persistent_layer_bytes.restype = c_int
    lib.hs_decode_persistent_tables_bytes.restype = c_int
    lib.hs_decode_persistent_grid.restype = c_int
    lib.hs_decode_persistent_slices.argtypes = [I, I]
    lib.hs_decode_persistent_slices.restype = c_int
    lib.hs_decode_persistent_supports.argtypes = [I] * 7
    lib.hs_decode_persistent_supports.restype = c_int
    lib.hs_decode_persistent_layer.argtypes = [P] * 13 + [F, F, F, I, I, I, LL]
    lib.hs_decode_persistent_layer.restype = c_int
    lib.hs_decode_persistent_tables.argtypes = [P, P, I, I, P, LL]
    lib.hs_decode_persistent_tables.restype = c_int
    lib.hs_decode_persistent.argtypes = ([P, P, I, P, P, P, P, F] + [I] * 5 + [P, I, I]
                                         + [P] * 11 + [I] + [P] * 7 + [I] * 4 + [P, P, I, P])
    lib.hs_decode_persistent.restype = c_int
    lib.hs_set_pdl.argtypes = [I]
    lib.hs_set_pdl.restype = None
    lib.hs_set_split_clusters.argtypes = [I]
    lib.hs_set_split_clusters.restype = None


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _want(t, name, dtype=None, dim=None, cuda=True):
    if not isinstance(t, torch.Tensor):
        raise KernelError(f"{name}: expected a tensor, got {type(t).__name__}")
    if cuda and not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list, set)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name}: dtype {t.dtype} not accepted (want {dtype})")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name}: expected {dim} dimensions, got shape {tuple(t.shape)}")
    return t


_FLOATS = (torch.float32, torch.bfloat16)


class CudaOps:
    """The hand-written sm_100a kernels, one method per operation."""

    name = "cuda"

    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise KernelError("hetero_serve_b200 needs a CUDA device: its kernels have no CPU path")
        dev = torch.device("cuda" if device is None else device)
        if dev.type != "cuda":
            raise KernelError(f"hetero_serve_b200 needs a CUDA device, got {dev}")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        # One object drives one device.  Its kernels are launched on that device's current
        # stream, so the device must be current while they are (the runner sees to it).
        self.device = dev
        self.lib = load_library()
        self.launches = 0          # kernels launched through this object (graph captures count once)
        self.tensor_cores = True   # bfloat16 linears on tcgen05 (False: CUDA cores, for tests)
        self.fast_attention = True  # bfloat16 attention on the split-context / tensor-core kernels
        self.tc_attention = True    # head size 64: prompt portions on the tcgen05 attention kernel
        self.sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        self.fuse_norm = True      # LayerNorm fused into the few-row linear kernel
        self.fuse_argmax = True    # greedy choice fused into the few-row head (linear_argmax)
        self.fuse_append = True    # key/value append fused into the decode attention
        self.pdl = True            # programmatic dependent launch (see the property below)
        self._skinny_need: dict = {}
        self._tc_need: dict = {}
        self._scratch: dict = {}
        self._retired: list = []
        self.decode_force = None   # (wide code, slices) of the decode attention, for tuning
        self.decode_mma = True     # tensor-core decode attention where the shape allows it
        #                            (head size 32/64/128, at most 16 query heads per kv head)
        self.takes_status_word = True   # sample() can store the status word behind the tokens
        self.tile_n = 0            # 0: chosen per shape; 64/128/192/256 force a tile width
        self.cta_pairs = -1        # -1: pairs of CTAs (cta_group::2) when there are many rows;
        #                            0: never; 1: always
        self.split_clusters = True  # few rows split over k: the splits of a tile exchange their
        #                            shares inside a thread-block cluster (False: through scratch)
        self.fused_decode_on = False  # pure decode steps of up to 16 tokens as ONE persistent kernel
        #                             (measured slower than the layer-by-layer path: off)
        self.skinny_max_rows = 16  # up to this many rows the weight-streaming kernel is used
        #                            (measured: from 17 rows on the tcgen05 kernel's split over k wins)
        # pipeline time-outs of the TMA/tcgen05 kernels are ORed into this word; the runner
        # replaces it with its own so that they surface with the step's results
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # -- kernels that parts bring themselves -------------------------------------------
    def stream(self) -> int:
        """The raw CUDA stream (of this object's device) kernels are to be launched on."""
        return self._stream()

    def register_kernel(self, symbol: str, argtypes, lib=None):
        """Declare an ``extern "C"`` entry point (returning int in the convention of this
        library: 0, a negative HS_ERR_* code or a positive cudaError_t) and return a function
        that calls it, counts the launch and raises :class:`KernelError` on a non-zero code.
        ``lib`` is a library opened with :meth:`load_extension`; by default the package's
        own.  A part calls this once (in ``bind``) and the returned function in ``forward``
        with raw pointers (``tensor.data_ptr()``), sizes and ``ops.stream()``."""
        lib = lib or self.lib
        try:
            fn = getattr(lib, symbol)
        except AttributeError:
            raise KernelError(f"the library exports no symbol {symbol!r}") from None
        fn.argtypes = list(argtypes)
        fn.restype = c_int

        def call(*args):
            self.launches += 1
            _check(fn(*args), symbol)
        call.__name__ = symbol
        return call

    def load_extension(self, name: str, sources):
        """Build (once) and open a library of CUDA sources from outside the package; see
        :func:`hetero_serve_b200.kernels.build.build_extension`."""
        path = _build.build_extension(name, sources)
        try:
            return ctypes.CDLL(str(path))
        except OSError as exc:
            raise KernelError(f"cannot load {path}: {exc}") from None

    @property
    def pdl(self) -> bool:
        """Programmatic dependent launch: kernels are launched so that their set-up (and what
        they fetch that no kernel of the step writes: weights, work lists) overlaps the end of
        the kernel before them; each waits before it first reads an earlier kernel's output.
        The few-row linear and the decode attention take it as an argument; the other kernels
        read a switch in the library, which is process-wide (the last setter wins)."""
        return self._pdl

    @pdl.setter
    def pdl(self, on: bool) -> None:
        self._pdl = bool(on)
        self.lib.hs_set_pdl(int(self._pdl))

    # -- embedding and norm -------------------------------------------------
    def embed(self, x, ids, pos, req, wte, wpe, status, feedback=None):
        """x[t] = wte[ids[t]] (+ wpe[pos[t]]); rows with req[t] < 0 become zero.  With
        ``feedback`` (int32 on the device) an id ``-(s + 1)`` stands for ``feedback[s]``."""
        _want(x, "x", torch.float32, 2)
        _want(wte, "wte", _FLOATS, 2)
        n, width = x.shape
        for t, nm in ((ids, "ids"), (pos, "pos"), (req, "req")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < n:
                raise KernelError(f"{nm}: {t.shape[0]} entries for {n} rows")
        if wte.shape[1] != width:
            raise KernelError(f"wte width {wte.shape[1]} != x width {width}")
        n_pos = 0
        if wpe is not None:
            _want(wpe, "wpe", wte.dtype, 2)
            if wpe.shape[1] != width:
                raise KernelError(f"wpe width {wpe.shape[1]} != x width {width}")
            n_pos = wpe.shape[0]
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
        self.launches += 1
        _check(self.lib.hs_embed(_ptr(x), _ptr(ids), _ptr(pos), _ptr(req), _ptr(wte), _ptr(wpe),
                                 n, width, wte.shape[0], n_pos, _DT[wte.dtype], _ptr(feedback),
                                 0 if feedback is None else feedback.shape[0], _ptr(status),
                                 self._stream()), "embed")

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        """out[i] = LayerNorm(x[rows[i]] if rows is given else x[i]) * gamma + beta."""
        _want(out, "out", _FLOATS, 2)
        _want(x, "x", torch.float32, 2)
        _want(gamma, "gamma", torch.float32, 1)
        _want(beta, "beta", torch.float32, 1)
        n, width = out.shape
        if x.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
            raise KernelError("layernorm: widths of out, x, gamma, beta differ")
        if rows is not None:
            _want(rows, "rows", torch.int32, 1)
            if rows.shape[0] < n:
                raise KernelError("layernorm: fewer row indices than output rows")
        elif x.shape[0] < n:
            raise KernelError("layernorm: x has fewer rows than out")
        self.launches += 1
        _check(self.lib.hs_layernorm(_ptr(out), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(rows), n,
                                     width, float(eps), _DT[out.dtype], self._stream()),
               f"layernorm(width={width})")

    # -- linear ---------------------------------------------------------------
    def linear(self, out, a, w, bias=None, act="none", residual=None):
        """out = act(a @ w.T + bias) (+ residual).  a [M,K], w [N,K], out [M,N].

        ``residual`` is float32 [M,N] and may be ``out`` itself (accumulate in place)."""
        _want(a, "a", _FLOATS, 2)
        _want(w, "w", a.dtype, 2)
        _want(out, "out", _FLOATS, 2)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError(f"linear: shapes a{tuple(a.shape)} w{tuple(w.shape)} "
                              f"out{tuple(out.shape)} do not fit")
        if a.dtype == torch.float32 and out.dtype != torch.float32:
            raise KernelError("linear: float32 inputs give float32 outputs")
        if bias is not None:
            _want(bias, "bias", torch.float32, 1)
            if bias.shape[0] != N:
                raise KernelError("linear: bias length != N")
        if residual is not None:
            _want(residual, "residual", torch.float32, 2)
            if tuple(residual.shape) != (M, N):
                raise KernelError("linear: residual shape != out shape")
        if act not in ACTIVATIONS:
            raise KernelError(f"linear: unknown activation {act!r}")
        self._linear(out, a, w, bias, ACTIVATIONS[act], residual, M, N, K)

    def _linear(self, out, a, w, bias, act, residual, M, N, K):
        """bfloat16 goes to the tcgen05 kernel when TMA can address the operands (K a multiple
        of 8, 16-byte aligned pointers); everything else, and all of float32, to the CUDA cores."""
        self.launches += 1
        if a.dtype == torch.bfloat16 and self._skinny_ok(M, N, K):
            if self._skinny(out, a, None, w, bias, act, residual, M, N, K):
                return
        if a.dtype == torch.bfloat16 and self.tensor_cores and K % 8 == 0:
            if CudaOps._lib_split_clusters != bool(self.split_clusters):   # a switch of the library
                CudaOps._lib_split_clusters = bool(self.split_clusters)
                self.lib.hs_set_split_clusters(int(CudaOps._lib_split_clusters))
            key = (M, N, K, self.tile_n, self.cta_pairs, bool(self.split_clusters))
            need = self._tc_need.get(key)
            if need is None:
                floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
                rc = self.lib.hs_linear_tcgen05_scratch(M, N, K, self.tile_n, self.cta_pairs,
                                                        ctypes.byref(floats),
                                                        ctypes.byref(counters))
                need = (floats.value, counters.value) if rc == 0 else (0, 0)
                self._tc_need[key] = need
            scratch = cnt = None
            if need[0]:
                scratch = self._scratch_buffer("tc_partial", need[0], torch.float32)
                cnt = self._scratch_buffer("tc_counters", need[1], torch.int32)
            code = self.lib.hs_linear_tcgen05(
                _ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), M, N, K, act,
                _DT[out.dtype], self.tile_n, self.cta_pairs, _ptr(scratch), _ptr(cnt),
                _ptr(self.status),
                self._stream())
            if code != -1:
                _check(code, f"linear_tcgen05(M={M},N={N},K={K})")
                return
        _check(self.lib.hs_linear_simt(_ptr(out), _ptr(a), _ptr(w), _ptr(bias), _ptr(residual),
                                       M, N, K, act, _DT[a.dtype], _DT[out.dtype],
                                       self._stream()), f"linear(M={M},N={N},K={K})")

    def _skinny_ok(self, M, N, K) -> bool:
        return self.tensor_cores and M <= self.skinny_max_rows

    def _skinny(self, out, a, norm, w, bias, act, residual, M, N, K) -> bool:
        """The weight-streaming kernel; ``norm = (x, gamma, beta, eps)`` fuses a LayerNorm of
        the float32 input.  False when the kernel does not take the shape."""
        key = (M, N, K, norm is not None)
        need = self._skinny_need.get(key)
        if need is None:
            floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
            code = self.lib.hs_linear_skinny_scratch(M, N, K, int(norm is not None),
                                                     ctypes.byref(floats), ctypes.byref(counters))
            need = (floats.value, counters.value) if code == 0 else False
            self._skinny_need[key] = need
        if need is False:
            return False
        scratch = cnt = None
        if need[0]:
            scratch = self._scratch_buffer("skinny_partial", need[0], torch.float32)
            cnt = self._scratch_buffer("skinny_counters", need[1], torch.int32)
        x = g = b = None
        eps = 0.0
        if norm is not None:
            x, g, b, eps = norm
        code = self.lib.hs_linear_skinny(
            _ptr(out), _ptr(a), _ptr(x), _ptr(g), _ptr(b), float(eps), _ptr(w), _ptr(bias),
            _ptr(residual), M, N, K, act, _DT[out.dtype], _ptr(scratch), _ptr(cnt),
            int(self.pdl), self._stream())
        if code == -1:
            return False
        _check(code, f"linear_skinny(M={M},N={N},K={K})")
        return True

    def linear_argmax(self, out, a, w, tokens, feedback=None, feedback_slot=None,
                      status_word=None) -> bool:
        """out = a @ w.T as float32 logits AND tokens[m] = argmax of row m (lowest index on
        ties), in the one few-row kernel: its CTAs keep their best per row while they stream
        the table, the last to finish picks.  ``tokens`` has a word more than rows, which
        receives ``status_word``; ``feedback[feedback_slot[m]]`` gets row m's token as in
        `sample`.  False (nothing done) for shapes or types the kernel does not take: the
        caller then runs `linear` and `sample`."""
        if not (self.tensor_cores and self.fuse_argmax and a.dtype == torch.bfloat16
                and w.dtype == torch.bfloat16 and out.dtype == torch.float32):
            return False
        _want(a, "a", torch.bfloat16, 2)
        _want(w, "w", torch.bfloat16, 2)
        _want(out, "out", torch.float32, 2)
        _want(tokens, "tokens", torch.int32, 1)
        M, K = a.shape
        N = w.shape[0]
        if M > self.skinny_max_rows or w.shape[1] != K or tuple(out.shape) != (M, N):
            return False
        if tokens.shape[0] < M + 1:
            raise KernelError("linear_argmax: tokens needs a word more than rows")
        if (feedback is None) != (feedback_slot is None):
            raise KernelError("linear_argmax: feedback and feedback_slot come together")
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
            _want(feedback_slot, "feedback_slot", torch.int32, 1)
            if feedback_slot.shape[0] < M:
                raise KernelError("linear_argmax: feedback_slot shorter than the rows")
        if status_word is not None:
            _want(status_word, "status_word", torch.int32, 1)
        key = ("argmax", M, N, K)
        need = self._skinny_need.get(key)
        if need is None:
            entries = ctypes.c_int(0)
            code = self.lib.hs_linear_skinny_argmax_scratch(M, N, K, ctypes.byref(entries))
            need = entries.value if code == 0 else False
            self._skinny_need[key] = need
        if need is False:
            return False
        val = self._scratch_buffer("argmax_val", need, torch.float32)
        idx = self._scratch_buffer("argmax_idx", need, torch.int32)
        cnt = self._scratch_buffer("argmax_counter", 1, torch.int32)
        code = self.lib.hs_linear_skinny_argmax(
            _ptr(out), _ptr(a), _ptr(w), M, N, K, _ptr(tokens), _ptr(feedback),
            _ptr(feedback_slot), _ptr(status_word), _ptr(val), _ptr(idx), _ptr(cnt),
            int(self.pdl), self._stream())
        if code == -1:
            return False
        _check(code, f"linear_argmax(M={M},N={N},K={K})")
        self.launches += 1
        return True

    def norm_linear(self, out, h, x, gamma, beta, eps, w, bias=None, act="none"):
        """out = act(LayerNorm(x) @ w.T + bias).  For few rows the normalisation is fused into
        the weight-streaming kernel; otherwise ``h`` receives LayerNorm(x) first."""
        M, K = x.shape
        N = w.shape[0]
        if (w.dtype == torch.bfloat16 and self.fuse_norm and self._skinny_ok(M, N, K)):
            _want(x, "x", torch.float32, 2)
            _want(w, "w", torch.bfloat16, 2)
            _want(out, "out", _FLOATS, 2)
            _want(gamma, "gamma", torch.float32, 1)
            _want(beta, "beta", torch.float32, 1)
            if w.shape[1] != K or tuple(out.shape) != (M, N) or gamma.shape[0] != K \
                    or beta.shape[0] != K:
                raise KernelError("norm_linear: shapes do not fit")
            if bias is not None:
                _want(bias, "bias", torch.float32, 1)
            if act not in ACTIVATIONS:
                raise KernelError(f"norm_linear: unknown activation {act!r}")
            self.launches += 1
            if self._skinny(out, None, (x, gamma, beta, eps), w, bias, ACTIVATIONS[act], None,
                            M, N, K):
                return
            self.launches -= 1
        self.layernorm(h, x, gamma, beta, eps)
        self.linear(out, h, w, bias, act=act)

    # -- cache and attention ------------------------------------------------------
    def _attn_common(self, qkv, pool, table, tok_pos, tok_req, g, n):
        _want(qkv, "qkv", _FLOATS, 2)
        _want(pool, "pool", qkv.dtype)
        _want(table, "table", torch.int32, 2)
        _want(tok_pos, "tok_pos", torch.int32, 1)
        _want(tok_req, "tok_req", torch.int32, 1)
        if qkv.shape[0] < n or tok_pos.shape[0] < n or tok_req.shape[0] < n:
            raise KernelError("attention: fewer rows than tokens")
        if qkv.shape[1] != g.qkv_stride or table.shape[1] != g.max_pages:
            raise KernelError("attention: geometry does not match the tensors")
        if pool.numel() != g.num_pages * g.page_elems():
            raise KernelError(f"attention: pool has {pool.numel()} elements, geometry wants "
                              f"{g.num_pages * g.page_elems()}")
        hd = g.head_dim
        if (g.q_off + g.n_heads * hd > g.qkv_stride or g.k_off + g.n_kv_heads * hd > g.qkv_stride
                or g.v_off + g.n_kv_heads * hd > g.qkv_stride):
            raise KernelError("attention: q/k/v columns exceed the fused row")

    def kv_append(self, pool, qkv, table, tok_pos, tok_req, g, status, n_tokens=None):
        """Write each token's key and value rows into its page (rows with req < 0 are skipped)."""
        n = qkv.shape[0] if n_tokens is None else n_tokens
        self._attn_common(qkv, pool, table, tok_pos, tok_req, g, n)
        self.launches += 1
        _check(self.lib.hs_kv_append(_ptr(pool), _ptr(qkv), _ptr(table), _ptr(tok_pos),
                                     _ptr(tok_req), n, g.n_heads, g.n_kv_heads, g.head_dim,
                                     g.page_size, g.num_pages, g.max_pages, g.q_off, g.k_off,
                                     g.v_off, g.qkv_stride, _DT[qkv.dtype], _ptr(status),
                                     self._stream()),
               f"kv_append(head_dim={g.head_dim})")

    def attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan=None,
                  _fuse_append=False):
        """out[t] = causal attention of token t's query over its request's pages.

        ``plan`` may carry a batch's work lists for the specialised kernels; the general
        kernel needs none."""
        _want(out, "out", qkv.dtype, 2)
        n = out.shape[0]
        if out.shape[1] != g.n_heads * g.head_dim:
            raise KernelError("attention: out width != n_heads * head_dim")
        self._attn_common(qkv, pool, table, tok_pos, tok_req, g, n)
        self._attention(out, qkv, pool, table, tok_pos, tok_req, g, float(scale), status, plan, n,
                        _fuse_append)

    # -- attention work lists ---------------------------------------------------------
    @staticmethod
    def attention_plan_ints(n_rows: int, n_requests: int) -> int:
        return 4 + plan_decode_ints(n_rows) + 4 * plan_tile_slots(n_rows)

    @staticmethod
    def plan_attention(view, host_batch, n_rows: int, n_requests: int, page_size: int,
                       bucketed: bool) -> tuple[int, int]:
        """Fill the plan section (a numpy int32 view of the step's metadata) for a batch given
        as ``[(request, slot, start, n_new)]`` in flat order; returns ``(decode_cap,
        tile_cap, single_new)``.  Requests bringing up to DECODE_MAX_NEW tokens go to the single-query
        list, the others are cut into tiles of 128 queries, longest context first."""
        dec = view[4:4 + 3 * n_rows]
        tiles = view[4 + plan_decode_ints(n_rows):]
        n_dec = n_tiles = max_ctx = 0
        t = 0
        single = True
        tile_list = []
        for row, (_req, _slot, start, n) in enumerate(host_batch):
            if n <= DECODE_MAX_NEW:
                single = single and n == 1
                for i in range(n):
                    dec[3 * n_dec:3 * n_dec + 3] = (t + i, row, start + i)
                    n_dec += 1
                max_ctx = max(max_ctx, start + n)
            else:
                for q0 in range(0, n, PREFILL_TILE):
                    tile_list.append((t + q0, min(PREFILL_TILE, n - q0), row, start + q0))
                    n_tiles += 1
            t += n
        # tiles with the most keys first, so that the long ones do not form the tail
        tile_list.sort(key=lambda ti: -(ti[3] + ti[1]))
        for i, ti in enumerate(tile_list):
            tiles[4 * i:4 * i + 4] = ti
        view[0], view[1], view[2], view[3] = n_dec, n_tiles, max_ctx, 0
        single = single and n_dec > 0
        if bucketed:
            return (size_class(n_dec) if n_dec else 0, size_class(n_tiles) if n_tiles else 0,
                    single)
        return n_dec, n_tiles, single

    def make_plan(self, host_batch, n_rows: int, page_size: int) -> AttentionPlan:
        """A plan built and uploaded on the spot (the runner packs it into the step's single
        upload instead)."""
        import numpy as np
        view = np.zeros(self.attention_plan_ints(n_rows, len(host_batch)), dtype=np.int32)
        dec, tiles, single = self.plan_attention(view, host_batch, n_rows, len(host_batch),
                                                 page_size, False)
        return AttentionPlan(torch.from_numpy(view).to(self.device), n_rows, dec, tiles, single)

    def _scratch_buffer(self, name, numel, dtype):
        key = (name, dtype)
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)       # captured graphs may still point into it
            buf = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            self._scratch[key] = buf
        return buf

    def decode_wide(self, decode_cap: int, n_heads: int) -> int:
        """Warps per CTA of the decode attention: 16 (code 2) while token x head count is below
        the SM count, 8 (code 1) up to twice that, else 4 (code 0)."""
        if self.decode_force is not None:
            return self.decode_force[0]
        pairs = decode_cap * n_heads
        return 2 if pairs <= self.sm_count else (1 if pairs <= 2 * self.sm_count else 0)

    def decode_splits(self, decode_cap: int, n_heads: int, max_context: int) -> int:
        """Slices between CTAs the context of a single-query token is cut into: one wave of
        CTAs over the SMs, slices of at least 64 keys (in the manner of the reference's
        ``choose_num_splits``, heteroserve/model/paged_attn_v3.py:212-232).  Slices cost a
        round trip through scratch memory, so they are used only when token x head count is
        small."""
        pairs = max(1, decode_cap * n_heads)
        wide = self.decode_wide(decode_cap, n_heads)
        if self.decode_force is not None:
            return self.decode_force[1]
        want = max(1, round(self.sm_count / pairs)) if wide == 2 else 1
        per_warp = 32 * 16 * (4, 8, 16)[wide]        # keys a CTA can cover: 32 pages per warp
        need = -(-max_context // per_warp)
        return max(1, need, min(want, max(1, max_context // 64), 32))

    FAST_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
    _lib_split_clusters = True     # what the library's switch was last set to

    def _fast_ok(self, qkv, g, plan, n, scale=1.0) -> bool:
        return (plan is not None and self.fast_attention and qkv.dtype == torch.bfloat16
                and g.window == 0 and g.head_dim in self.FAST_HEAD_DIMS and plan.n_rows >= n
                and scale > 0)

    def attention_append(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status,
                         plan=None, writes=True):
        """Append the new keys/values to the pages (if ``writes``), then attention.  When the
        step is made of single decoded tokens only, the decode kernel does both in one launch."""
        n = out.shape[0]
        fuse = (writes and self.fuse_append and self._fast_ok(qkv, g, plan, n, scale)
                and plan.tile_cap == 0 and plan.decode_cap > 0 and plan.single_new)
        if writes and not fuse:
            self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
        self.attention(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                       _fuse_append=fuse)

    def _attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan, n,
                   fuse=False):
        if self._fast_ok(qkv, g, plan, n, scale):
            self._attention_fast(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                                 fuse)
            return
        self.launches += 1
        # steps of prompt portions (four tokens a request or more on average): a CTA serves four
        # neighbours of the batch, which share the staged keys when they are one request's
        # (with a work list: the step has prompt portions; the counts may be padded ones)
        group = 4 if (plan.tile_cap > 0 if plan is not None else n >= 4 * table.shape[0]) else 1
        _check(self.lib.hs_attention_simt_grouped(
            _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req), n,
            g.n_heads, g.n_kv_heads, g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off,
            g.k_off, g.v_off, g.qkv_stride, g.window, scale, _DT[qkv.dtype], group, _ptr(status),
            self._stream()), f"attention(head_dim={g.head_dim}, heads={g.n_heads})")

    def _attention_fast(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan,
                        fuse=False):
        d = plan.data
        nr = plan.n_rows
        head = d
        dec_info = d[4:]
        tile_info = d[4 + plan_decode_ints(nr):]
        st = self._stream()
        if plan.decode_cap:
            max_ctx = g.max_pages * g.page_size
            group = g.n_heads // g.n_kv_heads
            use_mma = (self.decode_mma and self.decode_force is None
                       and g.head_dim in (32, 64, 128) and group <= 16)
            if use_mma:
                # slices of at most 2,048 keys; a long table and so few (token, head) pairs that
                # they leave SMs idle: more, shorter slices (of 512 keys or more), a CTA an SM
                splits = max(1, -(-max_ctx // 2048))
                pairs = plan.decode_cap * g.n_kv_heads
                if max_ctx >= 2048 and pairs * splits <= self.sm_count:
                    splits = max(splits, min(-(-max_ctx // 512), self.sm_count // pairs))
            else:
                splits = self.decode_splits(plan.decode_cap, g.n_heads, max_ctx)
            acc = ml = cnt = None
            if splits > 1:
                rows = plan.decode_cap * g.n_heads * splits
                acc = self._scratch_buffer("decode_acc", rows * g.head_dim, torch.float32)
                ml = self._scratch_buffer("decode_ml", rows * 2, torch.float32)
                cnt = self._scratch_buffer("decode_counters", plan.decode_cap * g.n_heads,
                                           torch.int32)
            self.launches += 1
            if use_mma:
                code = self.lib.hs_attention_decode_mma(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(dec_info), _ptr(head),
                    plan.decode_cap, g.n_heads, g.n_kv_heads, g.head_dim, g.page_size,
                    g.num_pages, g.max_pages, g.q_off, g.k_off, g.v_off, g.qkv_stride, scale,
                    splits, int(bool(fuse)), int(self.pdl), _ptr(acc), _ptr(ml), _ptr(cnt),
                    _ptr(status), st)
                what = f"attention_decode_mma(head_dim={g.head_dim})"
            else:
                code = self.lib.hs_attention_decode_append(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                    _ptr(dec_info), _ptr(head), plan.decode_cap, g.n_heads, g.n_kv_heads,
                    g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.k_off, g.v_off,
                    g.qkv_stride, g.window, scale, splits, int(bool(fuse)),
                    int(self.decode_wide(plan.decode_cap, g.n_heads)), int(self.pdl), _ptr(acc),
                    _ptr(ml), _ptr(cnt), _ptr(status), st)
                what = f"attention_decode(head_dim={g.head_dim})"
            if code == -1:
                # a shape the decode kernels do not take: the general kernel serves every token
                # of the batch (it needs no work list); a fused append is done first
                if fuse:
                    self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
                _check(self.lib.hs_attention_simt(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                    out.shape[0], g.n_heads, g.n_kv_heads, g.head_dim, g.page_size, g.num_pages,
                    g.max_pages, g.q_off, g.k_off, g.v_off, g.qkv_stride, g.window, scale,
                    _DT[qkv.dtype], _ptr(status), st),
                    f"attention(head_dim={g.head_dim}, heads={g.n_heads})")
                return
            _check(code, what)
        if plan.tile_cap:
            self.launches += 1
            counter = self._scratch_buffer("prefill_counter", 1, torch.int32)
            if self.tc_attention and g.head_dim == 64:
                code = self.lib.hs_attention_prefill_tc(
                    _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tile_info), _ptr(head),
                    plan.tile_cap, _ptr(counter), qkv.shape[0], g.n_heads, g.n_kv_heads,
                    g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.qkv_stride,
                    scale, _ptr(status), st)
                if code != -1:
                    _check(code, "attention_prefill_tc")
                    return
            _check(self.lib.hs_attention_prefill(
                _ptr(out), _ptr(qkv), _ptr(pool), _ptr(table), _ptr(tok_pos), _ptr(tok_req),
                _ptr(tile_info), _ptr(head), plan.tile_cap,
                _ptr(self._scratch_buffer("prefill_counter", 1, torch.int32)), g.n_heads, g.n_kv_heads,
                g.head_dim, g.page_size, g.num_pages, g.max_pages, g.q_off, g.qkv_stride, scale,
                _ptr(status), st), f"attention_prefill(head_dim={g.head_dim})")

    # -- the whole decode step in one kernel ----------------------------------------
    FUSED_MAX_TOKENS = 16

    def fused_decode_supports(self, *, width, inner, n_heads, head_dim, n_kv_heads, page_size,
                              window) -> bool:
        """Whether the persistent decode kernel serves a model of these sizes at all (bfloat16,
        heads of 64 without grouping, pages of 16, widths in multiples of 64 up to 2,048)."""
        return bool(self.fused_decode_on and self.lib.hs_decode_persistent_supports(
            int(width), int(inner), int(n_heads), int(head_dim), int(n_kv_heads),
            int(page_size), int(window)))

    def fused_decode_build(self, layers, *, head_weight, pool, width, inner, vocab):
        """Descriptor records of a model for :meth:`fused_decode`: per layer call its four
        matrices (repacked here, see :func:`pack_weight_units`: the kernel keeps its own copy of
        every matrix, laid out so that what a CTA streams is contiguous), its vectors and
        constants, and once the head and the tensor map of the cache storage.  ``layers`` is a list of dictionaries with the keys ``w_qkv w_out
        w_fc w_mlp`` ([features, k] bfloat16), ``b_qkv b_out b_fc b_mlp ln1_g ln1_b ln2_g ln2_b``
        (float32 or None for the biases), ``eps1 eps2 scale act entry``; ``pool`` is the cache
        group's storage ``[entries, pages, 2, heads, 16, 64]``."""
        lib = self.lib
        lb, tb = lib.hs_decode_persistent_layer_bytes(), lib.hs_decode_persistent_tables_bytes()
        host = torch.zeros(len(layers) * lb + tb, dtype=torch.uint8)
        base = host.data_ptr()
        _want(pool, "pool", torch.bfloat16, 6)
        rows_per_entry = pool.shape[1] * pool.shape[2] * pool.shape[3] * pool.shape[4]
        keep = [pool]
        packs: dict[int, torch.Tensor] = {}
        for i, L in enumerate(layers):
            for nm in ("w_qkv", "w_out", "w_fc", "w_mlp"):
                _want(L[nm], nm, torch.bfloat16, 2)
            for nm in ("ln1_g", "ln1_b", "ln2_g", "ln2_b"):
                _want(L[nm], nm, torch.float32, 1)
            for nm in ("b_qkv", "b_out", "b_fc", "b_mlp"):
                if L[nm] is not None:
                    _want(L[nm], nm, torch.float32, 1)
            if (tuple(L["w_qkv"].shape) != (3 * width, width) or tuple(L["w_out"].shape) != (width, width)
                    or tuple(L["w_fc"].shape) != (inner, width) or tuple(L["w_mlp"].shape) != (width, inner)):
                raise KernelError("fused_decode_build: matrix shapes do not fit the sizes")
            keep += [L[k] for k in L if isinstance(L[k], torch.Tensor) and not k.startswith("w_")]
            packed = [packs.setdefault(L[nm].data_ptr(), pack_weight_units(L[nm]))
                      for nm in ("w_qkv", "w_out", "w_fc", "w_mlp")]      # a shared layer: once
            _check(lib.hs_decode_persistent_layer(
                c_void_p(base + i * lb), _ptr(packed[0]), _ptr(packed[1]), _ptr(packed[2]),
                _ptr(packed[3]), _ptr(L["b_qkv"]), _ptr(L["b_out"]), _ptr(L["b_fc"]),
                _ptr(L["b_mlp"]), _ptr(L["ln1_g"]), _ptr(L["ln1_b"]), _ptr(L["ln2_g"]),
                _ptr(L["ln2_b"]), float(L["eps1"]), float(L["eps2"]), float(L["scale"]),
                int(ACTIVATIONS[L["act"]]), int(width), int(inner),
                ctypes.c_longlong(int(L["entry"]) * rows_per_entry)), "decode_persistent_layer")
        _want(head_weight, "head_weight", torch.bfloat16, 2)
        head_packed = pack_weight_units(head_weight)
        keep += list(packs.values()) + [head_packed]
        _check(lib.hs_decode_persistent_tables(
            c_void_p(base + len(layers) * lb), _ptr(head_packed), int(vocab), int(width),
            _ptr(pool), ctypes.c_longlong(pool.shape[0] * rows_per_entry)),
            "decode_persistent_tables")
        dev = host.to(self.device)
        return FusedTables(dev, len(layers), lb, keep)

    def fused_decode(self, tables, *, wte, wpe, lnf_g, lnf_b, eps_f, width, inner, vocab,
                     n_heads, pool, num_pages, max_pages, x, qkv, att, u, logits, tokens,
                     feedback, tok_ids, tok_pos, tok_req, table, logit_rows, samp_slot,
                     plan_head, n_tokens, n_requests, n_logit_rows, status, stop_after=0):
        """One decode step of up to 16 single-query tokens in one persistent kernel: embedding,
        every layer, final norm, head, greedy tokens (``tokens[:n_logit_rows]``, the status
        word behind them).  Buffers are the caller's; scratch is this object's."""
        M, W = int(n_tokens), int(n_logit_rows)
        if not 0 < M <= self.FUSED_MAX_TOKENS or W > self.FUSED_MAX_TOKENS:
            raise KernelError(f"fused_decode: {M} tokens / {W} wanted rows exceed "
                              f"{self.FUSED_MAX_TOKENS}")
        _want(x, "x", torch.float32, 2)
        for t, nm, wd in ((qkv, "qkv", 3 * width), (att, "att", width), (u, "u", inner)):
            _want(t, nm, torch.bfloat16, 2)
            if t.shape[0] < M or t.shape[1] != wd:
                raise KernelError(f"fused_decode: {nm} has shape {tuple(t.shape)}")
        if x.shape[0] < M or x.shape[1] != width:
            raise KernelError("fused_decode: x does not fit")
        if W:
            _want(logits, "logits", torch.float32, 2)
            if logits.shape[0] < W or logits.shape[1] != vocab:
                raise KernelError("fused_decode: logits do not fit")
        _want(tokens, "tokens", torch.int32, 1)
        if tokens.shape[0] < W + 1:
            raise KernelError("fused_decode: tokens has no room for the status word")
        for t, nm in ((tok_ids, "tok_ids"), (tok_pos, "tok_pos"), (tok_req, "tok_req")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < M:
                raise KernelError(f"fused_decode: {nm} shorter than the tokens")
        _want(table, "table", torch.int32, 2)
        if table.shape[1] != max_pages:
            raise KernelError("fused_decode: block table width != max_pages")
        grid = self.lib.hs_decode_persistent_grid()
        if grid <= 0:
            raise KernelError("fused_decode: the kernel does not fit this device")
        S = self.lib.hs_decode_persistent_slices(int(n_requests), int(n_heads))
        acc = ml = None
        if S > 1:
            acc = self._scratch_buffer("fused_att_acc", M * n_heads * S * 64, torch.float32)
            ml = self._scratch_buffer("fused_att_ml", M * n_heads * S * 2, torch.float32)
        amax_v = self._scratch_buffer("fused_amax_val", grid * 16, torch.float32)
        amax_i = self._scratch_buffer("fused_amax_idx", grid * 16, torch.int32)
        sync = self._scratch_buffer("fused_sync", 4, torch.int32)
        self.launches += 1
        _check(self.lib.hs_decode_persistent(
            tables.layers_ptr, tables.tables_ptr, tables.n_layers, _ptr(wte), _ptr(wpe),
            _ptr(lnf_g), _ptr(lnf_b), float(eps_f), int(width), int(inner), int(vocab),
            int(n_heads), int(wpe.shape[0]), _ptr(pool), int(num_pages), int(max_pages), _ptr(x),
            _ptr(qkv), _ptr(att), _ptr(u), _ptr(logits), _ptr(acc), _ptr(ml), _ptr(amax_v),
            _ptr(amax_i), _ptr(tokens), _ptr(feedback), int(feedback.shape[0]), _ptr(tok_ids),
            _ptr(tok_pos), _ptr(tok_req), _ptr(table), _ptr(logit_rows), _ptr(samp_slot),
            _ptr(plan_head), M, W, W, S, _ptr(sync), _ptr(status), int(stop_after),
            self._stream()), "decode_persistent")

    # -- sampling ---------------------------------------------------------------
    def argmax(self, out, logits):
        _want(out, "out", torch.int32, 1)
        _want(logits, "logits", torch.float32, 2)
        rows, vocab = logits.shape
        if out.shape[0] < rows:
            raise KernelError("argmax: out shorter than the rows")
        self.launches += 1
        _check(self.lib.hs_argmax(_ptr(out), _ptr(logits), rows, vocab, self._stream()), "argmax")

    def sample(self, out, logits, temperature, top_k, seed_lo, seed_hi, position,
               feedback=None, feedback_slot=None, status_word=None):
        """Per row: argmax if temperature <= 0, else a draw from softmax(logits/temperature)
        restricted to the top_k largest when 0 < top_k < vocab.  With ``feedback`` and
        ``feedback_slot`` row i also stores its token to ``feedback[feedback_slot[i]]`` (slots
        below zero are skipped).  With ``status_word`` (one int32 on the device) its value is
        stored to ``out[rows]``: the engine's status travels behind the tokens."""
        _want(out, "out", torch.int32, 1)
        _want(logits, "logits", torch.float32, 2)
        rows, vocab = logits.shape
        _want(temperature, "temperature", torch.float32, 1)
        for t, nm in ((top_k, "top_k"), (seed_lo, "seed_lo"), (seed_hi, "seed_hi"),
                      (position, "position")):
            _want(t, nm, torch.int32, 1)
            if t.shape[0] < rows:
                raise KernelError(f"sample: {nm} shorter than the rows")
        if out.shape[0] < rows or temperature.shape[0] < rows:
            raise KernelError("sample: out/temperature shorter than the rows")
        if (feedback is None) != (feedback_slot is None):
            raise KernelError("sample: feedback and feedback_slot come together")
        if feedback is not None:
            _want(feedback, "feedback", torch.int32, 1)
            _want(feedback_slot, "feedback_slot", torch.int32, 1)
            if feedback_slot.shape[0] < rows:
                raise KernelError("sample: feedback_slot shorter than the rows")
        if status_word is not None:
            _want(status_word, "status_word", torch.int32, 1)
            if out.shape[0] < rows + 1:
                raise KernelError("sample: out has no room for the status word")
        self.launches += 1
        _check(self.lib.hs_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(top_k),
                                  _ptr(seed_lo), _ptr(seed_hi), _ptr(position), rows, vocab,
                                  _ptr(feedback), _ptr(feedback_slot), _ptr(status_word),
                                  self._stream()), "sample")
