"""Toy parts that bring CUDA kernels of their own, defined and compiled here, not in the
framework: a norm without mean or bias (root-mean-square), a mixer with state of its own that
runs on the device (a decayed running sum per channel, carried in the state slots), and an
arrangement with ONE norm shared by a mixer and a feed-forward that run side by side.

They show three things the standard parts do not: a part can compile and call its own kernel
(`CudaOps.load_extension` / `register_kernel`; the package's wrapper file is not edited), an
arrangement can have other parts than norm1/mixer/norm2/feed_forward, and a model whose mixer
keeps per-request state is captured in CUDA graphs like any other when its parts run on the
device.  None of this becomes a model of anyone's."""

import pytest
import torch
from ctypes import c_float, c_int, c_void_p

import plain_gpt2
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import (Block, LayerCall, LayerSpec, Mixer, Model, ModelSpec, Norm,
                                     PartSpec, TensorRequest, register_arrangement,
                                     register_mixer, register_norm)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDTH, VOCAB, POSITIONS, DECAY, EPS = 48, 53, 96, 0.75, 1e-6

TOY_CU = r"""
#include "common.cuh"

namespace {

// y[r] = x[src(r)] / sqrt(mean(x^2) + eps) * w, one warp per row, float32 statistics
template <typename OutT>
__global__ void toy_rms_kernel(OutT* out, const float* x, const float* w, const int* rows,
                               int n, int width, float eps) {
  const int r = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (r >= n) return;
  const int lane = threadIdx.x % 32;
  const float* src = x + (size_t)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = lane; c < width; c += 32) ss += src[c] * src[c];
  ss = hs::warp_sum(ss);
  const float inv = rsqrtf(ss / width + eps);
  for (int c = lane; c < width; c += 32)
    out[(size_t)r * width + c] = hs::from_f<OutT>(src[c] * inv * w[c]);
}

// per request and channel: s = decay * s + h[t];  x[t] += gain * s, over the request's tokens
// of this step in order; s lives in state[slot] between steps
template <typename HT>
__global__ void toy_scan_kernel(float* x, const HT* h, float* state, const float* gain,
                                const int* req_start, const int* req_len, const int* req_slot,
                                int width, float decay) {
  const int r = blockIdx.x;
  const int n = req_len[r];
  if (n <= 0) return;                               // a padding request of the size class
  const int t0 = req_start[r];
  float* st = state + (size_t)req_slot[r] * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float s = st[c];
    for (int i = 0; i < n; ++i) {
      s = decay * s + hs::to_f(h[(size_t)(t0 + i) * width + c]);
      x[(size_t)(t0 + i) * width + c] += gain[c] * s;
    }
    st[c] = s;
  }
}

}  // namespace

HS_EXPORT int toy_rms(void* out, const float* x, const float* w, const int* rows, int n,
                      int width, float eps, int out_dtype, void* stream) {
  if (!out || !x || !w || n < 0 || width <= 0) return HS_ERR_ARGUMENT;
  if (n == 0) return HS_OK;
  dim3 grid((n + 3) / 4), block(128);
  if (out_dtype == HS_DT_F32)
    toy_rms_kernel<float><<<grid, block, 0, (cudaStream_t)stream>>>((float*)out, x, w, rows, n, width, eps);
  else
    toy_rms_kernel<__nv_bfloat16><<<grid, block, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)out, x, w, rows, n, width, eps);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int toy_scan(float* x, const void* h, float* state, const float* gain,
                       const int* req_start, const int* req_len, const int* req_slot,
                       int n_requests, int width, float decay, int h_dtype, void* stream) {
  if (!x || !h || !state || !gain || !req_start || !req_len || !req_slot) return HS_ERR_ARGUMENT;
  if (n_requests <= 0) return HS_OK;
  if (h_dtype == HS_DT_F32)
    toy_scan_kernel<float><<<n_requests, 64, 0, (cudaStream_t)stream>>>(
        x, (const float*)h, state, gain, req_start, req_len, req_slot, width, decay);
  else
    toy_scan_kernel<__nv_bfloat16><<<n_requests, 64, 0, (cudaStream_t)stream>>>(
        x, (const __nv_bfloat16*)h, state, gain, req_start, req_len, req_slot, width, decay);
  HS_LAUNCH_CHECK();
  return HS_OK;
}
"""

_DT = {torch.float32: 0, torch.bfloat16: 1}
_source = {}


def _library(ops, tmp_dir):
    if "lib" not in _source:
        path = tmp_dir / "toy_parts.cu"
        path.write_text(TOY_CU)
        _source["lib"] = ops.load_extension("toy_parts", [path])
    return _source["lib"]


class ToyRmsNorm(Norm):
    def __init__(self, *, width, eps, weight):
        self.width, self.eps, self.name = width, float(eps), weight
        self.fn = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.width,), "vector")}

    def bind(self, tensors):
        self.w = tensors[self.name]

    def forward(self, ctx, out, x, rows=None):
        if self.fn is None:         # declared once, on the library this test compiled
            P, I, F = c_void_p, c_int, c_float
            self.fn = ctx.ops.register_kernel("toy_rms", [P, P, P, P, I, I, F, I, P],
                                              lib=_source["lib"])
        self.fn(out.data_ptr(), x.data_ptr(), self.w.data_ptr(),
                None if rows is None else rows.data_ptr(), out.shape[0], self.width, self.eps,
                _DT[out.dtype], ctx.ops.stream())


class ToyScanMixer(Mixer):
    def __init__(self, *, width, gain):
        self.width, self.name = width, gain
        self.fn = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.width,), "vector")}

    def bind(self, tensors):
        self.gain = tensors[self.name]

    def state_shape(self):
        return (self.width,)

    def forward(self, ctx, h, x, cache):
        if self.fn is None:
            P, I, F = c_void_p, c_int, c_float
            self.fn = ctx.ops.register_kernel("toy_scan", [P, P, P, P, P, P, P, I, I, F, I, P],
                                              lib=_source["lib"])
        self.fn(x.data_ptr(), h.data_ptr(), ctx.state().data_ptr(), self.gain.data_ptr(),
                ctx.req_start.data_ptr(), ctx.req_len.data_ptr(), ctx.req_slot.data_ptr(),
                ctx.n_requests, self.width, DECAY, _DT[h.dtype], ctx.ops.stream())


class ParallelBlock(Block):
    """h = norm(x);  x += mixer(h) + feed_forward(h): one norm, two parts side by side."""

    slots = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, ctx, x, cache):
        h = ctx.buffer("normed", (x.shape[0], x.shape[1]), ctx.dtype)
        self.norm.forward(ctx, h, x)
        self.mixer.forward(ctx, h, x, cache)
        self.feed_forward.forward(ctx, h, x)


def _spec():
    W = WIDTH
    dense = lambda p: PartSpec("dense", dict(width=W, inner=2 * W, activation="gelu_tanh",   # noqa: E731
                                             in_weight=p + "fc", in_bias=None,
                                             out_weight=p + "pr", out_bias=None,
                                             stored_in_out=False))
    layers = (
        LayerSpec("toy_parallel", norm=PartSpec("toy_rms", dict(width=W, eps=EPS, weight="b0.nw")),
                  mixer=PartSpec("toy_scan", dict(width=W, gain="b0.gain")),
                  feed_forward=dense("b0.")),
        LayerSpec(norm1=PartSpec("layernorm", dict(width=W, eps=1e-5, weight="b1.n1w", bias="b1.n1b")),
                  mixer=PartSpec("causal_attention", dict(
                      width=W, n_heads=3, head_dim=16, scale=0.25, qkv_weight="b1.qkv",
                      qkv_bias=None, out_weight="b1.o", out_bias=None, stored_in_out=False)),
                  norm2=PartSpec("toy_rms", dict(width=W, eps=EPS, weight="b1.n2w")),
                  feed_forward=dense("b1.")),
    )
    return ModelSpec(
        name="toy-kernels", vocab_size=VOCAB, width=W, max_positions=POSITIONS,
        embedding=PartSpec("token_table", dict(vocab_size=VOCAB, width=W, table="emb")),
        position=PartSpec("none", {}), layers=layers, schedule=(LayerCall(0), LayerCall(1)),
        final_norm=PartSpec("toy_rms", dict(width=W, eps=EPS, weight="nfw")),
        head=PartSpec("linear", dict(vocab_size=VOCAB, width=W, weight="emb")))


def _rms(x, w):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + EPS) * w


def _plain(stored, tokens, round_to=None):
    w = {k: (v.to(round_to) if round_to is not None and v.dim() == 2 else v).double()
         for k, v in stored.items()}
    x = w["emb"][torch.tensor(tokens)]
    h = _rms(x, w["b0.nw"])
    s = torch.zeros(WIDTH, dtype=torch.float64)
    ys = []
    for t in range(len(tokens)):
        s = DECAY * s + h[t]
        ys.append(w["b0.gain"] * s)
    x = x + torch.stack(ys) + plain_gpt2.gelu_new(h @ w["b0.fc"].T) @ w["b0.pr"].T
    h = plain_gpt2.layer_norm(x, w["b1.n1w"], w["b1.n1b"], 1e-5)
    qkv = h @ w["b1.qkv"].T
    q, k, v = (plain_gpt2.split_heads(qkv[:, j * 48:(j + 1) * 48], 3) for j in range(3))
    x = x + plain_gpt2.causal_attention(q, k, v, 0.25) @ w["b1.o"].T
    x = x + plain_gpt2.gelu_new(_rms(x, w["b1.n2w"]) @ w["b1.fc"].T) @ w["b1.pr"].T
    return _rms(x, w["nfw"]) @ w["emb"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["float32", "bfloat16"])
def test_parts_with_their_own_kernels_state_and_arrangement_under_cuda_graphs(tmp_path, dtype):
    from hetero_serve_b200.kernels import CudaOps
    ops = CudaOps(DEV)
    _library(ops, tmp_path)
    register_norm("toy_rms", ToyRmsNorm, replace=True)
    register_mixer("toy_scan", ToyScanMixer, replace=True)
    register_arrangement("toy_parallel", ParallelBlock, replace=True)
    with pytest.raises(ValueError, match="missing"):          # an arrangement checks its parts
        Model(ModelSpec(name="bad", vocab_size=VOCAB, width=WIDTH, max_positions=8,
                        embedding=_spec().embedding, position=_spec().position,
                        layers=(LayerSpec("toy_parallel", mixer=_spec().layers[0].mixer),),
                        schedule=(LayerCall(0),), final_norm=_spec().final_norm,
                        head=_spec().head))
    model = Model(_spec())
    assert model.capturable and list(model.state_shapes.values()) == [(WIDTH,)]
    g = torch.Generator().manual_seed(8)
    stored = {n: torch.randn(r.shape, generator=g) * (0.25 if len(r.shape) == 2 else 0.1)
              + (1.0 if n.endswith("w") and len(r.shape) == 1 else 0.0)
              for n, r in model.tensor_requests().items()}
    model.bind(stored, dtype, DEV)
    rn = Runner(model, num_pages=12, page_size=16, max_requests=3, dtype=dtype, device=DEV,
                ops=ops, cuda_graphs=True)
    a = [(5 * i + 3) % VOCAB for i in range(60)]
    b = [(11 * i + 7) % VOCAB for i in range(40)]
    round_to = torch.bfloat16 if dtype == torch.bfloat16 else None
    ref = {"a": _plain(stored, a, round_to), "b": _plain(stored, b, round_to)}
    got = {"a": {}, "b": {}}
    plan = [[("a", 0, 20)], [("b", 0, 9), ("a", 20, 22)], [("a", 22, 45), ("b", 9, 10)]]
    # the same shapes again and again: the captured graphs are replayed, state and all
    plan += [[("a", 45 + i, 46 + i), ("b", 10 + i, 11 + i)] for i in range(15)]
    for step in plan:
        entries = [StepEntry(r, (a if r == "a" else b)[lo:hi], want=list(range(hi - lo)))
                   for r, lo, hi in step]
        res = rn.step(entries)
        for (r, w_), row in zip(res.rows, res.logits.double().cpu()):
            lo = [lo for rr, lo, hi in step if rr == r][0]
            got[r][lo + w_] = row
    assert len(rn._graphs) >= 3                               # captured, although there is state
    tol = 5e-5 if dtype == torch.float32 else 6e-2
    for r in ("a", "b"):
        err = max(float((got[r][i] - ref[r][i]).abs().max()) for i in got[r])
        assert err < tol, (r, err)
    # a slot is cleared for its next owner, also under graphs
    rn.close("a")
    res = rn.step([StepEntry("c", b[:20], want=[19])])
    assert (res.logits[0].double().cpu() - ref["b"][19]).abs().max() < tol
    rn.manager.check()
