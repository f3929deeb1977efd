"""A toy mixer with state of its own, defined here, is registered, built into a model and
stepped without any change to the framework's files: the mixer is a decayed running mean of
the inputs of a request (state: one vector per request in the state slots), written in plain
PyTorch.  It never becomes a model of anyone's; it shows that the part interface, the state
slots and the step function carry a mixer that is not attention."""

import pytest
import torch

import plain_gpt2
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import (LayerCall, LayerSpec, Mixer, Model, ModelSpec, PartSpec,
                                     TensorRequest, register_mixer)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DECAY = 0.8


class RunningMeanMixer(Mixer):
    """y_t = W (s_t),  s_t = DECAY * s_{t-1} + h_t  with s carried across steps in a state slot."""

    capturable = False      # it walks the batch on the host: no CUDA graph for its model

    def __init__(self, *, width, weight):
        self.width, self.name = width, weight
        self.w = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.width, self.width), "matrix")}

    def bind(self, tensors):
        self.w = tensors[self.name]

    def state_shape(self):
        return (self.width,)

    def forward(self, ctx, h, x, cache):
        state = ctx.state()                                  # [slots, width] float32
        t = 0
        for _req, slot, _start, n in ctx.host:               # the batch, request by request
            s = state[slot]
            for i in range(n):
                s = DECAY * s + h[t + i].float()
                x[t + i] += (self.w.float() @ s)
            state[slot] = s
            t += n


def _spec(width, vocab, positions, mixed: bool):
    def layer(i, toy):
        p = f"b{i}."
        mixer = (PartSpec("toy_running_mean", dict(width=width, weight=p + "mix")) if toy else
                 PartSpec("causal_attention", dict(
                     width=width, n_heads=2, head_dim=16, scale=0.25, qkv_weight=p + "qkv",
                     qkv_bias=None, out_weight=p + "o", out_bias=None, stored_in_out=False)))
        return LayerSpec(
            norm1=PartSpec("layernorm", dict(width=width, eps=1e-5, weight=p + "n1w", bias=p + "n1b")),
            mixer=mixer,
            norm2=PartSpec("layernorm", dict(width=width, eps=1e-5, weight=p + "n2w", bias=p + "n2b")),
            feed_forward=PartSpec("dense", dict(width=width, inner=2 * width, activation="gelu_tanh",
                                                in_weight=p + "fc", in_bias=None,
                                                out_weight=p + "pr", out_bias=None,
                                                stored_in_out=False)))
    layers = (layer(0, True), layer(1, False)) if mixed else (layer(0, True),)
    return ModelSpec(
        name="toy", vocab_size=vocab, width=width, max_positions=positions,
        embedding=PartSpec("token_table", dict(vocab_size=vocab, width=width, table="emb")),
        position=PartSpec("none", {}), layers=layers,
        schedule=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", dict(width=width, eps=1e-5, weight="nfw", bias="nfb")),
        head=PartSpec("linear", dict(vocab_size=vocab, width=width, weight="emb")))


def _plain(stored, spec, tokens):
    w = {k: v.double() for k, v in stored.items()}
    x = w["emb"][torch.tensor(tokens)]
    for i, ls in enumerate(spec.layers):
        p = f"b{i}."
        h = plain_gpt2.layer_norm(x, w[p + "n1w"], w[p + "n1b"], 1e-5)
        if ls.mixer.kind == "toy_running_mean":
            s = torch.zeros(x.shape[1], dtype=torch.float64)
            ys = []
            for t in range(len(tokens)):
                s = DECAY * s + h[t]
                ys.append(w[p + "mix"] @ s)
            x = x + torch.stack(ys)
        else:
            qkv = h @ w[p + "qkv"].T
            q, k, v = (plain_gpt2.split_heads(qkv[:, j * 32:(j + 1) * 32], 2) for j in range(3))
            x = x + plain_gpt2.causal_attention(q, k, v, 0.25) @ w[p + "o"].T
        h = plain_gpt2.layer_norm(x, w[p + "n2w"], w[p + "n2b"], 1e-5)
        x = x + plain_gpt2.gelu_new(h @ w[p + "fc"].T) @ w[p + "pr"].T
    return plain_gpt2.layer_norm(x, w["nfw"], w["nfb"], 1e-5) @ w["emb"].T


@pytest.mark.parametrize("mixed", [False, True], ids=["toy_only", "toy_and_attention"])
def test_toy_mixer_with_state_registers_builds_and_steps(mixed):
    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)
    spec = _spec(width=32, vocab=50, positions=64, mixed=mixed)
    model = Model(spec)
    assert list(model.state_shapes.values()) == [(32,)]
    assert len(model.cache_groups) == (1 if mixed else 0)       # pages only where attention is
    g = torch.Generator().manual_seed(3)
    stored = {n: torch.randn(r.shape, generator=g) * (0.2 if len(r.shape) == 2 else 0.1)
              + (1.0 if n.endswith("w") and len(r.shape) == 1 else 0.0)
              for n, r in model.tensor_requests().items()}
    model.bind(stored, torch.float32, DEV)
    rn = Runner(model, num_pages=8, page_size=16, max_requests=3, dtype=torch.float32, device=DEV,
                prefix_cache=True, cuda_graphs=True)
    assert not rn.manager.prefix_cache          # state rules prefix reuse out
    a = [(3 * i + 1) % 50 for i in range(30)]
    b = [(7 * i + 2) % 50 for i in range(21)]
    ref_a, ref_b = _plain(stored, spec, a), _plain(stored, spec, b)
    got = {"a": {}, "b": {}}
    # two requests interleaved, cut differently, each keeping its own state between steps
    plan = [[("a", 0, 7)], [("b", 0, 20), ("a", 7, 8)], [("a", 8, 19)], [("b", 20, 21), ("a", 19, 30)]]
    for step in plan:
        entries = [StepEntry(r, (a if r == "a" else b)[lo:hi], want=list(range(hi - lo)))
                   for r, lo, hi in step]
        res = rn.step(entries)
        for (r, w_), row in zip(res.rows, res.logits.double().cpu()):
            lo = [lo for rr, lo, hi in step if rr == r][0]
            got[r][lo + w_] = row
    for r, ref in (("a", ref_a), ("b", ref_b)):
        assert sorted(got[r]) == list(range(len(ref)))
        err = max(float((got[r][i] - ref[i]).abs().max()) for i in got[r])
        assert err < 5e-5, (r, err)
    # a slot is cleared when it is given to the next request
    rn.close("a")
    res = rn.step([StepEntry("c", b, want=[20])])
    assert (res.logits[0].double().cpu() - ref_b[20]).abs().max() < 5e-5
    rn.manager.check()
