"""Toy parts defined here, not in the framework: a feed-forward with routing (each token goes
to one of several small expert MLPs) and a position encoding that acts on queries and keys
instead of the embedding (a rotation of pairs by an angle that grows with the position).  Each
is registered from this file, built into a model beside the standard parts and stepped through
the runner under several ways of cutting the work; the logits must equal a plain computation
over whole sequences.  They never become a model of anyone's: they show that the part
interfaces carry parts that GPT-2 does not have."""

import math

import pytest
import torch

import plain_gpt2
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import (FeedForward, LayerCall, LayerSpec, Model, ModelSpec,
                                     PartSpec, PositionEncoding, TensorRequest,
                                     register_feed_forward, register_position)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WIDTH, HEADS, HEAD_DIM, VOCAB, POSITIONS, EXPERTS, INNER = 48, 3, 16, 61, 96, 3, 40


class RoutedFeedForward(FeedForward):
    """x += W2[e] gelu(W1[e] h) with e = argmax(h @ Wr^T), expert by expert (plain PyTorch)."""

    capturable = False          # which rows an expert gets is read back to the host

    def __init__(self, *, width, inner, experts, router, w_in, w_out):
        self.width, self.inner, self.experts = width, inner, experts
        self.names = (router, w_in, w_out)

    def tensor_requests(self):
        r, a, b = self.names
        return {r: TensorRequest((self.experts, self.width), "matrix"),
                a: TensorRequest((self.experts * self.inner, self.width), "matrix"),
                b: TensorRequest((self.experts * self.width, self.inner), "matrix")}

    def bind(self, tensors):
        r, a, b = self.names
        self.router = tensors[r]
        self.w_in = tensors[a].view(self.experts, self.inner, self.width)
        self.w_out = tensors[b].view(self.experts, self.width, self.inner)

    def forward(self, ctx, h, x):
        hf = h.float()
        choice = (hf @ self.router.float().T).argmax(-1)         # router logits in float32
        live = ctx.tok_req[:h.shape[0]] >= 0                     # padding rows of a size class
        for e in range(self.experts):
            rows = ((choice == e) & live).nonzero().squeeze(1)
            if rows.numel():
                u = plain_gpt2.gelu_new(hf[rows] @ self.w_in[e].float().T)
                x[rows] += u @ self.w_out[e].float().T


class PairRotation(PositionEncoding):
    """Rotates the pairs (2i, 2i+1) of every query and key head by pos * base^(-2i/D)."""

    acts_in_mixer = True

    def __init__(self, *, base):
        self.base = float(base)

    def transform_qk(self, ctx, qkv, g):
        T = qkv.shape[0]
        pos = ctx.tok_pos[:T].float().clamp(min=0)
        D = g.head_dim
        inv = self.base ** (-torch.arange(0, D, 2, device=qkv.device, dtype=torch.float32) / D)
        ang = pos[:, None] * inv[None, :]                        # angles in float32
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        for off, heads in ((g.q_off, g.n_heads), (g.k_off, g.n_kv_heads)):
            v = qkv[:, off:off + heads * D].float().view(T, heads, D // 2, 2)
            a, b = v[..., 0], v[..., 1]
            out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1)
            qkv[:, off:off + heads * D] = out.view(T, heads * D).to(qkv.dtype)


def _spec():
    def layer(i):
        p = f"b{i}."
        return LayerSpec(
            norm1=PartSpec("layernorm", dict(width=WIDTH, eps=1e-5, weight=p + "n1w", bias=p + "n1b")),
            mixer=PartSpec("causal_attention", dict(
                width=WIDTH, n_heads=HEADS, head_dim=HEAD_DIM, scale=1 / math.sqrt(HEAD_DIM),
                qkv_weight=p + "qkv", qkv_bias=None, out_weight=p + "o", out_bias=None,
                stored_in_out=False)),
            norm2=PartSpec("layernorm", dict(width=WIDTH, eps=1e-5, weight=p + "n2w", bias=p + "n2b")),
            feed_forward=(PartSpec("toy_routed", dict(width=WIDTH, inner=INNER, experts=EXPERTS,
                                                      router=p + "r", w_in=p + "e1", w_out=p + "e2"))
                          if i == 0 else
                          PartSpec("dense", dict(width=WIDTH, inner=2 * WIDTH, activation="gelu_tanh",
                                                 in_weight=p + "fc", in_bias=None,
                                                 out_weight=p + "pr", out_bias=None,
                                                 stored_in_out=False))))
    return ModelSpec(
        name="toy-parts", vocab_size=VOCAB, width=WIDTH, max_positions=POSITIONS,
        embedding=PartSpec("token_table", dict(vocab_size=VOCAB, width=WIDTH, table="emb")),
        position=PartSpec("toy_pair_rotation", dict(base=100.0)),
        layers=(layer(0), layer(1)), schedule=(LayerCall(0), LayerCall(1)),
        final_norm=PartSpec("layernorm", dict(width=WIDTH, eps=1e-5, weight="nfw", bias="nfb")),
        head=PartSpec("linear", dict(vocab_size=VOCAB, width=WIDTH, weight="emb")))


def _rotate(t, pos, base):
    """[H, T, D] rotated like PairRotation, in float64."""
    H, T, D = t.shape
    inv = base ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)
    ang = pos.double()[:, None] * inv[None, :]
    v = t.reshape(H, T, D // 2, 2)
    a, b = v[..., 0], v[..., 1]
    return torch.stack((a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()), -1).reshape(H, T, D)


def _plain(stored, tokens):
    w = {k: v.double() for k, v in stored.items()}
    x = w["emb"][torch.tensor(tokens)]
    pos = torch.arange(len(tokens))
    E = HEADS * HEAD_DIM
    for i in range(2):
        p = f"b{i}."
        h = plain_gpt2.layer_norm(x, w[p + "n1w"], w[p + "n1b"], 1e-5)
        qkv = h @ w[p + "qkv"].T
        q, k, v = (plain_gpt2.split_heads(qkv[:, j * E:(j + 1) * E], HEADS) for j in range(3))
        q, k = _rotate(q, pos, 100.0), _rotate(k, pos, 100.0)
        x = x + plain_gpt2.causal_attention(q, k, v, 1 / math.sqrt(HEAD_DIM)) @ w[p + "o"].T
        h = plain_gpt2.layer_norm(x, w[p + "n2w"], w[p + "n2b"], 1e-5)
        if i == 0:
            choice = (h @ w[p + "r"].T).argmax(-1)
            w1 = w[p + "e1"].view(EXPERTS, INNER, WIDTH)
            w2 = w[p + "e2"].view(EXPERTS, WIDTH, INNER)
            y = torch.stack([w2[int(e)] @ plain_gpt2.gelu_new(w1[int(e)] @ h[t])
                             for t, e in enumerate(choice)])
            x = x + y
        else:
            x = x + plain_gpt2.gelu_new(h @ w[p + "fc"].T) @ w[p + "pr"].T
    return plain_gpt2.layer_norm(x, w["nfw"], w["nfb"], 1e-5) @ w["emb"].T, choice


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_routed_feed_forward_and_rotating_positions_register_build_and_step(graphs):
    register_feed_forward("toy_routed", RoutedFeedForward, replace=True)
    register_position("toy_pair_rotation", PairRotation, replace=True)
    spec = _spec()
    model = Model(spec)
    g = torch.Generator().manual_seed(5)
    stored = {n: torch.randn(r.shape, generator=g) * (0.25 if len(r.shape) == 2 else 0.1)
              + (1.0 if n.endswith("w") and len(r.shape) == 1 else 0.0)
              for n, r in model.tensor_requests().items()}
    model.bind(stored, torch.float32, DEV)
    rn = Runner(model, num_pages=9, page_size=16, max_requests=3, dtype=torch.float32, device=DEV,
                cuda_graphs=graphs)
    a = [(5 * i + 3) % VOCAB for i in range(70)]
    b = [(11 * i + 7) % VOCAB for i in range(37)]
    (ref_a, choice_a), (ref_b, _) = _plain(stored, a), _plain(stored, b)
    assert len(set(choice_a.tolist())) == EXPERTS          # every expert gets tokens
    got = {"a": {}, "b": {}}
    # portions of changing size, down to two tokens, then tokens one by one, mixed
    plan = [[("a", 0, 33)], [("b", 0, 2), ("a", 33, 35)], [("b", 2, 30), ("a", 35, 36)],
            [("a", 36, 64), ("b", 30, 31)]]
    plan += [[("a", 64 + i, 65 + i), ("b", 31 + i, 32 + i)] for i in range(6)]
    for step in plan:
        entries = [StepEntry(r, (a if r == "a" else b)[lo:hi], want=list(range(hi - lo)))
                   for r, lo, hi in step]
        res = rn.step(entries)
        for (r, w_), row in zip(res.rows, res.logits.double().cpu()):
            lo = [lo for rr, lo, hi in step if rr == r][0]
            got[r][lo + w_] = row
    for r, ref in (("a", ref_a), ("b", ref_b)):
        assert sorted(got[r]) == list(range(len(got[r])))
        err = max(float((got[r][i] - ref[i]).abs().max()) for i in got[r])
        assert err < 5e-5, (r, err)
    # pages are used again by a third request, with the same result
    rn.close("a")
    res = rn.step([StepEntry("c", a[:40], want=[39])])
    assert (res.logits[0].double().cpu() - ref_a[39]).abs().max() < 5e-5
    rn.manager.check()
