"""Each part of a layer alone on the GPU, built through the registries from a PartSpec with
sizes of its own, against the plain formulas: position table + embedding, LayerNorm, causal
attention (with grouped heads and with a window), dense feed-forward, head; and the block
arrangement.  Also: a schedule that runs a layer twice and one whose second call reads the
first call's cache."""

import pytest
import torch

import plain_gpt2
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import (LayerCall, LayerSpec, Model, ModelSpec, PartSpec,
                                     build_part)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _model(width=48, heads=3, kv_heads=None, head_dim=16, inner=80, vocab=61, positions=40,
           layers=1, schedule=None, window=0, act="gelu_erf", eps=1e-4, scale=0.21):
    kv = kv_heads or heads
    qkv_w = (heads + 2 * kv) * head_dim
    specs = []
    for i in range(layers):
        p = f"L{i}."
        specs.append(LayerSpec(
            norm1=PartSpec("layernorm", dict(width=width, eps=eps, weight=p + "n1.w", bias=p + "n1.b")),
            mixer=PartSpec("causal_attention", dict(
                width=width, n_heads=heads, n_kv_heads=kv, head_dim=head_dim, scale=scale,
                window=window, qkv_weight=p + "qkv.w", qkv_bias=p + "qkv.b",
                out_weight=p + "o.w", out_bias=None, stored_in_out=False)),
            norm2=PartSpec("layernorm", dict(width=width, eps=eps, weight=p + "n2.w", bias=p + "n2.b")),
            feed_forward=PartSpec("dense", dict(
                width=width, inner=inner, activation=act, in_weight=p + "fc.w", in_bias=p + "fc.b",
                out_weight=p + "pr.w", out_bias=p + "pr.b", stored_in_out=False))))
    spec = ModelSpec(
        name="parts-test", vocab_size=vocab, width=width, max_positions=positions,
        embedding=PartSpec("token_table", dict(vocab_size=vocab, width=width, table="emb")),
        position=PartSpec("learned", dict(max_positions=positions, width=width, table="pos")),
        layers=tuple(specs),
        schedule=tuple(schedule) if schedule else tuple(LayerCall(i) for i in range(layers)),
        final_norm=PartSpec("layernorm", dict(width=width, eps=eps, weight="nf.w", bias="nf.b")),
        head=PartSpec("linear", dict(vocab_size=vocab, width=width, weight="head")))
    model = Model(spec)
    g = torch.Generator().manual_seed(7)
    stored = {}
    for name, req in model.tensor_requests().items():
        # matrices scaled by their fan-in so that activations and scores stay of order one
        # (huge scores would make the softmax a step function, which no 8-bit mantissa follows)
        t = torch.randn(req.shape, generator=g) * (0.8 / req.shape[-1] ** 0.5
                                                   if len(req.shape) == 2 else 0.2)
        if name.endswith(".w") and len(req.shape) == 1:
            t = t + 1.0
        stored[name] = t
    return model, stored, dict(width=width, heads=heads, kv=kv, head_dim=head_dim, inner=inner,
                               vocab=vocab, window=window, act=act, eps=eps, scale=scale)


def _plain_forward(stored, geo, tokens, calls):
    """The same model from the plain part functions, float64; `calls` is the schedule as
    (layer, reads_cache_of) pairs: a reader reuses the keys/values its source call made."""
    w = {k: v.double() for k, v in stored.items()}
    H, KV, D = geo["heads"], geo["kv"], geo["head_dim"]
    act = plain_gpt2.gelu_erf if geo["act"] == "gelu_erf" else plain_gpt2.gelu_new
    scale = float(torch.tensor(geo["scale"], dtype=torch.float64).float())
    ids = torch.tensor(tokens)
    x = plain_gpt2.embed(w["emb"], w["pos"], ids, torch.arange(len(tokens)))
    kv_of = {}
    for idx, (layer, source) in enumerate(calls):
        p = f"L{layer}."
        h = plain_gpt2.layer_norm(x, w[p + "n1.w"], w[p + "n1.b"], geo["eps"])
        qkv = h @ w[p + "qkv.w"].T + w[p + "qkv.b"]
        q = plain_gpt2.split_heads(qkv[:, :H * D], H)
        if source is None:
            k = plain_gpt2.split_heads(qkv[:, H * D:(H + KV) * D], KV)
            v = plain_gpt2.split_heads(qkv[:, (H + KV) * D:], KV)
            kv_of[idx] = (k, v)
        else:
            k, v = kv_of[source]
        rep = H // KV
        ctx = plain_gpt2.causal_attention(q, k.repeat_interleave(rep, 0), v.repeat_interleave(rep, 0),
                                          scale, window=geo["window"] or None)
        x = x + ctx @ w[p + "o.w"].T
        h = plain_gpt2.layer_norm(x, w[p + "n2.w"], w[p + "n2.b"], geo["eps"])
        x = x + act(h @ w[p + "fc.w"].T + w[p + "fc.b"]) @ w[p + "pr.w"].T + w[p + "pr.b"]
    return plain_gpt2.layer_norm(x, w["nf.w"], w["nf.b"], geo["eps"]) @ w["head"].T


def _run(model, stored, tokens, dtype, cuts=None):
    model.bind(stored, dtype, DEV)
    rn = Runner(model, num_pages=8, page_size=16, max_requests=2, dtype=dtype, device=DEV)
    cuts = cuts or [len(tokens)]
    out, at = [], 0
    for n in cuts:
        res = rn.step([StepEntry("a", tokens[at:at + n], want=list(range(n)))])
        out.append(res.logits.double().cpu())
        at += n
    return torch.cat(out)


CASES = {
    "plain": dict(),
    "grouped_heads": dict(heads=6, kv_heads=2, width=96),
    "window": dict(window=5),
    "big_head": dict(heads=1, head_dim=128, width=128, inner=144),
    "gelu_tanh_two_layers": dict(act="gelu_tanh", layers=2),
}


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_of_parts_equals_the_plain_formulas(case, dtype):
    model, stored, geo = _model(**CASES[case])
    if dtype == torch.bfloat16:
        stored = {k: (v.bfloat16().float() if v.dim() == 2 else v) for k, v in stored.items()}
    tokens = [(7 * i + 3) % geo["vocab"] for i in range(33)]
    calls = [(c.layer, None) for c in model.schedule]
    ref = _plain_forward(stored, geo, tokens, calls)
    # the tolerance of the tiny-model tests (2.5e-2 for logits of order one), per unit of scale
    tol = 5e-5 if dtype == torch.float32 else 2.5e-2 * max(1.0, float(ref.abs().max()))
    whole = _run(model, stored, tokens, dtype)
    assert (whole - ref).abs().max() < tol
    cut = _run(model, stored, tokens, dtype, cuts=[20, 2, 1, 9, 1])
    assert (cut - ref).abs().max() < tol


def test_schedule_may_run_a_layer_twice():
    model, stored, geo = _model(layers=2, schedule=[LayerCall(0), LayerCall(1), LayerCall(0)])
    assert [c.cache for c in model.schedule] == [0, 1, 2]         # three cache entries, two layers
    assert len(model.cache_groups) == 1 and len(model.cache_groups[0].entries) == 3
    tokens = list(range(25))
    ref = _plain_forward(stored, geo, tokens, [(0, None), (1, None), (0, None)])
    got = _run(model, stored, tokens, torch.float32, cuts=[11, 14])
    assert (got - ref).abs().max() < 5e-5


def test_a_layer_may_read_another_layers_cache():
    sched = [LayerCall(0, cache=0), LayerCall(1, cache=0, writes_cache=False)]
    model, stored, geo = _model(layers=2, schedule=sched)
    assert len(model.cache_groups[0].entries) == 1                # one entry serves both calls
    tokens = list(range(30))
    ref = _plain_forward(stored, geo, tokens, [(0, None), (1, 0)])
    got = _run(model, stored, tokens, torch.float32, cuts=[17, 1, 12])
    assert (got - ref).abs().max() < 5e-5
    with pytest.raises(ValueError, match="before any call wrote"):
        _model(layers=2, schedule=[LayerCall(0, cache=0, writes_cache=False), LayerCall(1, cache=0)])


def test_layers_with_different_needs_get_page_groups_of_their_own():
    """One model, two kinds of mixer: a layer that keeps every key and a layer with a window."""
    m1, s1, geo = _model(layers=1)
    full = m1.spec.layers[0]
    win = LayerSpec(norm1=full.norm1, norm2=full.norm2, feed_forward=full.feed_forward,
                    mixer=PartSpec("causal_attention", dict(full.mixer.params, window=6)))
    import dataclasses
    spec = dataclasses.replace(m1.spec, layers=(full, win), schedule=(LayerCall(0), LayerCall(1)))
    model = Model(spec)
    assert sorted(g.window for g in model.cache_groups) == [0, 6]
    tokens = [(5 * i + 1) % geo["vocab"] for i in range(36)]
    model.bind(s1, torch.float32, DEV)
    rn = Runner(model, num_pages=4, page_size=16, max_requests=2, dtype=torch.float32, device=DEV)
    got = torch.cat([rn.step([StepEntry("a", tokens[a:b], want=list(range(b - a)))]).logits.cpu()
                     for a, b in ((0, 20), (20, 21), (21, 36))]).double()
    # plain: layer 0 without a window, the same weights again with a window of 6
    w = {k: v.double() for k, v in s1.items()}
    geo_w = dict(geo, window=6)
    x_ref = _two_kinds_plain(w, geo, geo_w, tokens)
    assert (got - x_ref).abs().max() < 5e-5
    # the windowed group has given pages back, the full group has not
    gi_win = [i for i, g in enumerate(model.cache_groups) if g.window == 6][0]
    assert rn.manager.table("a", gi_win)[0] == -1 and rn.manager.table("a", 1 - gi_win)[0] >= 0
    rn.manager.check()


def _two_kinds_plain(w, geo, geo_w, tokens):
    H, D = geo["heads"], geo["head_dim"]
    scale = float(torch.tensor(geo["scale"], dtype=torch.float64).float())
    x = plain_gpt2.embed(w["emb"], w["pos"], torch.tensor(tokens), torch.arange(len(tokens)))
    for window in (None, 6):
        p = "L0."
        h = plain_gpt2.layer_norm(x, w[p + "n1.w"], w[p + "n1.b"], geo["eps"])
        qkv = h @ w[p + "qkv.w"].T + w[p + "qkv.b"]
        q, k, v = (plain_gpt2.split_heads(qkv[:, i * H * D:(i + 1) * H * D], H) for i in range(3))
        x = x + plain_gpt2.causal_attention(q, k, v, scale, window=window) @ w[p + "o.w"].T
        h = plain_gpt2.layer_norm(x, w[p + "n2.w"], w[p + "n2.b"], geo["eps"])
        x = x + plain_gpt2.gelu_erf(h @ w[p + "fc.w"].T + w[p + "fc.b"]) @ w[p + "pr.w"].T + w[p + "pr.b"]
    return plain_gpt2.layer_norm(x, w["nf.w"], w["nf.b"], geo["eps"]) @ w["head"].T


def test_parts_refuse_bad_parameters():
    with pytest.raises(ValueError, match="multiple of 16"):
        build_part("mixer", PartSpec("causal_attention", dict(
            width=20, n_heads=2, head_dim=10, scale=1.0, qkv_weight="a", qkv_bias=None,
            out_weight="b", out_bias=None)))
    with pytest.raises(ValueError, match="multiple of n_kv_heads"):
        build_part("mixer", PartSpec("causal_attention", dict(
            width=48, n_heads=3, n_kv_heads=2, head_dim=16, scale=1.0, qkv_weight="a",
            qkv_bias=None, out_weight="b", out_bias=None)))
    with pytest.raises(ValueError, match="unknown activation"):
        build_part("feed_forward", PartSpec("dense", dict(
            width=8, inner=8, activation="swish", in_weight="a", in_bias=None, out_weight="b",
            out_bias=None)))
    with pytest.raises(ValueError, match="unknown mixer kind"):
        build_part("mixer", PartSpec("no_such_mixer", {}))
