"""The plain implementation itself (no GPU): anchored once on the reference's own CPU
engine, and checked for the properties the other tests lean on."""

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gpt2
from hetero_serve_b200.weights import random_weights

GOLDEN = Path(__file__).parent / "golden" / "tiny_a_reference.npz"


@pytest.fixture(scope="module")
def golden():
    g = np.load(GOLDEN)
    cfg = json.loads(bytes(g["config"]).decode())
    _, tensors = random_weights(cfg, int(g["seed"]))
    return g, cfg, plain_gpt2.prepare_weights(tensors)


def test_matches_the_reference_engine_on_a_whole_prompt(golden):
    g, cfg, w = golden
    logits = plain_gpt2.forward(cfg, w, g["prompt"].tolist())
    # the reference computes in float32 with numpy's summation order: rounding differs
    assert np.abs(logits[-1].numpy() - g["whole_last"]).max() < 2e-6
    assert np.abs(logits[-1].numpy() - g["chunked_last"]).max() < 2e-6


def test_matches_the_reference_engine_while_decoding(golden):
    g, cfg, w = golden
    toks = g["prompt"].tolist() + g["greedy_tokens"].tolist()[:-1]
    logits = plain_gpt2.forward(cfg, w, toks)
    n = len(g["prompt"])
    for i in range(g["decode_logits"].shape[0]):
        assert np.abs(logits[n + i].numpy() - g["decode_logits"][i]).max() < 2e-6
    assert plain_gpt2.greedy_generate(cfg, w, g["prompt"].tolist(), 7) == g["greedy_tokens"].tolist()


def test_causality_a_later_token_changes_nothing_before_it(tiny):
    toks = tiny.tokens(20, 3)
    a = plain_gpt2.forward(tiny.config, tiny.plain, toks)
    toks2 = toks[:12] + [(toks[12] + 1) % tiny.config["vocab_size"]] + toks[13:]
    b = plain_gpt2.forward(tiny.config, tiny.plain, toks2)
    assert torch.equal(a[:12], b[:12]) and not torch.allclose(a[12:], b[12:])


def test_parts_against_torch():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    g, b = torch.randn(12, dtype=torch.float64), torch.randn(12, dtype=torch.float64)
    assert torch.allclose(plain_gpt2.layer_norm(x, g, b, 1e-5),
                          torch.nn.functional.layer_norm(x, (12,), g, b, 1e-5))
    assert torch.allclose(plain_gpt2.gelu_new(x), torch.nn.functional.gelu(x, approximate="tanh"))
    assert torch.allclose(plain_gpt2.gelu_erf(x), torch.nn.functional.gelu(x))
    assert torch.allclose(plain_gpt2.softmax(x), torch.softmax(x, -1))
    q, k, v = (torch.randn(2, 6, 4, dtype=torch.float64) for _ in range(3))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.3)
    out = plain_gpt2.causal_attention(q, k, v, 0.3)
    assert torch.allclose(out, ref.permute(1, 0, 2).reshape(6, 8))
    # a window of 1 sees only the token itself
    w1 = plain_gpt2.causal_attention(q, k, v, 0.3, window=1)
    assert torch.allclose(w1, v.permute(1, 0, 2).reshape(6, 8))


def test_scale_options():
    assert plain_gpt2.attention_scale(64, 0) == 0.125
    assert abs(plain_gpt2.attention_scale(32, 2, True, True) - 1 / math.sqrt(32) / 3) < 1e-8
    assert plain_gpt2.attention_scale(32, 1, False, True) == 0.5


def test_inverse_layer_scaling_equals_folding_it_into_the_query(tiny_models):
    """1/(layer+1) on the scores is the same as scaling that layer's query weights."""
    m = tiny_models["tiny_b"]
    toks = m.tokens(15, 5)
    a = plain_gpt2.forward(m.config, m.plain, toks)
    cfg = dict(m.config, scale_attn_by_inverse_layer_idx=False)
    w = dict(m.plain)
    E = cfg["n_embd"]
    for i in range(cfg["n_layer"]):
        cw = w[f"h.{i}.attn.c_attn.weight"].clone(); cb = w[f"h.{i}.attn.c_attn.bias"].clone()
        cw[:, :E] /= (i + 1); cb[:E] /= (i + 1)
        w[f"h.{i}.attn.c_attn.weight"], w[f"h.{i}.attn.c_attn.bias"] = cw, cb
    b = plain_gpt2.forward(cfg, w, toks)
    assert (a - b).abs().max() < 1e-7


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    assert plain_gpt2.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert plain_gpt2.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == \
        [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    from hetero_serve_b200.sampling import uniform_for_position
    for seed, pos in ((0, 0), (1, 5), (2 ** 40 + 3, 1000)):
        assert uniform_for_position(seed, pos) == plain_gpt2.uniform_for(seed, pos)
        assert 0.0 <= plain_gpt2.uniform_for(seed, pos) < 1.0


def test_sampler_rules():
    lg = torch.tensor([0.0, 3.0, 3.0, -1.0, 2.0])
    assert plain_gpt2.sample_token(lg, 0.0, 0, 0.99) == 1                 # argmax, lowest index
    assert plain_gpt2.sample_token(lg, 1.0, 1, 0.99) == 1                 # top-1 == argmax
    assert plain_gpt2.sample_token(lg, 1.0, 2, 0.99) == 2                 # ties: lower indices
    assert plain_gpt2.sample_token(lg, 1.0, 2, 0.01) == 1
    assert plain_gpt2.sample_token(lg, 1.0, 0, 0.0) == 0
    counts = [0] * 5
    for i in range(4000):
        counts[plain_gpt2.sample_token(lg, 1.0, 0, (i + 0.5) / 4000)] += 1
    p = torch.softmax(lg.double(), 0)
    assert all(abs(c / 4000 - float(pi)) < 2e-3 for c, pi in zip(counts, p))
