"""The engine at the real widths of GPT-2 small, medium, large and XL (a few layers of each,
random weights): widths 768 / 1024 / 1280 / 1600, 12 / 16 / 20 / 25 heads of 64, inner 4x, the real vocabulary
of 50,257 (odd, no power of two).  In 32-bit and in bfloat16, whole prompts against decoding
and portions, compared with the plain implementation on the last positions."""

import json

import pytest
import torch

import plain_gpt2
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.weights import read_safetensors, write_model_dir

pytestmark = pytest.mark.gpu

SIZES = {
    "small": dict(n_layer=2, n_embd=768, n_head=12),
    "medium": dict(n_layer=3, n_embd=1024, n_head=16),
    "large": dict(n_layer=2, n_embd=1280, n_head=20),
    "xl": dict(n_layer=2, n_embd=1600, n_head=25),
}


@pytest.fixture(scope="module", params=list(SIZES))
def real_model(request, tmp_path_factory):
    sz = SIZES[request.param]
    cfg = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", vocab_size=50257,
               n_positions=1024, n_inner=None, layer_norm_epsilon=1e-5,
               activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, **sz)
    d = tmp_path_factory.mktemp("real_" + request.param)
    write_model_dir(d, cfg, 3, "float32")
    raw = read_safetensors(d / "model.safetensors")
    return request.param, str(d), json.loads((d / "config.json").read_text()), raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_every_cut_agrees_with_the_plain_model(real_model, dtype):
    name, d, cfg, raw = real_model
    g = torch.Generator().manual_seed(11)
    a = torch.randint(0, 50257, (150,), generator=g).tolist()
    b = torch.randint(0, 50257, (41,), generator=g).tolist()
    w = plain_gpt2.prepare_weights(raw, dtype=torch.float32,
                                   round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    # float32 plain arithmetic is enough here: the comparison is at 1e-3 of a logit
    ref_a = plain_gpt2.forward(cfg, w, a, dtype=torch.float32)
    ref_b = plain_gpt2.forward(cfg, w, b, dtype=torch.float32)
    model, _ = load_model(d, dtype, "cuda:0")
    rn = Runner(model, num_pages=24, page_size=16, max_requests=4, dtype=model.dtype,
                device="cuda:0", cuda_graphs=(dtype == "bfloat16"))
    tol = 2e-3 if dtype == "float32" else 6e-2
    got = {}
    # a whole; b as a portion beside a's decoded tokens; then both decode together
    # (the logits of a step live in a buffer the next step reuses: copy what is kept)
    r = rn.step([StepEntry("a", a[:140], want=[0, 139])]).logits.clone()
    got[("a", 0)], got[("a", 139)] = r[0], r[1]
    r = rn.step([StepEntry("a", a[140:141], want=[0]),
                 StepEntry("b", b[:30], want=[29])]).logits.clone()
    got[("a", 140)], got[("b", 29)] = r[0], r[1]
    r = rn.step([StepEntry("b", b[30:33], want=[2]),
                 StepEntry("a", a[141:149], want=[7])]).logits.clone()
    got[("b", 32)], got[("a", 148)] = r[0], r[1]
    for i in range(33, 41):
        r = rn.step([StepEntry("a", a[149:150], want=[0])] * (i == 33) +
                    [StepEntry("b", b[i:i + 1], want=[0])]).logits.clone()
        if i == 33:
            got[("a", 149)] = r[0]
        got[("b", i)] = r[-1]
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = (ref_a if rid == "a" else ref_b)[pos]
        assert torch.isfinite(row).all()
        worst = max(worst, float((row.float().cpu() - ref).abs().max()))
    assert worst < tol, (name, dtype, worst)
    rn.manager.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_depth_medium_long_prompt_then_decoding(tmp_path_factory, dtype):
    """GPT-2 medium at its full depth of 24 layers: one prompt of 1,016 tokens in one step,
    then 8 tokens decoded one by one up to the end of the position table, against the plain
    model in float64 on the CPU (first, middle and last place of the prompt, every decoded
    place).  Depth is what the few-layer tests above leave out: 24 layers of accumulated
    rounding on a residual stream that grows."""
    cfg = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", vocab_size=50257,
               n_positions=1024, n_inner=None, layer_norm_epsilon=1e-5,
               activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, n_layer=24, n_embd=1024, n_head=16)
    d = tmp_path_factory.mktemp("medium_full_" + dtype)
    write_model_dir(d, cfg, 5, "float32")
    raw = read_safetensors(d / "model.safetensors")
    cfg = json.loads((d / "config.json").read_text())
    g = torch.Generator().manual_seed(21)
    toks = torch.randint(0, 50257, (1024,), generator=g).tolist()
    w = plain_gpt2.prepare_weights(raw, dtype=torch.float64,
                                   round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    places = [0, 511, 1015] + list(range(1016, 1024))
    ref = plain_gpt2.forward(cfg, w, toks, dtype=torch.float64, rows=places)
    del w
    model, _ = load_model(str(d), dtype, "cuda:0")
    rn = Runner(model, num_pages=66, page_size=16, max_requests=2, dtype=model.dtype,
                device="cuda:0", cuda_graphs=(dtype == "bfloat16"))
    got = [rn.step([StepEntry("a", toks[:1016], want=[0, 511, 1015])]).logits.double().cpu()]
    for p in range(1016, 1024):
        got.append(rn.step([StepEntry("a", [toks[p]], want=[0])]).logits.double().cpu())
    got = torch.cat(got)
    err = (got - ref).abs().max(dim=1).values
    # float32: 24 layers of float32 sums against float64; bfloat16: activations rounded to 8
    # bits between kernels, 24 layers deep
    tol = 5e-4 if dtype == "float32" else 1e-1
    assert float(err.max()) < tol, [round(float(e), 6) for e in err]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_table_of_4096_positions(tmp_path, dtype):
    """A configuration with a longer table than the family's 1,024: a prompt of 2,900 tokens
    in two portions (prefill tiles that look back over thousands of keys, a portion starting
    mid-context), then single tokens whose context is cut into slices between CTAs (beyond
    2,048 keys), beside a short request.  Compared with the plain model on the rows kept."""
    cfg = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", vocab_size=331,
               n_positions=4096, n_layer=2, n_embd=128, n_head=2, n_inner=None,
               layer_norm_epsilon=1e-5, activation_function="gelu_new",
               scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True)
    write_model_dir(tmp_path, cfg, 5, "float32")
    raw = read_safetensors(tmp_path / "model.safetensors")
    cfg = json.loads((tmp_path / "config.json").read_text())
    g = torch.Generator().manual_seed(21)
    a = torch.randint(0, 331, (2906,), generator=g).tolist()
    b = torch.randint(0, 331, (40,), generator=g).tolist()
    w = plain_gpt2.prepare_weights(raw, dtype=torch.float32,
                                   round_to=torch.bfloat16 if dtype == "bfloat16" else None)
    ref_a = plain_gpt2.forward(cfg, w, a, dtype=torch.float32, rows=[1499, 2899, 2900, 2905])
    ref_b = plain_gpt2.forward(cfg, w, b, dtype=torch.float32, rows=[33, 39])
    model, _ = load_model(str(tmp_path), dtype, "cuda:0")
    rn = Runner(model, num_pages=200, page_size=16, max_requests=4, dtype=model.dtype,
                device="cuda:0", cuda_graphs=(dtype == "bfloat16"))
    got = []
    got.append(rn.step([StepEntry("a", a[:1500], want=[1499])]).logits[0].clone())
    r = rn.step([StepEntry("a", a[1500:2900], want=[1399]),
                 StepEntry("b", b[:34], want=[33])]).logits.clone()
    got.append(r[0]); keep_b = [r[1]]
    for i in range(6):
        r = rn.step([StepEntry("a", a[2900 + i:2901 + i], want=[0]),
                     StepEntry("b", b[34 + i:35 + i], want=[0])]).logits.clone()
        if i in (0, 5):
            got.append(r[0])
        if i == 5:
            keep_b.append(r[1])
    tol = 2e-3 if dtype == "float32" else 6e-2
    for row, ref in zip(got + keep_b, list(ref_a) + list(ref_b)):
        assert torch.isfinite(row).all()
        assert float((row.float().cpu() - ref).abs().max()) < tol
    rn.manager.check()
