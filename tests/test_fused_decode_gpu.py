"""The whole-step decode kernel (csrc/decode_persistent.cu) against the plain implementation
and against the layer-by-layer path it replaces.

It serves heads of 64, which neither tiny configuration of the other tests has, so two more are
made here that again differ in every size and option: widths 128 / 192 (2 / 3 heads), inner
widths 320 (not 4x) / 768, three / two layers, vocabularies 1000 / 517 (not a multiple of the
16-feature tile), eps 1e-6 / 1e-5, erf / tanh GELU, inverse-layer scaling on / off.  Steps of
single decoded tokens take the kernel; prompts and mixed steps run layer by layer, so every
test below also crosses between the two paths on the same cache pages."""

import json

import pytest
import torch

import plain_gpt2
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.weights import read_safetensors, write_model_dir

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_BASE = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", tie_word_embeddings=True)
CONFIGS = {
    "c": (dict(_BASE, n_layer=3, n_embd=128, n_head=2, n_inner=320, vocab_size=1000,
               n_positions=256, layer_norm_epsilon=1e-6, activation_function="gelu",
               scale_attn_by_inverse_layer_idx=True), 1),
    "d": (dict(_BASE, n_layer=2, n_embd=192, n_head=3, n_inner=None, vocab_size=517,
               n_positions=160, layer_norm_epsilon=1e-5, activation_function="gelu_new",
               scale_attn_by_inverse_layer_idx=False), 2),
}
TOL = 2.5e-2          # bfloat16 between kernels: the tolerance of the other bfloat16 tests


@pytest.fixture(scope="module", params=list(CONFIGS))
def heads64(request, tmp_path_factory):
    cfg, seed = CONFIGS[request.param]
    d = tmp_path_factory.mktemp("heads64_" + request.param)
    write_model_dir(d, cfg, seed, "float32")
    raw = read_safetensors(d / "model.safetensors")
    cfg = json.loads((d / "config.json").read_text())
    plain = plain_gpt2.prepare_weights(raw, round_to=torch.bfloat16)
    return str(d), cfg, plain


def _runner(d, graphs, pages=72, requests=16):
    model, _ = load_model(d, "bfloat16", DEV)
    rn = Runner(model, num_pages=pages, page_size=16, max_requests=requests,
                dtype=torch.bfloat16, device=DEV, cuda_graphs=graphs, fused_decode=True)
    assert rn.fused is not None             # the model has the shape the kernel serves
    return rn


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
@pytest.mark.parametrize("lens", [(5, 17, 70), (1,), (64, 63, 65, 128, 127, 16, 15, 100, 33, 2, 90),
                                  (150,), (40,) * 16],
                         ids=["three", "one_from_the_start", "eleven_edges", "one_long", "sixteen"])
def test_decode_steps_in_one_kernel_agree_with_the_plain_model(heads64, lens, graphs):
    d, cfg, plain = heads64
    n_pos = cfg["n_positions"]
    steps = 8
    seqs = [_tokens(cfg, min(n + steps, n_pos), 50 + i) for i, n in enumerate(lens)]
    lens = [min(n, len(s) - 1) for n, s in zip(lens, seqs)]
    rn = _runner(d, graphs)
    ids = [f"r{i}" for i in range(len(lens))]
    for r, s, n in zip(ids, seqs, lens):                      # prompts: layer by layer
        rn.step([StepEntry(r, s[:n])])
    launches = []
    for k in range(steps):
        entries = [StepEntry(r, [s[n + k]], want=[0]) for r, s, n in zip(ids, seqs, lens)
                   if n + k < len(s)]
        if not entries:
            break
        before = rn.kernel_launches
        res = rn.step(entries, sample=True)
        launches.append(rn.kernel_launches - before)
        got, toks = res.logits.double().cpu(), res.tokens_host()
        for row, (e, tok) in enumerate(zip(entries, toks)):
            i = ids.index(e.req_id)
            want = plain_gpt2.forward(cfg, plain, seqs[i][:lens[i] + k + 1])[-1]
            assert (got[row] - want).abs().max() < TOL, (e.req_id, k)
            assert tok == int(torch.argmax(res.logits[row]))   # lowest index on ties
    assert min(launches) == 1                                  # the step was one launch
    rn.manager.check()


def test_the_kernel_and_the_layers_agree_and_share_the_cache(heads64):
    """The same requests decoded with the kernel on and off: logits agree to rounding, the pages
    each path appended are read by the other (the paths alternate step by step)."""
    d, cfg, plain = heads64
    lens = (30, 77, 9, 64)
    seqs = [_tokens(cfg, n + 12, 80 + i) for i, n in enumerate(lens)]
    outs = {}
    for mode in ("kernel", "layers", "alternating"):
        rn = _runner(d, graphs=False)
        fused = rn.fused
        for i, (s, n) in enumerate(zip(seqs, lens)):
            rn.step([StepEntry(f"r{i}", s[:n])])
        rows = []
        for k in range(12):
            rn.fused = fused if mode == "kernel" or (mode == "alternating" and k % 2) else None
            res = rn.step([StepEntry(f"r{i}", [s[n + k]], want=[0])
                           for i, (s, n) in enumerate(zip(seqs, lens))])
            rows.append(res.logits.float().cpu().clone())
        outs[mode] = torch.stack(rows)
    assert (outs["kernel"] - outs["layers"]).abs().max() < TOL
    assert (outs["alternating"] - outs["layers"]).abs().max() < TOL
    want = plain_gpt2.forward(cfg, plain, seqs[1][:lens[1] + 12])[-1]
    assert (outs["kernel"][-1, 1].double() - want).abs().max() < TOL


def test_a_far_key_decides_the_output_in_every_slice(heads64):
    """One request alone: its context is cut into slices between CTAs.  One cached key of the
    first layer is scaled up so that its score stands out, at several distances; the kernel
    must follow the layer-by-layer path wherever the key lies (a slice dropped, or merged with
    a wrong weight, would show), and the key must matter."""
    d, cfg, plain = heads64
    n = min(cfg["n_positions"] - 2, 200)
    toks = _tokens(cfg, n + 1, 7)

    def last_logits(far, use_kernel):
        rn = _runner(d, graphs=False)
        rn.step([StepEntry("a", toks[:n])])
        if far is not None:
            page, slot = rn.manager.table("a")[far // 16], far % 16
            rn.storage.pools[0][0, page, 0, 0, slot, :] *= 30.0      # entry 0, keys, head 0
        if not use_kernel:
            rn.fused = None
        return rn.step([StepEntry("a", [toks[n]], want=[0])]).logits[0].float().cpu().clone()

    base = last_logits(None, True)
    want = plain_gpt2.forward(cfg, plain, toks)[-1]
    assert (base.double() - want).abs().max() < TOL
    moved = 0
    for far in (0, 63, 64, 130, n - 1):
        a, b = last_logits(far, True), last_logits(far, False)
        assert (a - b).abs().max() < TOL, far
        moved += int((a - base).abs().max() > 1e-3)
    assert moved >= 3                       # the planted key changed the result


def test_sampling_with_a_temperature_still_goes_through_the_sampler(heads64):
    d, cfg, plain = heads64
    toks = _tokens(cfg, 21, 9)
    rn = _runner(d, graphs=True)
    rn.step([StepEntry("a", toks[:20])])
    res = rn.step([StepEntry("a", [toks[20]], want=[0], temperature=0.9, top_k=50, seed=11)],
                  sample=True)
    row = res.logits[0].double().cpu()
    u = plain_gpt2.uniform_for(11, 21)
    assert res.tokens_host()[0] == plain_gpt2.sample_token(row, 0.9, 50, u)


def test_models_the_kernel_does_not_serve_run_layer_by_layer(tiny_models):
    model, _ = load_model(tiny_models["tiny_a"].dir, "bfloat16", DEV)      # heads of 16
    rn = Runner(model, num_pages=8, page_size=16, max_requests=2, dtype=torch.bfloat16, device=DEV,
                fused_decode=True)
    assert rn.fused is None
