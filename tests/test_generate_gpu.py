"""Generation through the Python entry point on the GPU: greedy and sampled tokens against
the plain implementation, prefix reuse, preemption, CUDA graphs, the command line."""

import json
import subprocess
import sys

import pytest
import torch

import plain_gpt2
from conftest import ROOT, TINY
from hetero_serve_b200 import EngineConfig, LLMEngine, Request
from hetero_serve_b200.weights import random_weights, read_safetensors, write_safetensors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lively(tmp_path_factory):
    """Random weights make a tied-head GPT-2 repeat its last token, which would hide most
    faults of generation.  Here the blocks' output projections are scaled up so that what
    the layers compute decides the next token; outputs then wander through the vocabulary."""
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp("lively_" + name)
        _, w = random_weights(cfg, seed)
        for k in w:
            if k.endswith("c_proj.weight"):
                w[k] = w[k] * 60.0
        (d / "config.json").write_text(json.dumps(cfg))
        write_safetensors(d / "model.safetensors", w)
        out[name] = (str(d), cfg, plain_gpt2.prepare_weights(read_safetensors(d / "model.safetensors")))
    return out


def _prompts(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]


def _check_greedy_path(cfg, w, prompt, out, margin):
    """Every generated token is the plain argmax of its position, up to `margin` in logit."""
    logits = plain_gpt2.forward(cfg, w, prompt + out[:-1])
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert float(row.max() - row[tok]) <= margin, (i, tok, int(row.argmax()))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_equals_the_plain_model(lively, name):
    d, cfg, w = lively[name]
    lens = (5, 17, 33) if name == "tiny_a" else (1, 16, 31, 70)
    prompts = _prompts(cfg, lens, 11)
    want = [plain_gpt2.greedy_generate(cfg, w, p, 16) for p in prompts]
    assert len({t for o in want for t in o}) > 10          # the outputs are not one token
    for graphs in (False, True):
        eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=32, max_batch=4,
                                        max_prefill_tokens=24, cuda_graphs=graphs))
        got = eng.generate(prompts, max_new_tokens=16, stop_at_eos=False)
        assert got == want, graphs
        eng.runner.manager.check()
        assert eng.runner.manager.free_slots() == eng.config.live_requests


@pytest.mark.parametrize("policy", ["prefill_first", "mixed"])
def test_bfloat16_generation_follows_the_plain_argmax(lively, policy):
    d, cfg, _ = lively["tiny_b"]
    wb = plain_gpt2.prepare_weights(read_safetensors(d + "/model.safetensors"),
                                    round_to=torch.bfloat16)
    prompts = _prompts(cfg, (1, 16, 31, 70), 12)
    eng = LLMEngine(d, EngineConfig(dtype="bfloat16", num_blocks=32, max_batch=4,
                                    max_prefill_tokens=24, policy=policy))
    got = eng.generate(prompts, max_new_tokens=12, stop_at_eos=False)
    for p, o in zip(prompts, got):
        assert len(o) == 12
        _check_greedy_path(cfg, wb, p, o, margin=0.15)


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_greedy_rows_are_chosen_by_the_head_kernel_itself(lively, graphs):
    """A bfloat16 step whose rows all take the argmax has no sampling launch: the few-row head
    picks while it streams the table.  Its tokens are the argmax of the logits it returns
    (lowest index on ties), a temperature in the batch brings the sampler back, and a prompt's
    last row is chosen the same way."""
    from hetero_serve_b200.engine.loading import load_model
    from hetero_serve_b200.engine.step import Runner, StepEntry
    d, cfg, _ = lively["tiny_b"]
    model, _ = load_model(d, "bfloat16", "cuda:0")
    rn = Runner(model, num_pages=16, page_size=16, max_requests=4, dtype=torch.bfloat16,
                device="cuda:0", cuda_graphs=graphs)
    prompts = _prompts(cfg, (9, 20, 5), 77)
    res = rn.step([StepEntry(f"r{i}", p, want=[len(p) - 1]) for i, p in enumerate(prompts)],
                  sample=True)
    assert res.tokens_host() == [int(torch.argmax(r)) for r in res.logits]
    counts = {}
    for n, temp in enumerate((0.0, 0.0, 0.7, 0.7, 0.0, 0.0, 0.7, 0.0)):
        before = rn.kernel_launches
        res = rn.step([StepEntry(f"r{i}", [3 + i], want=[0], temperature=temp if i == 1 else 0.0,
                                 seed=5) for i in range(3)], sample=True)
        if n >= 4:      # the first steps of a kind may run twice (once eagerly, once captured;
                        # a captured step exists once per metadata block, and the blocks alternate)
            counts.setdefault(temp, []).append(rn.kernel_launches - before)
        toks = res.tokens_host()
        for i in (0, 2):
            assert toks[i] == int(torch.argmax(res.logits[i]))
    assert len(set(counts[0.0])) == 1
    assert counts[0.7][0] == counts[0.0][0] + 1              # the sampler is a launch of its own
    rn.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_shape_that_keeps_coming_back_alternates_between_two_metadata_blocks(lively, dtype):
    """With CUDA graphs a shape used often enough uploads its metadata on a side stream into
    one of two device blocks, with a graph for each.  Twenty decode steps of three requests
    (the threshold lowered to two uses) give the logits and tokens of a runner without
    graphs, step by step; a prompt in between, and a request that ends, change the shape and
    come back to it."""
    from hetero_serve_b200.engine.loading import load_model
    from hetero_serve_b200.engine.step import Runner, StepEntry
    d, cfg, _ = lively["tiny_a"]
    prompts = _prompts(cfg, (9, 20, 5, 12), 31)
    outs = []
    for graphs in (False, True):
        model, _ = load_model(d, dtype, "cuda:0")
        rn = Runner(model, num_pages=24, page_size=16, max_requests=4, dtype=model.dtype,
                    device="cuda:0", cuda_graphs=graphs)
        rn.hot_shape_uses = 2
        live = ["r0", "r1", "r2"]
        last = {}
        for i, r in enumerate(live):
            res = rn.step([StepEntry(r, prompts[i], want=[len(prompts[i]) - 1])], sample=True)
            last[r] = res.tokens_host()[0]
        seen = []
        for n in range(20):
            if n == 7:                                   # another shape in between
                res = rn.step([StepEntry("r3", prompts[3], want=[len(prompts[3]) - 1])], sample=True)
                last["r3"] = res.tokens_host()[0]
            if n == 12:
                rn.close("r1")
                live = ["r0", "r2", "r3"]
            res = rn.step([StepEntry(r, [last[r]], want=[0]) for r in live], sample=True)
            toks = res.tokens_host()
            seen.append((res.logits.float().cpu().clone(), list(toks)))
            for r, t in zip(live, toks):
                last[r] = t
        if graphs:
            assert sum(1 for k in rn._graphs if k[-1] == 1) >= 1      # the second block was used
        rn.check_status()
        outs.append(seen)
    for (la, ta), (lb, tb) in zip(*outs):
        assert ta == tb
        assert torch.equal(la, lb)


def test_temperature_and_top_k_sampling_match_the_plain_sampler(lively):
    d, cfg, w = lively["tiny_b"]
    prompts = _prompts(cfg, (9, 40), 13)
    eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=32, max_batch=4))
    first = None
    for temp, top_k in ((0.8, 0), (1.3, 20)):
        got = eng.generate(prompts, max_new_tokens=10, temperature=temp, top_k=top_k, seed=5,
                           stop_at_eos=False)
        # a fixed seed reproduces, in another batch composition too
        again = eng.generate(prompts[::-1], max_new_tokens=10, temperature=temp, top_k=top_k,
                             seed=5, stop_at_eos=False)
        assert eng.generate(prompts, max_new_tokens=10, temperature=temp, top_k=top_k, seed=5,
                            stop_at_eos=False) == got
        assert len(again) == len(got)
        first = first or got
        for i, (p, o) in enumerate(zip(prompts, got)):
            ctx = list(p)
            for tok in o:
                row = plain_gpt2.forward(cfg, w, ctx)[-1]
                u = plain_gpt2.uniform_for(5 + i, len(ctx))
                assert tok == plain_gpt2.sample_token(row, temp, top_k, u)
                ctx.append(tok)
    # another seed gives other tokens
    b = eng.generate(prompts, max_new_tokens=10, temperature=0.8, seed=6, stop_at_eos=False)
    assert b != first


def test_prefix_hit_skips_prefill_and_changes_no_token(lively):
    d, cfg, w = lively["tiny_b"]
    shared = _prompts(cfg, (16,), 14)[0]
    p2, p4 = shared, shared + _prompts(cfg, (54,), 15)[0]          # 16 and 70 tokens
    eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=32, max_batch=4,
                                    max_prefill_tokens=24))
    r2 = eng.submit(Request(p2, max_new_tokens=8, stop_at_eos=False))
    r4 = eng.submit(Request(p4, max_new_tokens=8, stop_at_eos=False))
    assert r2.cached_prefix_tokens == 0
    assert r4.cached_prefix_tokens == 16 and r4.prefill_tokens_computed == 54
    assert r4.output_ids == plain_gpt2.greedy_generate(cfg, w, p4, 8)
    cold = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=32, prefix_cache=False))
    assert cold.submit(Request(p4, max_new_tokens=8, stop_at_eos=False)).output_ids == r4.output_ids


def test_preemption_recomputes_and_changes_no_token(lively):
    d, cfg, w = lively["tiny_a"]
    prompts = _prompts(cfg, (30, 28, 25), 16)
    want = [plain_gpt2.greedy_generate(cfg, w, p, 30) for p in prompts]
    eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=9, max_batch=4,
                                    max_prefill_tokens=32, prefix_cache=False))
    seqs = [eng.submit_nowait(Request(p, max_new_tokens=30, stop_at_eos=False, temperature=0.0))
            for p in prompts]
    recs = eng.run_until_done()
    assert sum(r.preemptions for r in recs) >= 1
    assert [s.output_ids for s in seqs] == want
    eng.runner.manager.check()


def test_eos_and_context_limit(lively):
    d, cfg, w = lively["tiny_a"]
    p = _prompts(cfg, (20,), 17)[0]
    free = plain_gpt2.greedy_generate(cfg, w, p, 12)
    cfg2 = dict(cfg, eos_token_id=free[4])
    import pathlib, shutil, tempfile
    with tempfile.TemporaryDirectory() as t:
        shutil.copy(d + "/model.safetensors", t)
        pathlib.Path(t, "config.json").write_text(json.dumps(cfg2))
        eng = LLMEngine(t, EngineConfig(dtype="float32", num_blocks=16))
        r = eng.submit(Request(p, max_new_tokens=12))
        first = free.index(free[4])
        assert r.output_ids == free[:first + 1] and r.finish_reason == "eos"
    eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=16, max_ctx=26))
    r = eng.submit(Request(p, max_new_tokens=50, stop_at_eos=False))
    assert len(r.output_ids) == 6 and r.finish_reason == "max_ctx"
    # up to the very end of the position table
    long = _prompts(cfg, (120,), 18)[0]
    eng = LLMEngine(d, EngineConfig(dtype="float32", num_blocks=16))
    r = eng.submit(Request(long, max_new_tokens=50, stop_at_eos=False))
    assert len(long) + len(r.output_ids) == cfg["n_positions"]
    assert r.output_ids == plain_gpt2.greedy_generate(cfg, w, long, 50)[:len(r.output_ids)]


@pytest.mark.parametrize("policy", ["prefill_first", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pipelined_steps_change_no_token(lively, dtype, policy):
    """With ``pipeline`` a decode step is launched before the host has read the token the step
    before it sampled (the step takes it from device memory).  Sampled and greedy requests, an
    end-of-sequence token met on the way, few pages (preemption) and CUDA graphs: every token is
    the one the engine gives when it reads each step's tokens before the next launch."""
    d, cfg, w = lively["tiny_a"]
    prompts = _prompts(cfg, (30, 28, 25, 7, 3), 21)
    free = plain_gpt2.greedy_generate(cfg, w, prompts[0], 30)
    k = next(i for i in range(5, 30) if free[i] not in free[:i])     # first met at place k
    cfg2 = dict(cfg, eos_token_id=free[k])
    import pathlib, shutil, tempfile
    with tempfile.TemporaryDirectory() as t:
        shutil.copy(d + "/model.safetensors", t)
        pathlib.Path(t, "config.json").write_text(json.dumps(cfg2))
        outs = {}
        for pipeline in (False, True, "side streams"):
            eng = LLMEngine(t, EngineConfig(dtype=dtype, num_blocks=10, max_batch=4,
                                            max_prefill_tokens=32, prefix_cache=False,
                                            policy=policy, pipeline=bool(pipeline)))
            if pipeline == "side streams":
                # every shape at once takes the route of shapes that keep coming back: metadata
                # up and tokens down on side streams, two blocks, two graphs
                eng.runner.hot_shape_uses = 0
            seqs = [eng.submit_nowait(Request(p, max_new_tokens=30, temperature=0.9 * (i % 2),
                                              top_k=12 * (i % 2), seed=3 + i,
                                              stop_at_eos=(i != 1)))
                    for i, p in enumerate(prompts)]
            recs = eng.run_until_done()
            outs[pipeline] = [(s.output_ids, s.finish_reason) for s in seqs]
            assert sum(r.preemptions for r in recs) >= 1
            eng.runner.manager.check()
            assert eng.runner.manager.free_slots() == eng.config.live_requests
        assert outs[True] == outs[False]
        assert outs["side streams"] == outs[False]
        if dtype == "float32":
            assert outs[True][0] == (free[:k + 1], "eos")
        assert any(r == "max_new_tokens" for _, r in outs[True])


def test_command_line(lively):
    d, cfg, w = lively["tiny_a"]
    p = _prompts(cfg, (12,), 19)[0]
    res = subprocess.run(
        [sys.executable, "-m", "hetero_serve_b200", "--weights", d, "--dtype", "float32",
         "--num-blocks", "16", "--max-new-tokens", "6", "--no-eos-stop", "--json",
         "--prompt-ids", ",".join(map(str, p))],
        capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.strip().splitlines()]
    assert lines[0]["output_ids"] == plain_gpt2.greedy_generate(cfg, w, p, 6)
    assert lines[-1]["n_requests"] == 1


def test_command_line_prompt_file_and_sample_seed(lively, tmp_path):
    """Prompts from a file (one a line, commas or blanks), and a sampling seed of its own:
    request i draws with seed + i, as the plain sampler does."""
    d, cfg, w = lively["tiny_b"]
    prompts = _prompts(cfg, (9, 20), 23)
    f = tmp_path / "prompts.txt"
    f.write_text(",".join(map(str, prompts[0])) + "\n\n" + " ".join(map(str, prompts[1])) + "\n")
    res = subprocess.run(
        [sys.executable, "-m", "hetero_serve_b200", "--weights", d, "--dtype", "float32",
         "--num-blocks", "16", "--max-new-tokens", "5", "--no-eos-stop", "--json",
         "--temperature", "0.8", "--sample-seed", "41", "--seed", "3", "--prompt-file", str(f)],
        capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.strip().splitlines()]
    assert lines[-1]["n_requests"] == 2
    for i, p in enumerate(prompts):
        ctx = list(p)
        for tok in lines[i]["output_ids"]:
            row = plain_gpt2.forward(cfg, w, ctx)[-1]
            assert tok == plain_gpt2.sample_token(row, 0.8, 0, plain_gpt2.uniform_for(41 + i, len(ctx)))
            ctx.append(tok)


def test_command_line_and_demo_with_random_weights():
    """`--model NAME` builds seeded random weights for a named configuration (no folder given)."""
    res = subprocess.run(
        [sys.executable, "-m", "hetero_serve_b200", "--model", "tiny-b", "--dtype", "bfloat16",
         "--num-blocks", "16", "--max-new-tokens", "5", "--no-eos-stop", "--json",
         "--random-prompts", "3:9", "--temperature", "0.7", "--top-k", "20"],
        capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.strip().splitlines()]
    assert [len(l["output_ids"]) for l in lines[:3]] == [5, 5, 5]
    assert lines[-1]["n_requests"] == 3
    demo = subprocess.run([sys.executable, "run_demo.py", "--model", "tiny"],
                          capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert demo.returncode == 0, demo.stderr[-2000:]
