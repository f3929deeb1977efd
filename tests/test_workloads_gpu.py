"""Whole workloads through the Python entry point at the real widths of GPT-2 large and XL (two
layers each, random weights), shaped like the larger configurations the reference is quoted on:
many requests of mixed lengths, some sharing a prompt prefix, prompts cut into portions, and a
cache pool small enough to force recompute-preemption.  Every request must get exactly the
tokens it gets from an engine with room for everything and no prefix reuse (float32: the same
arithmetic whatever the batching), and the cache manager must come out whole."""

import json
import random

import pytest

from hetero_serve_b200 import EngineConfig, LLMEngine, Request
from hetero_serve_b200.weights import write_model_dir

pytestmark = pytest.mark.gpu

SIZES = {
    "large": dict(n_layer=2, n_embd=1280, n_head=20),
    "xl": dict(n_layer=2, n_embd=1600, n_head=25),
}


@pytest.fixture(scope="module", params=list(SIZES))
def model_dir(request, tmp_path_factory):
    cfg = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", vocab_size=50257,
               n_positions=1024, n_inner=None, layer_norm_epsilon=1e-5,
               activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, eos_token_id=50256, **SIZES[request.param])
    d = tmp_path_factory.mktemp("workload_" + request.param)
    write_model_dir(d, cfg, 5, "float32")
    return str(d)


def _requests(n, seed):
    rng = random.Random(seed)
    shared = [rng.randrange(50257) for _ in range(64)]
    reqs = []
    for i in range(n):
        length = rng.randint(20, 260)
        body = [rng.randrange(50257) for _ in range(length)]
        prompt = shared + body if i % 4 == 0 else body          # a quarter share 64 tokens
        reqs.append(Request(prompt, max_new_tokens=rng.randint(4, 20), seed=i,
                            temperature=0.0 if i % 3 else 0.8, top_k=0 if i % 3 else 50,
                            stop_at_eos=False, req_id=f"w{i}"))
    return reqs


def _run(model_dir, reqs, **cfg):
    eng = LLMEngine(model_dir, EngineConfig(dtype="float32", **cfg))
    seqs = []
    pending = list(reqs)
    rng = random.Random(1)
    records = []
    while pending or eng.has_work():
        for _ in range(rng.randint(0, 3)):                       # requests keep arriving
            if pending:
                r = pending.pop(0)
                seqs.append(eng.submit_nowait(Request(r.prompt_ids, r.max_new_tokens, r.temperature,
                                                      r.top_k, r.seed, r.stop_at_eos, r.req_id)))
        if eng.has_work():
            records.extend(eng.step())
    eng.runner.manager.check()
    assert eng.runner.manager.free_slots() == eng.config.live_requests
    return eng, {s.req_id: list(s.output_ids) for s in seqs}, records


@pytest.mark.parametrize("policy", ["prefill_first", "mixed"])
def test_many_requests_small_pool_same_tokens_as_a_roomy_engine(model_dir, policy):
    reqs = _requests(20, seed=3)
    # room for about three of the longest requests: admissions wait, decoding preempts
    tight, out_tight, rec = _run(model_dir, reqs, num_blocks=64, max_batch=8, max_requests=8,
                                 max_prefill_tokens=128, policy=policy, prefix_cache=True)
    roomy, out_roomy, _ = _run(model_dir, reqs, num_blocks=1024, max_batch=8, max_requests=8,
                               max_prefill_tokens=512, policy="prefill_first", prefix_cache=False,
                               pipeline=False)
    assert out_tight == out_roomy
    assert all(len(out_tight[r.req_id]) == r.max_new_tokens for r in reqs)
    msg = tight.state_message()
    assert msg["finished"] == len(reqs) and msg["preemptions"] >= 1
    assert msg["tokens_saved_by_cache"] >= 64            # somebody reused the shared prefix
    assert msg["prefill_steps"] + msg["mixed_steps"] > len(reqs)   # prompts were cut into portions
    assert json.dumps(msg)                                # the state message is plain data
