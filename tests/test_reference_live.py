"""Live anchors on the reference itself, when its checkout is on this machine
(the folder named by ``HETEROSERVE_SOURCE``, or the default below; skipped otherwise — the committed golden
file under tests/golden/ then stands alone).  The reference's CPU code is imported from that
path and run beside this repository's: nothing of it is copied here.

* the plain implementation against ``NumpyEngine`` (heteroserve/model/numpy_engine.py:89-214)
  on Tiny A, and on a Tiny-B-shaped model as far as the reference can express it
  (``n_inner = 320`` through the tensors' shapes, tanh GELU, the inverse-layer scaling folded
  into the query columns);
* the cache manager against ``BlockAllocator`` (heteroserve/kv/blocks.py:62-351) under random
  sequences of allocate / grow / publish / free: same page numbers, same hits, same
  evictions;
* the run summary against ``summarise`` (heteroserve/metrics.py:123-180).
"""

import os
import random
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_gpt2
from conftest import TINY_A, TINY_B
from hetero_serve_b200.cache import CacheManager, GroupSpec, OutOfPages
from hetero_serve_b200.cache.manager import chain_hashes
from hetero_serve_b200.weights import random_weights

REF = Path(os.environ.get("HETEROSERVE_SOURCE", "/root/reference"))
pytestmark = pytest.mark.skipif(not (REF / "heteroserve" / "model" / "numpy_engine.py").is_file(),
                                reason="no checkout of the reference on this machine")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, str(REF))
    try:
        from heteroserve import metrics
        from heteroserve.config import KVConfig, ModelConfig
        from heteroserve.kv import blocks
        from heteroserve.model.numpy_engine import NumpyEngine
        from heteroserve.model.weights import GPT2Weights, LayerWeights
    finally:
        sys.path.remove(str(REF))
    return dict(metrics=metrics, KVConfig=KVConfig, ModelConfig=ModelConfig, blocks=blocks,
                NumpyEngine=NumpyEngine, GPT2Weights=GPT2Weights, LayerWeights=LayerWeights)


def _reference_engine(ref, cfg, tensors):
    w = {k: v.numpy().astype(np.float32) for k, v in tensors.items()}
    mc = ref["ModelConfig"](name="t", n_layer=cfg["n_layer"], n_head=cfg["n_head"],
                            n_embd=cfg["n_embd"], vocab_size=cfg["vocab_size"],
                            n_ctx=cfg["n_positions"], layer_norm_eps=cfg["layer_norm_epsilon"])
    layers = []
    for i in range(mc.n_layer):
        p = f"h.{i}."
        layers.append(ref["LayerWeights"](
            ln1_g=w[p + "ln_1.weight"], ln1_b=w[p + "ln_1.bias"],
            attn_w=w[p + "attn.c_attn.weight"], attn_b=w[p + "attn.c_attn.bias"],
            proj_w=w[p + "attn.c_proj.weight"], proj_b=w[p + "attn.c_proj.bias"],
            ln2_g=w[p + "ln_2.weight"], ln2_b=w[p + "ln_2.bias"],
            fc_w=w[p + "mlp.c_fc.weight"], fc_b=w[p + "mlp.c_fc.bias"],
            fcp_w=w[p + "mlp.c_proj.weight"], fcp_b=w[p + "mlp.c_proj.bias"]))
    gw = ref["GPT2Weights"](cfg=mc, wte=w["wte.weight"], wpe=w["wpe.weight"], layers=layers,
                            lnf_g=w["ln_f.weight"], lnf_b=w["ln_f.bias"])
    return ref["NumpyEngine"](gw, mc)


def _compare(ref_engine, cfg, weights, prompt, n_decode=5):
    """Whole prompt, the prompt in two portions, and greedy decoding, against the plain model."""
    prompt = np.asarray(prompt, dtype=np.int64)
    whole, k, v = ref_engine.prefill(prompt, 0)
    cut = max(1, len(prompt) // 2)
    _l, k1, v1 = ref_engine.prefill(prompt[:cut], 0)
    chunked, _k, _v = ref_engine.prefill(prompt[cut:], cut, k1, v1) if cut < len(prompt) else (whole, k, v)
    toks = prompt.tolist()
    plain = plain_gpt2.forward(cfg, weights, toks)
    worst = max(np.abs(plain[-1].numpy() - whole).max(), np.abs(plain[-1].numpy() - chunked).max())
    nxt = int(np.argmax(whole))
    for step in range(n_decode):
        logits, kn, vn = ref_engine.decode_batch(np.array([nxt]), np.array([len(toks)]), [k], [v])
        toks.append(nxt)
        k, v = np.concatenate([k, kn[0]], axis=2), np.concatenate([v, vn[0]], axis=2)
        plain = plain_gpt2.forward(cfg, weights, toks)
        worst = max(worst, np.abs(plain[-1].numpy() - logits[0]).max())
        nxt = int(np.argmax(logits[0]))
    return float(worst)


def test_plain_model_equals_the_reference_engine_on_tiny_a(ref):
    cfg, tensors = random_weights(TINY_A, 0)
    eng = _reference_engine(ref, cfg, tensors)
    w = plain_gpt2.prepare_weights(tensors)
    for n, seed in ((17, 1), (33, 2), (5, 3)):
        prompt = np.random.default_rng(seed).integers(0, cfg["vocab_size"], size=n)
        assert _compare(eng, cfg, w, prompt) < 3e-6


def test_plain_model_equals_the_reference_engine_on_what_it_can_express_of_tiny_b(ref):
    """Tiny B's sizes (3 layers, 3 heads of 32, inner width 320, vocabulary 1000, eps 1e-6) and
    its inverse-layer scaling, which the reference lacks, folded into the query columns of
    c_attn; the activation is the reference's tanh GELU."""
    cfg = dict(TINY_B, activation_function="gelu_new")
    cfg, tensors = random_weights(cfg, 1)
    w = plain_gpt2.prepare_weights(tensors)                       # the plain model scales scores
    folded = {k: v.clone() for k, v in tensors.items()}
    E = cfg["n_embd"]
    for i in range(cfg["n_layer"]):
        folded[f"h.{i}.attn.c_attn.weight"][:, :E] /= (i + 1)
        folded[f"h.{i}.attn.c_attn.bias"][:E] /= (i + 1)
    eng = _reference_engine(ref, cfg, folded)                     # the reference does not
    for n, seed in ((31, 4), (70, 5), (1, 6)):
        prompt = np.random.default_rng(seed).integers(0, cfg["vocab_size"], size=n)
        assert _compare(eng, cfg, w, prompt) < 5e-6


# ---------------------------------------------------------------------------------------


def test_cache_manager_and_the_reference_allocator_make_the_same_decisions(ref):
    """The same random sequence of requests into both: allocate with prefix reuse, grow token
    by token, publish full pages, free.  Page numbers, cached-token counts, evictions and the
    free count agree at every step.  (This manager caps a match at (len-1)//page pages so that
    a shared page is never rewritten; the reference matches whole prompts and caps later, in
    its worker.  The prompts here always end inside a page, where the two agree.)"""
    blocks = ref["blocks"]
    PS, NB = 16, 24
    mc = ref["ModelConfig"](name="t", n_layer=1, n_head=1, n_embd=16, vocab_size=64, n_ctx=256)
    theirs = blocks.BlockAllocator(ref["KVConfig"](block_size=PS, num_blocks=NB), mc,
                                   allocate_pool=False)
    ours = CacheManager([GroupSpec()], NB, PS, max_requests=8, prefix_cache=True)
    assert blocks.chain_hashes(list(range(40)), PS) == chain_hashes(list(range(40)), PS)
    rng = random.Random(7)
    stems = [[rng.randrange(64) for _ in range(48)] for _ in range(3)]
    live: dict[str, dict] = {}
    n_id = 0
    for step in range(600):
        action = rng.random()
        if action < 0.35 and len(live) < 6:
            stem = rng.choice(stems)
            toks = stem[:rng.choice((0, 16, 32, 48))] + [rng.randrange(64)
                                                          for _ in range(rng.randrange(1, 15))]
            rid = f"r{n_id}"
            n_id += 1
            try:
                alloc = theirs.allocate(toks)
            except blocks.OutOfBlocks:
                with pytest.raises(OutOfPages):
                    ours.open(rid, toks)
                    ours.reserve(rid, len(toks))
                if rid in ours:
                    ours.close(rid)
                continue
            opened = ours.open(rid, toks)
            ours.reserve(rid, len(toks))
            ours.commit(rid, len(toks))
            assert ours.table(rid) == alloc.block_ids, (step, "allocate")
            assert opened.cached_tokens == alloc.num_cached_tokens
            live[rid] = dict(tokens=toks, blocks=list(alloc.block_ids))
        elif action < 0.65 and live:
            rid = rng.choice(sorted(live))
            r = live[rid]
            r["tokens"].append(rng.randrange(64))
            try:
                theirs.grow(r["blocks"], len(r["tokens"]))
            except blocks.OutOfBlocks:
                with pytest.raises(OutOfPages):
                    ours.reserve(rid, len(r["tokens"]))
                r["tokens"].pop()
                continue
            ours.reserve(rid, len(r["tokens"]))
            ours.commit(rid, len(r["tokens"]))
            assert ours.table(rid) == r["blocks"], (step, "grow")
        elif action < 0.8 and live:
            rid = rng.choice(sorted(live))
            r = live[rid]
            theirs.register_full_blocks(r["tokens"], r["blocks"])
            ours.publish(rid, r["tokens"])
        elif live:
            rid = rng.choice(sorted(live))
            r = live.pop(rid)
            theirs.register_full_blocks(r["tokens"], r["blocks"])
            ours.publish(rid, r["tokens"])
            theirs.free_sequence(r["blocks"])
            ours.close(rid)
        assert ours.pages_free() == theirs.num_free, step
        assert ours.pools[0].evictions == theirs.stat_evictions, step
        ours.check()
    assert theirs.stat_evictions > 0 and theirs.stat_hits > 0       # the sequence did exercise both


def test_summary_equals_the_reference_summary(ref):
    from hetero_serve_b200.engine.metrics import RequestRecord, percentile, summarise
    m = ref["metrics"]
    rng = random.Random(3)
    for n in (1, 2, 5, 40):
        vals = [rng.random() for _ in range(n)]
        for p in (0.0, 0.5, 0.95, 1.0):
            assert percentile(vals, p) == pytest.approx(m.percentile(vals, p), rel=1e-12, abs=1e-15)
    ours, theirs = [], []
    for i in range(30):
        t0 = rng.random()
        first = t0 + rng.random() * 0.1
        done = first + rng.random()
        gen = rng.randrange(1, 20)
        kw = dict(prompt_tokens=rng.randrange(1, 100), generated_tokens=gen,
                  cached_prefix_tokens=rng.choice((0, 16, 32)), preemptions=rng.randrange(2),
                  t_submit=t0, t_first_token=first, t_done=done if i % 7 else 0.0)
        ours.append(RequestRecord(req_id=i, **kw))
        theirs.append(m.RequestRecord(req_id=str(i), **kw))
    a, b = summarise(ours, 3.5), m.summarise(theirs, 3.5).as_dict()
    shared = [k for k in a if k in b]
    assert len(shared) >= 12
    for key in shared:          # the reference rounds its quantiles to 4-5 places
        assert a[key] == pytest.approx(b[key], abs=6e-5, nan_ok=True), key
