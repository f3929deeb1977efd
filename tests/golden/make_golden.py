#!/usr/bin/env python3
"""Writes ``tests/golden/tiny_a_reference.npz``: outputs of the reference's own CPU engine
(``heteroserve/model/numpy_engine.py`` of mneha05/hetero-serve) on a tiny random GPT-2.

    python tests/golden/make_golden.py /path/to/hetero-serve

The weights are this repository's seeded random weights for the configuration below
(written and read back through its safetensors code), handed to the reference as its own
``GPT2Weights`` / ``LayerWeights`` dataclasses.  The reference engine then runs

* a 17-token prompt whole (``prefill``) — the last position's logits,
* the same prompt as 12 + 5 tokens with the past passed in (chunked ``prefill``),
* six greedy ``decode_batch`` steps after the prompt — logits of each step.

Only options the reference has are used: tanh GELU, 4x inner width, 1/sqrt(head_dim).
``tests/test_plain.py`` compares the plain implementation with these outputs.
"""

import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

CONFIG = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2, "n_embd": 64,
          "n_head": 4, "n_inner": 256, "vocab_size": 512, "n_positions": 128,
          "layer_norm_epsilon": 1e-5, "activation_function": "gelu_new",
          "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True}
SEED = 0
PROMPT_SEED = 1234


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from heteroserve.config import ModelConfig
    from heteroserve.model.numpy_engine import NumpyEngine
    from heteroserve.model.weights import GPT2Weights, LayerWeights

    from hetero_serve_b200.weights import random_weights

    _, tensors = random_weights(CONFIG, SEED)
    w = {k: v.numpy().astype(np.float32) for k, v in tensors.items()}
    cfg = ModelConfig(name="tiny-a", n_layer=2, n_head=4, n_embd=64, vocab_size=512, n_ctx=128,
                      layer_norm_eps=1e-5)
    layers = []
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        layers.append(LayerWeights(
            ln1_g=w[p + "ln_1.weight"], ln1_b=w[p + "ln_1.bias"],
            attn_w=w[p + "attn.c_attn.weight"], attn_b=w[p + "attn.c_attn.bias"],
            proj_w=w[p + "attn.c_proj.weight"], proj_b=w[p + "attn.c_proj.bias"],
            ln2_g=w[p + "ln_2.weight"], ln2_b=w[p + "ln_2.bias"],
            fc_w=w[p + "mlp.c_fc.weight"], fc_b=w[p + "mlp.c_fc.bias"],
            fcp_w=w[p + "mlp.c_proj.weight"], fcp_b=w[p + "mlp.c_proj.bias"]))
    gw = GPT2Weights(cfg=cfg, wte=w["wte.weight"], wpe=w["wpe.weight"], layers=layers,
                     lnf_g=w["ln_f.weight"], lnf_b=w["ln_f.bias"])
    eng = NumpyEngine(gw, cfg)

    prompt = np.random.default_rng(PROMPT_SEED).integers(0, 512, size=17).astype(np.int64)
    whole, k, v = eng.prefill(prompt, 0)
    l1, k1, v1 = eng.prefill(prompt[:12], 0)
    chunked, k2, v2 = eng.prefill(prompt[12:], 12, k1, v1)
    past_k, past_v = k, v
    toks = [int(np.argmax(whole))]
    dec = []
    for step in range(6):
        pos = 17 + step
        logits, kn, vn = eng.decode_batch(np.array([toks[-1]]), np.array([pos]),
                                          [past_k], [past_v])
        dec.append(logits[0])
        past_k = np.concatenate([past_k, kn[0]], axis=2)
        past_v = np.concatenate([past_v, vn[0]], axis=2)
        toks.append(int(np.argmax(logits[0])))
    np.savez_compressed(HERE / "tiny_a_reference.npz", prompt=prompt,
                        whole_last=whole.astype(np.float32),
                        chunked_last=chunked.astype(np.float32),
                        decode_logits=np.stack(dec).astype(np.float32),
                        greedy_tokens=np.array(toks, dtype=np.int64),
                        config=np.frombuffer(json.dumps(CONFIG).encode(), dtype=np.uint8),
                        seed=np.array(SEED))
    print("wrote", HERE / "tiny_a_reference.npz", "greedy tokens", toks)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
