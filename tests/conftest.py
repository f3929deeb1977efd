"""Shared fixtures: two tiny GPT-2 configurations that differ in every size and option,
model folders with random weights (made in temporary folders, never committed), and the
plain implementation's view of the same weights."""

import json
import os
import sys
from pathlib import Path

import pytest
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
for p in (str(ROOT), str(HERE)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


_BASE = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "tie_word_embeddings": True}

# every size and option differs: layers, width, heads, head size (16 / 32), inner width
# (4x / not 4x), vocabulary (a power of two / not), table length, eps, activation, scaling
TINY_A = dict(_BASE, n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512,
              n_positions=128, layer_norm_epsilon=1e-5, activation_function="gelu_new",
              scale_attn_by_inverse_layer_idx=False, eos_token_id=511)
TINY_B = dict(_BASE, n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000,
              n_positions=256, layer_norm_epsilon=1e-6, activation_function="gelu",
              scale_attn_by_inverse_layer_idx=True, eos_token_id=999)
TINY = {"tiny_a": (TINY_A, 0), "tiny_b": (TINY_B, 1)}


class TinyModel:
    def __init__(self, name, folder, config, seed):
        from hetero_serve_b200.weights import read_safetensors
        import plain_gpt2
        self.name, self.dir, self.config, self.seed = name, str(folder), config, seed
        self.raw = read_safetensors(Path(folder) / "model.safetensors")
        self.plain = plain_gpt2.prepare_weights(self.raw)                       # float64
        self.plain_bf16 = plain_gpt2.prepare_weights(self.raw, round_to=torch.bfloat16)
        self._cache = {}

    def weights_for(self, dtype):
        return self.plain_bf16 if dtype == "bfloat16" else self.plain

    def logits(self, tokens, dtype="float32"):
        """Plain logits [T, V] (float64 arithmetic; bfloat16 → weights rounded first)."""
        import plain_gpt2
        key = (tuple(tokens), dtype)
        if key not in self._cache:
            self._cache[key] = plain_gpt2.forward(self.config, self.weights_for(dtype), tokens)
        return self._cache[key]

    def tokens(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.config["vocab_size"], (n,), generator=g).tolist()


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    from hetero_serve_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed) in TINY.items():
        folder = tmp_path_factory.mktemp(name)
        write_model_dir(folder, cfg, seed, "float32")
        out[name] = TinyModel(name, folder, json.loads((folder / "config.json").read_text()), seed)
    return out


@pytest.fixture(params=["tiny_a", "tiny_b"])
def tiny(request, tiny_models):
    return tiny_models[request.param]


# logits of these models are O(1); tolerances are absolute, per precision.
# float32: kernels accumulate in float32 over at most a few hundred terms.
# bfloat16: activations between kernels are rounded to 8 bits of mantissa.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
