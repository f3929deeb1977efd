"""Named GPT-2 configurations for the random-weights mode, written as config.json
dictionaries.  ``gpt2`` is the reference's default ``ModelConfig()``
(heteroserve/config.py:22-33); ``tiny`` is its ``ModelConfig.tiny()`` (config.py:72-83);
the others are the sizes the benchmark and the tests name.
"""

from __future__ import annotations

from .model_config import ConfigError

_BASE = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
         "tie_word_embeddings": True, "eos_token_id": 50256}

PRESETS: dict[str, dict] = {
    "tiny-a": dict(_BASE, n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512,
                   n_positions=128, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                   scale_attn_by_inverse_layer_idx=False, eos_token_id=511),
    "tiny-b": dict(_BASE, n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000,
                   n_positions=256, layer_norm_epsilon=1e-6, activation_function="gelu",
                   scale_attn_by_inverse_layer_idx=True, eos_token_id=999),
    "tiny": dict(_BASE, n_layer=4, n_embd=256, n_head=4, n_inner=None, vocab_size=50257,
                 n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2": dict(_BASE, n_layer=12, n_embd=768, n_head=12, n_inner=None, vocab_size=50257,
                 n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "gpt2-medium": dict(_BASE, n_layer=24, n_embd=1024, n_head=16, n_inner=4096,
                        vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                        activation_function="gelu_new"),
    "gpt2-large": dict(_BASE, n_layer=36, n_embd=1280, n_head=20, n_inner=5120,
                       vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                       activation_function="gelu_new"),
    "gpt2-xl": dict(_BASE, n_layer=48, n_embd=1600, n_head=25, n_inner=6400,
                    vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5,
                    activation_function="gelu_new"),
}
_ALIASES = {"tinya": "tiny-a", "tinyb": "tiny-b", "medium": "gpt2-medium",
            "large": "gpt2-large", "xl": "gpt2-xl"}


def preset(name: str) -> dict:
    key = _ALIASES.get(name.lower().replace("_", "-"), name.lower().replace("_", "-"))
    if key not in PRESETS:
        raise ConfigError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    return dict(PRESETS[key])
