"""Weights by name, their errors, and the random-weights mode (no GPU)."""

import json

import pytest
import torch

from hetero_serve_b200.architectures.gpt2 import build_spec
from hetero_serve_b200.architectures.gpt2 import GPT2Config
from hetero_serve_b200.parts import Model
from hetero_serve_b200.weights import (SafetensorsError, WeightError, load_checkpoint,
                                       random_weights, read_safetensors, write_model_dir,
                                       write_safetensors)
from conftest import TINY_A, TINY_B


def _model(cfg):
    return Model(build_spec(GPT2Config.from_dict(cfg)))


def test_safetensors_roundtrip_keeps_types(tmp_path):
    t = {"f": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "h": torch.randn(2, 2).half(),
         "i": torch.arange(6, dtype=torch.int64).reshape(2, 3), "s": torch.tensor(1.5),
         "e": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", t, {"note": "test"})
    r = read_safetensors(tmp_path / "x.safetensors")
    assert r["f"].dtype == torch.float32 and torch.equal(r["f"], t["f"])
    assert r["b"].dtype == torch.bfloat16 and torch.equal(r["b"], t["b"])     # stays bfloat16
    assert r["h"].dtype == torch.float16
    assert r["i"].dtype == torch.int32 and r["i"].tolist() == t["i"].tolist()  # tables → int32
    assert r["s"].shape == () and r["e"].shape == (0, 4)


def test_safetensors_rejects_garbage(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        read_safetensors(p)
    p.write_bytes((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        read_safetensors(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not\n?.*match|does not match"):
        read_safetensors(p)
    hdr = json.dumps({"a": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_safetensors(p)


def test_random_weights_are_seeded_and_follow_the_scheme():
    _, a = random_weights(TINY_A, 0)
    _, b = random_weights(TINY_A, 0)
    _, c = random_weights(TINY_A, 1)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["wte.weight"], c["wte.weight"])
    assert a["h.0.attn.c_attn.weight"].shape == (64, 192)           # Conv1D: [in, out]
    assert a["h.1.mlp.c_fc.weight"].shape == (64, 256)
    assert abs(float(a["wte.weight"].std()) - 0.02) < 0.002
    assert abs(float(a["h.0.mlp.c_proj.weight"].std()) - 0.02 / 2.0) < 0.002   # 0.02/sqrt(2*2)
    assert abs(float(a["h.0.ln_1.weight"].mean()) - 1.0) < 0.02
    assert float(a["h.0.attn.c_attn.bias"].abs().max()) > 0          # biases are not zero
    assert "lm_head.weight" not in a                                   # tied


def test_model_folder_roundtrip(tmp_path):
    d = write_model_dir(tmp_path / "m", TINY_B, 1, "float32")
    assert json.loads((d / "config.json").read_text())["n_inner"] == 320
    model = _model(TINY_B)
    stored = load_checkpoint(d, model)
    _, fresh = random_weights(TINY_B, 1)
    assert set(stored) == set(fresh)
    assert all(torch.equal(stored[k], fresh[k]) for k in fresh)
    model.bind(stored, torch.float32, "cpu")
    mixer = model.blocks[0].mixer
    assert mixer.w_qkv.shape == (288, 96)                # transposed once to [out, in]
    assert torch.equal(mixer.w_qkv, fresh["h.0.attn.c_attn.weight"].t())
    assert model.head.weight is model.embedding.table   # tied: one tensor


def test_bfloat16_folder_keeps_matrices_bf16_and_vectors_fp32(tmp_path):
    d = write_model_dir(tmp_path / "m", TINY_A, 0, "bfloat16")
    raw = read_safetensors(d / "model.safetensors")
    assert raw["wte.weight"].dtype == torch.bfloat16
    assert raw["h.0.mlp.c_fc.weight"].dtype == torch.bfloat16
    assert raw["h.0.ln_1.weight"].dtype == torch.float32      # stored in 32-bit: stays so
    model = _model(TINY_A)
    model.bind(load_checkpoint(d, model), torch.bfloat16, "cpu")
    assert model.embedding.table.dtype == torch.bfloat16
    assert model.blocks[0].norm1.weight.dtype == torch.float32
    assert model.blocks[0].mixer.b_qkv.dtype == torch.float32


def test_prefixes_and_buffers_are_accepted(tmp_path):
    _, w = random_weights(TINY_A, 0)
    w2 = {"transformer." + k: v for k, v in w.items()}
    w2["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)           # causal-mask buffers
    w2["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    w2["lm_head.weight"] = w["wte.weight"].clone()                      # tied copy
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(tmp_path / "model.safetensors", w2)
    stored = load_checkpoint(tmp_path, _model(TINY_A))
    assert set(stored) == set(w)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    _, w = random_weights(TINY_A, 0)
    del w["h.1.ln_2.bias"]
    del w["wpe.weight"]
    w["h.0.attn.c_attn.weight"] = torch.zeros(192, 64)       # transposed by mistake
    w["h.0.mlp.c_fc.bias"] = torch.zeros(255)
    w["h.7.ln_1.weight"] = torch.zeros(64)                   # a layer the config has not
    w["rotary.inv_freq"] = torch.zeros(8)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(tmp_path / "model.safetensors", w)
    with pytest.raises(WeightError) as ei:
        load_checkpoint(tmp_path, _model(TINY_A))
    e = ei.value
    assert e.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert e.unexpected == ["h.7.ln_1.weight", "rotary.inv_freq"]
    assert e.wrong_shape == {"h.0.attn.c_attn.weight": ((192, 64), (64, 192)),
                             "h.0.mlp.c_fc.bias": ((255,), (256,))}
    msg = str(e)
    for needle in ("missing (2)", "wpe.weight", "unexpected (2)", "rotary.inv_freq",
                   "h.0.attn.c_attn.weight is [192, 64], expected [64, 192]"):
        assert needle in msg


def test_missing_file_and_sharded_checkpoint(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_checkpoint(tmp_path, _model(TINY_A))
    (tmp_path / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(WeightError, match="sharded"):
        load_checkpoint(tmp_path, _model(TINY_A))


def test_untied_head_needs_its_own_tensor(tmp_path):
    cfg = dict(TINY_A, tie_word_embeddings=False)
    _, w = random_weights(cfg, 0)
    assert "lm_head.weight" in w
    del w["lm_head.weight"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", w)
    with pytest.raises(WeightError) as ei:
        load_checkpoint(tmp_path, _model(cfg))
    assert ei.value.missing == ["lm_head.weight"]
