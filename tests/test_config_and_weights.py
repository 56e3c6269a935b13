"""Configuration, registry, safetensors reading and the loader's errors (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

from tiny_configs import TINY_A, TINY_B, tiny_config

from mini_gpt_inference_b200.config import (ConfigError, GPTConfig, UnknownArchitectureError,
                                            load_config, lookup)
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import (WeightsError, check_and_bind, load_checkpoint,
                                             load_file, random_tensors, save_file,
                                             write_random_model)


def _model(cfg):
    return DecoderModel(lookup(cfg.architecture).describe(cfg))


def test_config_reads_reference_field_names():
    # src/minigpt_infer/config.py:10-18: block_size is the position table's length.
    cfg = GPTConfig.from_dict({"vocab_size": 50304, "block_size": 512, "n_layer": 8, "n_head": 8,
                               "n_embd": 512, "dropout": 0.0, "bias": False})
    assert cfg.n_positions == 512 and cfg.n_inner == 2048 and cfg.head_dim == 64
    assert cfg.layer_norm_epsilon == 1e-5 and cfg.bias is False
    # the reference's own parameter count (docs/PLAN.md:44-59)
    assert cfg.num_parameters() == 51_192_320 + 0


def test_config_requires_every_size():
    with pytest.raises(ConfigError, match="n_layer"):
        GPTConfig.from_dict({"vocab_size": 10, "block_size": 8, "n_head": 2, "n_embd": 8})


@pytest.mark.parametrize("patch,match", [
    ({"n_head": 5}, "divisible"),
    ({"activation_function": "relu"}, "activation_function"),
    ({"tie_word_embeddings": False}, "tie_word_embeddings"),
    ({"n_layer": 0}, "n_layer"),
    ({"layer_norm_epsilon": -1.0}, "layer_norm_epsilon"),
])
def test_config_rejects(patch, match):
    with pytest.raises(ConfigError, match=match):
        GPTConfig.from_dict({**TINY_A, **patch})


def test_config_aliases_conflict():
    with pytest.raises(ConfigError, match="twice"):
        GPTConfig.from_dict({**TINY_A, "block_size": 99})


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = tiny_config("A"), tiny_config("B")
    for name in ("vocab_size", "n_positions", "n_layer", "n_head", "n_embd", "n_inner", "bias",
                 "layer_norm_epsilon", "head_dim"):
        assert getattr(a, name) != getattr(b, name), name
    assert b.vocab_size % 2 == 1 and b.n_embd & (b.n_embd - 1) != 0


def test_registry_and_model_folder(tmp_path):
    cfg = tiny_config("A")
    folder = write_random_model(tmp_path / "m", cfg, seed=1)
    family, loaded = load_config(folder)
    assert family.name == "MiniGPTLMHeadModel" and loaded == cfg
    raw = json.loads((folder / "config.json").read_text())
    raw["architectures"] = ["SomethingElse"]
    (folder / "config.json").write_text(json.dumps(raw))
    with pytest.raises(UnknownArchitectureError, match="SomethingElse.*known"):
        load_config(folder)
    # no architecture key at all: the reference's bare field dict
    (folder / "config.json").write_text(json.dumps(
        {"vocab_size": 256, "block_size": 64, "n_layer": 2, "n_head": 4, "n_embd": 64, "bias": True}))
    assert load_config(folder)[1].n_positions == 64


def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "s": torch.tensor(2.5)}
    save_file(tensors, tmp_path / "x.safetensors", {"k": "v"})
    back = load_file(tmp_path / "x.safetensors")
    assert set(back) == set(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and torch.equal(back[k], tensors[k])
    # readable by the safetensors package too, if it is there
    try:
        from safetensors.torch import load_file as theirs
    except ImportError:
        return
    other = theirs(str(tmp_path / "x.safetensors"))
    assert all(torch.equal(other[k], tensors[k]) for k in tensors)


def test_random_weights_follow_the_scheme_and_the_seed(tmp_path):
    cfg = tiny_config("A")
    m = _model(cfg)
    t1, t2, t3 = random_tensors(m, 5), random_tensors(m, 5), random_tensors(m, 6)
    assert all(torch.equal(t1[k], t2[k]) for k in t1)
    assert any(not torch.equal(t1[k], t3[k]) for k in t1)
    assert "lm_head.weight" not in t1                      # tied: stored once
    assert abs(t1["tok_emb.weight"].std().item() - 0.02) < 2e-3
    # residual projections N(0, 0.02 / sqrt(2 L))    (src/minigpt_infer/model.py:132-136)
    want = 0.02 / (2 * cfg.n_layer) ** 0.5
    assert abs(t1["blocks.0.mlp.proj.weight"].std().item() - want) < 2e-3
    assert abs(t1["ln_f.weight"].mean().item() - 1.0) < 0.05
    assert t1["blocks.0.attn.qkv.bias"].abs().max() > 0    # biases are not zero: a dropped bias shows
    folder = write_random_model(tmp_path / "bf", cfg, 5, "bfloat16")
    stored = load_file(folder / "model.safetensors")
    assert all(v.dtype == torch.bfloat16 for v in stored.values())


def test_loader_keeps_storage_dtype_and_strips_prefixes():
    cfg = tiny_config("B")
    m = _model(cfg)
    tensors = random_tensors(m, 2)
    mixed = {("module._orig_mod." + k if True else k): v for k, v in tensors.items()}
    mixed["module._orig_mod.tok_emb.weight"] = tensors["tok_emb.weight"].to(torch.bfloat16)
    bound = check_and_bind(mixed, m.tensor_specs())
    assert bound["tok_emb.weight"].dtype == torch.bfloat16
    assert bound["pos_emb.weight"].dtype == torch.float32
    assert set(bound) == set(tensors)


def test_loader_reports_everything_at_once(tmp_path):
    cfg = tiny_config("A")
    m = _model(cfg)
    tensors = random_tensors(m, 3)
    del tensors["blocks.1.ln2.bias"]
    del tensors["pos_emb.weight"]
    tensors["blocks.0.attn.rotary.inv_freq"] = torch.zeros(4)
    tensors["blocks.0.mlp.fc.weight"] = torch.zeros(cfg.n_inner + 1, cfg.n_embd)
    save_file(tensors, tmp_path / "model.safetensors")
    with pytest.raises(WeightsError) as err:
        load_checkpoint(tmp_path, m.tensor_specs())
    e = err.value
    assert sorted(e.missing) == ["blocks.1.ln2.bias", "pos_emb.weight"]
    assert e.unexpected == ["blocks.0.attn.rotary.inv_freq"]
    assert len(e.wrong_shape) == 1 and "blocks.0.mlp.fc.weight" in e.wrong_shape[0]
    text = str(e)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (1)", "(257, 64)", "(256, 64)"):
        assert piece in text, text


def test_bias_tensors_without_bias_option_are_unexpected():
    cfg_b = tiny_config("B")                                # bias = False
    m = _model(cfg_b)
    tensors = random_tensors(m, 1)
    tensors["blocks.0.attn.qkv.bias"] = torch.zeros(3 * cfg_b.n_embd)
    with pytest.raises(WeightsError, match="unexpected"):
        check_and_bind(tensors, m.tensor_specs())


def test_tied_head_stored_twice_must_agree():
    cfg = tiny_config("A")
    m = _model(cfg)
    tensors = random_tensors(m, 4)
    tensors["lm_head.weight"] = tensors["tok_emb.weight"].clone()
    check_and_bind(tensors, m.tensor_specs())              # equal copy: fine
    tensors["lm_head.weight"][0, 0] += 1.0
    with pytest.raises(WeightsError, match="tied"):
        check_and_bind(tensors, m.tensor_specs())


def test_missing_file(tmp_path):
    with pytest.raises(WeightsError, match="model.safetensors"):
        load_checkpoint(tmp_path, {})
    (tmp_path / "model.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(WeightsError, match="too short"):
        load_checkpoint(tmp_path, {})


def test_malformed_safetensors_files_give_clear_errors(tmp_path):
    import json
    import struct

    from mini_gpt_inference_b200.weights.safetensors_io import SafetensorsError

    def attempt(data: bytes, match: str):
        path = tmp_path / "bad.safetensors"
        path.write_bytes(data)
        with pytest.raises(SafetensorsError, match=match):
            load_file(path)

    def with_header(header: dict, payload: bytes) -> bytes:
        raw = json.dumps(header).encode()
        return struct.pack("<Q", len(raw)) + raw + payload

    attempt(b"", "too short")
    attempt(struct.pack("<Q", 1 << 40) + b"{}", "does not fit")
    attempt(struct.pack("<Q", 5) + b"hello", "not JSON")
    attempt(with_header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8), "offsets")
    attempt(with_header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 8), "offsets")
    attempt(with_header({"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 8]}}, b"\0" * 8), "shape")
    attempt(with_header({"a": {"dtype": "Q7", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8), "unsupported dtype")
    # a header whose structure is wrong is reported as such, whatever Python would have raised
    attempt(with_header({"a": {"dtype": "F32", "shape": [2]}}, b"\0" * 8), "data_offsets")
    attempt(with_header({"a": [1, 2]}, b"\0" * 8), "not an object")
    attempt(struct.pack("<Q", 2) + b"[]", "not a JSON object")
    attempt(with_header({"a": {"dtype": "F32", "shape": [-2, -1], "data_offsets": [0, 8]}}, b"\0" * 8), "shape")
    attempt(with_header({"a": {"dtype": "F32", "shape": "2", "data_offsets": [0, 8]}}, b"\0" * 8), "shape")
    attempt(with_header({"a": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}, b"\0" * 8), "data_offsets")
    attempt(with_header({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8.0]}}, b"\0" * 8), "data_offsets")
    attempt(with_header({"a": {"dtype": 7, "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8), "unsupported dtype")
    attempt(with_header({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                         "b": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8), "overlap")


def test_loader_reports_wrong_dtypes_with_the_rest():
    """Storage is kept as it is (bfloat16, 32-bit); a tensor stored as anything else is not
    converted behind the user's back but named, in the same error as the other faults."""
    cfg = tiny_config("A")
    m = _model(cfg)
    tensors = random_tensors(m, 3)
    tensors["blocks.0.mlp.fc.weight"] = tensors["blocks.0.mlp.fc.weight"].to(torch.float16)
    tensors["ln_f.weight"] = tensors["ln_f.weight"].to(torch.float64)
    tensors["tok_emb.weight"] = tensors["tok_emb.weight"].to(torch.int32)
    del tensors["ln_f.bias"]
    with pytest.raises(WeightsError) as err:
        check_and_bind(tensors, m.tensor_specs())
    e = err.value
    assert e.missing == ["ln_f.bias"] and len(e.wrong_dtype) == 3
    text = str(e)
    for piece in ("wrong dtype (3)", "blocks.0.mlp.fc.weight: checkpoint float16", "ln_f.weight: checkpoint float64",
                  "tok_emb.weight: checkpoint int32", "bfloat16 or float32", "missing (1)"):
        assert piece in text, text
