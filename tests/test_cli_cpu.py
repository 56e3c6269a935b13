"""The command line without a GPU: writing a random-weights model folder, and what it refuses."""

from __future__ import annotations

import json

import pytest

from mini_gpt_inference_b200 import cli
from mini_gpt_inference_b200.config import GPTConfig
from mini_gpt_inference_b200.weights import load_file


def _config_file(tmp_path, **extra):
    raw = dict(vocab_size=131, block_size=40, n_layer=2, n_head=3, n_embd=48, bias=True, **extra)
    path = tmp_path / "c.json"
    path.write_text(json.dumps(raw))
    return path, raw


def test_random_weights_mode_writes_a_model_folder(tmp_path, capsys):
    config, raw = _config_file(tmp_path)
    folder = tmp_path / "m"
    code = cli.main(["--random-weights", "5", "--config", str(config), "--write-model", str(folder),
                     "--weights-dtype", "bfloat16"])
    assert code == 0 and "seed 5" in capsys.readouterr().out
    cfg = GPTConfig.from_json(folder / "config.json")
    assert (cfg.vocab_size, cfg.n_positions, cfg.n_layer, cfg.n_head, cfg.n_embd) == (131, 40, 2, 3, 48)
    tensors = load_file(folder / "model.safetensors")
    assert tensors["tok_emb.weight"].shape == (131, 48)
    assert tensors["blocks.1.attn.qkv.weight"].shape == (144, 48)
    assert str(tensors["blocks.0.mlp.fc.weight"].dtype) == "torch.bfloat16"
    # the same seed gives the same folder, another seed another one
    again = tmp_path / "m2"
    cli.main(["--random-weights", "5", "--config", str(config), "--write-model", str(again),
              "--weights-dtype", "bfloat16"])
    other = tmp_path / "m3"
    cli.main(["--random-weights", "6", "--config", str(config), "--write-model", str(other),
              "--weights-dtype", "bfloat16"])
    same = load_file(again / "model.safetensors")
    diff = load_file(other / "model.safetensors")
    assert all((tensors[k].float() == same[k].float()).all() for k in tensors)
    assert any((tensors[k].float() != diff[k].float()).any() for k in tensors)


def test_refusals(tmp_path):
    config, _ = _config_file(tmp_path)
    with pytest.raises(SystemExit, match="--config and --write-model"):
        cli.main(["--random-weights", "1", "--config", str(config)])
    with pytest.raises(SystemExit, match="--model is required"):
        cli.main(["--prompt-ids", "1,2,3"])
    with pytest.raises(SystemExit, match="--prompt-ids or --prompt"):
        cli.main(["--model", str(tmp_path)])
    with pytest.raises(SystemExit):
        cli.main(["--dtype", "float16", "--model", str(tmp_path), "--prompt-ids", "1"])


def test_option_names_of_the_reference_are_kept():
    """scripts/download_checkpoint.py:20-25 (--prompt, --max-new-tokens; temperature 0.8 and top-k 50
    as the sampling defaults) and scripts/serve.py:23-33 (--device, --kv-block-size,
    --num-kv-blocks, --max-batch-size)."""
    args = cli.build_parser().parse_args(["--model", "x", "--prompt", "hi"])
    assert (args.max_new_tokens, args.temperature, args.top_k) == (60, 0.8, 50)
    assert (args.kv_block_size, args.num_kv_blocks, args.device) == (16, 2048, "cuda:0")
    assert args.max_batch_size > 0 and args.max_num_batched_tokens > 0
    assert args.vocab_limit is None
    assert cli.build_parser().parse_args(["--model", "x", "--vocab-limit", "50257"]).vocab_limit == 50257
