"""Command line: generate from a model folder, or write a random-weights model folder.

Option names and meanings are the reference's where it has them:
``--prompt`` and ``--max-new-tokens`` (scripts/download_checkpoint.py:20-25, which samples
with temperature 0.8 and top-k 50 — the defaults here), ``--device``, ``--kv-block-size``,
``--num-kv-blocks`` and ``--max-batch-size`` (scripts/serve.py:23-33).  The reference fetches
its checkpoint from a hub (``--repo-id``, ``--filename``); this engine reads a local folder
(``--model``) with ``config.json`` and ``model.safetensors``.  The reference's scripts mask the
padding rows of the vocabulary (src/minigpt_infer/tokenizer.py:37-46); here ``--vocab-limit`` does.

    generate --model DIR --prompt-ids 5,17,3 --max-new-tokens 20
    generate --random-weights 0 --config config.json --write-model DIR
"""

from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--prompt", default=None,
                    help="text prompt (needs the GPT-2 tokenizer files of tiktoken on this machine)")
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--max-new-tokens", type=int, default=60)
    ap.add_argument("--temperature", type=float, default=0.8, help="0 = greedy")
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--vocab-limit", type=int, default=None,
                    help="ids at and above this are never sampled: rows that only pad the embedding "
                         "table (the reference masks ids >= 50257 of its 50304 rows)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--kv-block-size", type=int, default=16)
    ap.add_argument("--num-kv-blocks", type=int, default=2048)
    ap.add_argument("--max-batch-size", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                    help="write a model folder with random weights (needs --config, --write-model)")
    ap.add_argument("--config", help="config.json to take the sizes from (with --random-weights)")
    ap.add_argument("--write-model", help="folder to write (with --random-weights)")
    ap.add_argument("--weights-dtype", choices=["bfloat16", "float32"], default="float32")
    return ap


def _encode(text: str) -> list[int]:
    try:
        import tiktoken

        return tiktoken.get_encoding("gpt2").encode(text)
    except Exception as exc:  # noqa: BLE001 - missing package or missing vocabulary files
        raise SystemExit(f"--prompt needs tiktoken's GPT-2 files ({type(exc).__name__}: {exc}); "
                         "pass --prompt-ids instead") from None


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.random_weights is not None:
        if not (args.config and args.write_model):
            raise SystemExit("--random-weights needs --config and --write-model")
        from .config.model_config import read_config_json
        from .config.registry import family_for
        from .weights.random_init import write_random_model

        raw = read_config_json(args.config)
        family = family_for(raw)
        cfg = family.config_class.from_dict(raw, architecture=family.name)
        folder = write_random_model(args.write_model, cfg, args.random_weights, args.weights_dtype)
        print(f"wrote {folder} ({cfg.num_parameters() / 1e6:.1f}M parameters, seed {args.random_weights})")
        if not args.model:
            return 0
    if not args.model:
        raise SystemExit("--model is required")
    if args.prompt_ids:
        prompt = [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    elif args.prompt is not None:
        prompt = _encode(args.prompt)
    else:
        raise SystemExit("give --prompt-ids or --prompt")

    from . import EngineConfig, LLMEngine, SamplingParams

    engine = LLMEngine.from_pretrained(args.model, EngineConfig(
        block_size=args.kv_block_size, num_blocks=args.num_kv_blocks,
        max_batch_size=args.max_batch_size, max_num_batched_tokens=args.max_num_batched_tokens,
        dtype=args.dtype, device=args.device), vocab_limit=args.vocab_limit)
    print(f"config: {engine.config}", file=sys.stderr)
    print(f"params: {engine.config.num_parameters() / 1e6:.1f}M", file=sys.stderr)
    params = SamplingParams(max_tokens=args.max_new_tokens, temperature=args.temperature,
                            top_k=args.top_k, top_p=args.top_p, seed=args.seed)
    out = engine.generate([prompt], params)[0]
    print(json.dumps({"prompt_ids": prompt, "token_ids": out["token_ids"],
                      "finish_reason": out["finish_reason"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
