"""Typed model configuration for the GPT-2 style decoder, read from ``config.json``.

The fields are the ones the reference keeps in its ``GPTConfig`` dataclass
(src/minigpt_infer/config.py:10-18) plus the constants that the reference fixes
in code and that a config file has to be able to state:

* ``n_inner``: the reference hard-codes ``4 * n_embd`` (src/minigpt_infer/model.py:96);
* ``layer_norm_epsilon``: the reference uses ``nn.LayerNorm``'s default 1e-5
  (src/minigpt_infer/model.py:107-109, 127);
* ``activation_function``: fixed to tanh-GELU (src/minigpt_infer/model.py:101);
* ``tie_word_embeddings``: fixed to tied (src/minigpt_infer/model.py:128-130).

Every size is required; nothing in the engine carries a model size of its own.
"""

from __future__ import annotations

import json
import warnings
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can run."""


_GELU_TANH_NAMES = ("gelu_tanh", "gelu_new", "gelu_pytorch_tanh")

# config.json key -> field name, for the spellings a GPT-2 style config may use.
_ALIASES = {
    "block_size": "n_positions",      # the reference's own name (config.py:13)
    "n_ctx": "n_positions",
    "max_position_embeddings": "n_positions",
    "layer_norm_eps": "layer_norm_epsilon",
}

_IGNORED_KEYS = {
    "architectures", "model_type", "torch_dtype", "dtype", "transformers_version",
    "_name_or_path", "bos_token_id", "eos_token_id", "pad_token_id", "use_cache",
}


@dataclass(frozen=True)
class GPTConfig:
    """Sizes and constants of one GPT-2 style decoder."""

    vocab_size: int
    n_positions: int
    n_layer: int
    n_head: int
    n_embd: int
    n_inner: int
    bias: bool = False
    layer_norm_epsilon: float = 1e-5
    activation_function: str = "gelu_tanh"
    tie_word_embeddings: bool = True
    dropout: float = 0.0
    architecture: str = "MiniGPTLMHeadModel"
    torch_dtype: str = "float32"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    def __post_init__(self) -> None:
        problems = []
        for name in ("vocab_size", "n_positions", "n_layer", "n_head", "n_embd", "n_inner"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                problems.append(f"{name} must be a positive integer, got {value!r}")
        if not problems and self.n_embd % self.n_head != 0:
            # src/minigpt_infer/model.py:39 asserts the same.
            problems.append(
                f"n_embd ({self.n_embd}) must be divisible by n_head ({self.n_head})")
        if self.activation_function not in _GELU_TANH_NAMES:
            problems.append(
                f"activation_function {self.activation_function!r} is not supported; "
                f"this architecture uses tanh-GELU ({', '.join(_GELU_TANH_NAMES)})")
        if not self.tie_word_embeddings:
            problems.append("tie_word_embeddings must be true: the output head shares "
                            "tok_emb.weight in this architecture")
        if not (isinstance(self.layer_norm_epsilon, float) and self.layer_norm_epsilon > 0):
            problems.append(
                f"layer_norm_epsilon must be a positive float, got {self.layer_norm_epsilon!r}")
        if problems:
            raise ConfigError("invalid GPT config: " + "; ".join(problems))

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], architecture: str | None = None) -> "GPTConfig":
        values: dict[str, Any] = {}
        extra: dict[str, Any] = {}
        known = set(cls.__dataclass_fields__) - {"extra", "architecture"}
        for key, value in raw.items():
            name = _ALIASES.get(key, key)
            if name in known:
                if name in values and values[name] != value:
                    raise ConfigError(
                        f"config.json gives {name} twice with different values "
                        f"({values[name]!r} and {value!r} via {key!r})")
                values[name] = value
            elif key not in _IGNORED_KEYS:
                extra[key] = value
        if "torch_dtype" not in values and "dtype" in raw:
            values["torch_dtype"] = raw["dtype"]
        missing = [k for k in ("vocab_size", "n_positions", "n_layer", "n_head", "n_embd")
                   if k not in values]
        if missing:
            raise ConfigError(
                "config.json lacks required key(s): " + ", ".join(missing)
                + " (n_positions may be spelled block_size)")
        if values.get("n_inner") is None:
            # src/minigpt_infer/model.py:96: hidden width is 4 * n_embd.
            values["n_inner"] = 4 * int(values["n_embd"])
        if "layer_norm_epsilon" in values:
            values["layer_norm_epsilon"] = float(values["layer_norm_epsilon"])
        if "bias" in values:
            values["bias"] = bool(values["bias"])
        if extra:
            warnings.warn("config.json keys not used by this architecture: "
                          + ", ".join(sorted(extra)), stacklevel=2)
        if architecture is not None:
            values["architecture"] = architecture
        return cls(extra=extra, **values)

    @classmethod
    def from_json(cls, path: str | Path) -> "GPTConfig":
        from .registry import architecture_name

        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        raw = read_config_json(path)
        return cls.from_dict(raw, architecture=architecture_name(raw))

    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        out.pop("extra")
        arch = out.pop("architecture")
        out["architectures"] = [arch]
        out["model_type"] = "minigpt"
        return out

    def save(self, model_dir: str | Path) -> Path:
        model_dir = Path(model_dir)
        model_dir.mkdir(parents=True, exist_ok=True)
        path = model_dir / "config.json"
        path.write_text(json.dumps(self.to_dict(), indent=2) + "\n")
        return path

    def num_parameters(self) -> int:
        c, f, layers = self.n_embd, self.n_inner, self.n_layer
        per_layer = 3 * c * c + c * c + 2 * c * f + 2 * c
        if self.bias:
            per_layer += 3 * c + c + f + c + 2 * c
        total = self.vocab_size * c + self.n_positions * c + layers * per_layer + c
        if self.bias:
            total += c
        return total


def read_config_json(path: str | Path) -> dict[str, Any]:
    path = Path(path)
    if not path.is_file():
        raise ConfigError(f"no config.json at {path}")
    try:
        raw = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw
