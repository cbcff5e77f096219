"""Model shapes.  The reference builds whatever HF ``AutoConfig`` names (train.py:86-88) and
discovers decoder layers at ``model.model.layers`` (Llama-like) or ``model.transformer.h``
(GPT-2, the family of its shipped run script); both families exist here as own modules with
those attribute paths, and the named shapes below replace the hub lookup."""
from __future__ import annotations

from dataclasses import dataclass, asdict


@dataclass
class ModelConfig:
    family: str = "llama"          # "llama" | "gpt2"
    vocab_size: int = 8192
    d_model: int = 256
    n_layers: int = 2
    n_heads: int = 4
    n_kv_heads: int = 4
    ffn: int = 1024
    max_seq: int = 4096
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = False
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def to_dict(self) -> dict:
        return asdict(self)

    def num_params(self) -> int:
        d, f, v, L = self.d_model, self.ffn, self.vocab_size, self.n_layers
        hd = self.head_dim
        if self.family == "llama":
            per = d * (self.n_heads + 2 * self.n_kv_heads) * hd + d * d + 3 * d * f + 2 * d
            return L * per + v * d * (1 if self.tie_embeddings else 2) + d
        per = (3 * d * d + 3 * d) + (d * d + d) + (2 * d * f + f + d) + 4 * d
        return L * per + v * d + self.max_seq * d + 2 * d


SHAPES: dict[str, ModelConfig] = {
    # CPU/gloo plumbing run
    "tiny": ModelConfig("llama", 8192, 256, 2, 4, 4, 1024, 4096, 10000.0),
    # GPU smoke: head_dim 128, every GEMM dim a multiple of the tcgen05 tile
    "small": ModelConfig("llama", 32768, 1024, 4, 8, 2, 4096, 4096, 500000.0),
    "llama3-8b": ModelConfig("llama", 128256, 4096, 32, 32, 8, 14336, 8192, 500000.0),
    "llama2-13b": ModelConfig("llama", 32000, 5120, 40, 40, 40, 13824, 4096, 10000.0),
    "34b": ModelConfig("llama", 32000, 8192, 48, 64, 8, 22016, 16384, 1000000.0),
    "gpt2-tiny": ModelConfig("gpt2", 8192, 256, 2, 4, 4, 1024, 1024, tie_embeddings=True),
    "gpt2-xl": ModelConfig("gpt2", 50257, 1600, 48, 25, 25, 6400, 1024, tie_embeddings=True),
}


# Hub ids the reference's ``-m`` flag is given (reference: run.sh:1, train.py:86-88) -> local shapes.
HUB_ALIASES: dict[str, str] = {
    "openai-community/gpt2-xl": "gpt2-xl",
    "gpt2-xl": "gpt2-xl",
    "meta-llama/meta-llama-3-8b": "llama3-8b",
    "meta-llama/llama-3.1-8b": "llama3-8b",
    "meta-llama/llama-2-13b-hf": "llama2-13b",
    "codellama/codellama-34b-hf": "34b",
}


def config_from_hf_dict(d: dict) -> ModelConfig:
    """A ``config.json`` of a HF Llama- or GPT-2-family checkpoint -> ``ModelConfig``."""
    mt = d.get("model_type", "llama")
    if mt == "gpt2":
        dm = d["n_embd"]
        return ModelConfig("gpt2", d["vocab_size"], dm, d["n_layer"], d["n_head"], d["n_head"],
                           d.get("n_inner") or 4 * dm, d.get("n_positions", 1024),
                           norm_eps=d.get("layer_norm_epsilon", 1e-5), tie_embeddings=True,
                           init_std=d.get("initializer_range", 0.02))
    return ModelConfig("llama", d["vocab_size"], d["hidden_size"], d["num_hidden_layers"], d["num_attention_heads"],
                       d.get("num_key_value_heads", d["num_attention_heads"]), d["intermediate_size"],
                       d.get("max_position_embeddings", 4096), d.get("rope_theta", 10000.0),
                       d.get("rms_norm_eps", 1e-5), bool(d.get("tie_word_embeddings", False)),
                       d.get("initializer_range", 0.02))


def get_config(name: str) -> ModelConfig:
    """A named shape, a hub id of one of them, or a local directory / ``config.json`` in HF format
    (the reference resolves ``-m`` through ``AutoConfig.from_pretrained``, which also reads local
    directories; reference: train.py:86-88)."""
    import json
    import os

    if name in SHAPES:
        return SHAPES[name]
    alias = HUB_ALIASES.get(name.lower())
    if alias is not None:
        return SHAPES[alias]
    path = os.path.join(name, "config.json") if os.path.isdir(name) else name
    if os.path.isfile(path):
        with open(path) as fp:
            return config_from_hf_dict(json.load(fp))
    raise KeyError(f"unknown model {name!r}; known shapes: {sorted(SHAPES)}, hub ids: {sorted(HUB_ALIASES)}, "
                   "or a local directory with a HF config.json")
