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


def get_config(name: str) -> ModelConfig:
    if name not in SHAPES:
        raise KeyError(f"unknown model shape {name!r}; known: {sorted(SHAPES)}")
    return SHAPES[name]
