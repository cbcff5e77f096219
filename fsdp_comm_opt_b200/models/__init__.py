from .config import ModelConfig, SHAPES, get_config
from .llama import LlamaForCausalLM, CausalLMOutput
from .gpt2 import GPT2ForCausalLM


def build_model(cfg: ModelConfig):
    """Instantiate the family named by ``cfg.family`` (on the current default device, e.g. meta)."""
    if cfg.family == "llama":
        return LlamaForCausalLM(cfg)
    if cfg.family == "gpt2":
        return GPT2ForCausalLM(cfg)
    raise ValueError(f"unknown model family {cfg.family!r}")


def decoder_layers(model):
    """Layer discovery with the reference's rule (reference: train.py:99-104)."""
    if hasattr(model, "transformer") and hasattr(model.transformer, "h"):
        return model.transformer.h
    if hasattr(model, "model") and hasattr(model.model, "layers"):
        return model.model.layers
    raise ValueError("Unknown model structure")
