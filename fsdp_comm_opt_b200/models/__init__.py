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


def shard_groups(model):
    """Groups of the flat-shard engine in execution order: the embedding, one group per decoder
    block, the head.  Parameters used at both ends of the step (tied output embedding, GPT-2's
    tables and final LayerNorm, which its forward reads functionally) form one persistent group."""
    from ..parallel.flat_shard import GroupSpec

    layers = list(decoder_layers(model))
    blocks = [GroupSpec(f"layers.{i}", [m]) for i, m in enumerate(layers)]
    if hasattr(model, "transformer"):
        t = model.transformer
        return [GroupSpec("root", [t.wte, t.wpe, t.ln_f], persistent=True)] + blocks
    if model.lm_head.weight is model.model.embed_tokens.weight:
        return [GroupSpec("root", [model.model.embed_tokens, model.model.norm, model.lm_head], persistent=True)] + blocks
    return ([GroupSpec("embed", [model.model.embed_tokens], backward_needs_params=False)] + blocks
            + [GroupSpec("head", [model.model.norm, model.lm_head])])
