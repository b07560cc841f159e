"""Qwen3 dense (``Qwen3ForCausalLM``): its config.json keys and its description as parts.

Keys, defaults and checks follow nanovllm/models/qwen3.py:128-144 and :202-203.  Two
defaults differ on purpose: ``attention_bias`` absent means false here (the reference
treats absent as true and then drops the q/k norms, nanovllm/models/qwen3.py:133,68-70, which
no Qwen3 checkpoint uses), and true is refused; ``rope_theta`` may also sit inside a
``rope_scaling`` / ``rope_parameters`` object, which then wins (nanovllm/models/qwen3.py:54-55).
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import ConfigError, ModelConfig, parse_dtype, take
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartUse, part

ARCHITECTURE = "Qwen3ForCausalLM"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"

    @classmethod
    def from_json_dict(cls, raw: dict) -> "Qwen3Config":
        hidden = take(raw, "hidden_size", int)
        heads = take(raw, "num_attention_heads", int)
        kv_heads = take(raw, "num_key_value_heads", int, heads)
        if heads <= 0 or kv_heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: hidden_size and head counts must be positive")
        head_dim = take(raw, "head_dim", int, None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: no head_dim given and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be positive and even (rotary pairs)")
        act = take(raw, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        if take(raw, "attention_bias", bool, False):
            raise ConfigError("config.json: attention_bias=true is not supported (Qwen3 checkpoints use q/k norms "
                              "and no bias)")
        theta = take(raw, "rope_theta", float, 1000000.0)
        for key in ("rope_scaling", "rope_parameters"):
            sub = raw.get(key)
            if isinstance(sub, dict) and sub.get("rope_theta") is not None:
                theta = float(sub["rope_theta"])
        dtype_name = raw.get("torch_dtype", raw.get("dtype"))
        if dtype_name is None:
            raise ConfigError("config.json: neither 'torch_dtype' nor 'dtype' is given")
        eos = raw.get("eos_token_id")
        if isinstance(eos, list):
            raise ConfigError("config.json: several eos_token_id values are not supported")
        layers = take(raw, "num_hidden_layers", int)
        vocab = take(raw, "vocab_size", int)
        inter = take(raw, "intermediate_size", int)
        max_pos = take(raw, "max_position_embeddings", int)
        if layers <= 0 or vocab <= 0 or inter <= 0 or max_pos <= 0:
            raise ConfigError("config.json: num_hidden_layers, vocab_size, intermediate_size and "
                              "max_position_embeddings must be positive")
        return cls(
            architecture=ARCHITECTURE, model_type=take(raw, "model_type", str, "qwen3"),
            vocab_size=vocab, hidden_size=hidden, max_position_embeddings=max_pos,
            dtype=parse_dtype(dtype_name), eos_token_id=eos if isinstance(eos, int) and not isinstance(eos, bool) else None,
            num_hidden_layers=layers, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
            intermediate_size=inter, rms_norm_eps=take(raw, "rms_norm_eps", float, 1e-6), rope_theta=theta,
            tie_word_embeddings=take(raw, "tie_word_embeddings", bool, False), attention_bias=False, hidden_act=act)

    def to_json_dict(self) -> dict:
        return {
            "architectures": [ARCHITECTURE], "model_type": self.model_type,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "hidden_act": self.hidden_act,
            "vocab_size": self.vocab_size, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings, "attention_bias": False,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": str(self.dtype).replace("torch.", ""),
            **({"eos_token_id": self.eos_token_id} if self.eos_token_id is not None else {}),
        }


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    """Qwen3 as data: every layer is the same pre-norm block of GQA attention and SwiGLU, run once in order."""
    rope = part("rope", theta=cfg.rope_theta, rotary_dim=cfg.head_dim, max_position=cfg.max_position_embeddings)
    mixer = part("gqa_attention", num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                 head_dim=cfg.head_dim, qk_norm_eps=cfg.rms_norm_eps, position=rope)
    ffn = part("swiglu", intermediate_size=cfg.intermediate_size)
    norm = part("rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps)
    layers = tuple(
        LayerSpec(block=part("prenorm_residual"),
                  mixer=PartUse(mixer, f"model.layers.{i}.self_attn."),
                  mixer_norm=PartUse(norm, f"model.layers.{i}.input_layernorm."),
                  ffn=PartUse(ffn, f"model.layers.{i}.mlp."),
                  ffn_norm=PartUse(norm, f"model.layers.{i}.post_attention_layernorm."))
        for i in range(cfg.num_hidden_layers))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartUse(part("token_embedding", vocab_size=cfg.vocab_size), "model.embed_tokens."),
        layers=layers, order=tuple(LayerRun(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartUse(norm, "model.norm."),
        head=PartUse(part("lm_head", vocab_size=cfg.vocab_size, tied=cfg.tie_word_embeddings), "lm_head."),
        # a tied checkpoint may still carry the head's copy of the table
        ignored_checkpoint_tensors=("lm_head.weight",) if cfg.tie_word_embeddings else ())


register_architecture(ARCHITECTURE, model_types=("qwen3",), parse_config=Qwen3Config.from_json_dict,
                      build_spec=build_spec)
