"""Typed configuration of the Qwen2.5 dense architecture (`Qwen2ForCausalLM`).

Every size and constant is read from the model folder's `config.json`; nothing
here carries a default for a value that the file is expected to give.  The keys
are the ones the reference reads (somi_inference/models/qwen2_adapter.py:205-225:
vocab_size, hidden_size, intermediate_size, num_hidden_layers,
num_attention_heads, num_key_value_heads, max_position_embeddings, rms_norm_eps,
rope_parameters.rope_theta) plus the ones it leaves unread but the architecture
defines: head_dim, tie_word_embeddings, hidden_act and the three sliding-window
fields.  The reference derives head_dim as hidden_size // num_attention_heads
(somi_inference/entrypoints/llm.py:101) and always ties the head to the embedding
(somi_inference/models/qwen2_adapter.py:60-62); here an explicit `head_dim`
wins over the quotient and `tie_word_embeddings` is honoured.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

ARCHITECTURE = "Qwen2ForCausalLM"


class ConfigError(ValueError):
    """A config.json that lacks a key, or holds a value the engine refuses."""


_REQUIRED_INT = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "max_position_embeddings")


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    hidden_act: str
    use_sliding_window: bool
    sliding_window: int | None
    max_window_layers: int | None
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    torch_dtype: str | None = None

    architecture = ARCHITECTURE

    # ---------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen2Config":
        missing = [k for k in _REQUIRED_INT if k not in d]
        if "rms_norm_eps" not in d:
            missing.append("rms_norm_eps")
        rope = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope.get("rope_theta"))
        if theta is None:
            missing.append("rope_theta (or rope_parameters.rope_theta)")
        if "tie_word_embeddings" not in d:
            missing.append("tie_word_embeddings")
        if missing:
            raise ConfigError("config.json lacks: " + ", ".join(missing))
        for k in _REQUIRED_INT:
            if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] <= 0:
                raise ConfigError(f"config.json: {k} must be a positive integer, got {d[k]!r}")
        for scaling in (d.get("rope_scaling"), rope):
            if isinstance(scaling, dict):
                kind = scaling.get("rope_type", scaling.get("type"))
                if kind not in (None, "default"):
                    raise ConfigError(f"config.json: rope scaling {kind!r} is not supported")
        heads = d["num_attention_heads"]
        head_dim = d.get("head_dim")
        if head_dim is None:
            if d["hidden_size"] % heads:
                raise ConfigError("config.json: hidden_size is not divisible by "
                                  "num_attention_heads and no head_dim is given")
            head_dim = d["hidden_size"] // heads
        use_window = bool(d.get("use_sliding_window", False))
        cfg = cls(
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"],
            num_hidden_layers=d["num_hidden_layers"], num_attention_heads=heads,
            num_key_value_heads=d["num_key_value_heads"], head_dim=int(head_dim),
            max_position_embeddings=d["max_position_embeddings"],
            rms_norm_eps=float(d["rms_norm_eps"]), rope_theta=float(theta),
            tie_word_embeddings=bool(d["tie_word_embeddings"]),
            hidden_act=str(d.get("hidden_act", "silu")),
            use_sliding_window=use_window,
            sliding_window=d.get("sliding_window"),
            max_window_layers=d.get("max_window_layers"),
            bos_token_id=d.get("bos_token_id"), eos_token_id=d.get("eos_token_id"),
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "Qwen2Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "qwen2"
        return {k: v for k, v in d.items() if v is not None}

    # ------------------------------------------------------------- validation
    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotary encoding")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0.0:
            raise ConfigError("rope_theta must be positive")
        if self.use_sliding_window:
            if not isinstance(self.sliding_window, int) or self.sliding_window <= 0:
                raise ConfigError("use_sliding_window is set but sliding_window is not a positive integer")
            if not isinstance(self.max_window_layers, int) or self.max_window_layers < 0:
                raise ConfigError("use_sliding_window is set but max_window_layers is not given")

    # ------------------------------------------------------------ layer kinds
    def layer_window(self, layer: int) -> int | None:
        """Window of `layer`, or None for attention over all keys.

        The reference never passes a window to its attention
        (somi_inference/models/qwen2.py:262,272,318-320), i.e. runs with the
        fields off.  When `use_sliding_window` is true the architecture's rule
        applies: layers with index >= max_window_layers see only the last
        `sliding_window` keys (the query's own position included).
        """
        if self.use_sliding_window and layer >= int(self.max_window_layers):
            return int(self.sliding_window)
        return None

    def to_model_spec(self) -> ModelSpec:
        """Layers, parts and tensor names of this model (names as in the weight file).

        The reference renames the file's tensors to its own module names
        (somi_inference/models/qwen2_adapter.py:149-189); here the file's names
        are the canonical ones and every part is told its own.
        """
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps,
                                        "names": {"weight": name}})
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "qkv_bias": True,    # fixed by the architecture (qwen2.py:268-270)
                "out_bias": False,   # (qwen2.py:271)
                "window": self.layer_window(i),
                "position": PartSpec("rope", {"head_dim": self.head_dim,
                                              "theta": self.rope_theta,
                                              "max_positions": self.max_position_embeddings}),
                "names": {"q_weight": f"{p}.self_attn.q_proj.weight",
                          "k_weight": f"{p}.self_attn.k_proj.weight",
                          "v_weight": f"{p}.self_attn.v_proj.weight",
                          "o_weight": f"{p}.self_attn.o_proj.weight",
                          "q_bias": f"{p}.self_attn.q_proj.bias",
                          "k_bias": f"{p}.self_attn.k_proj.bias",
                          "v_bias": f"{p}.self_attn.v_proj.bias"},
            })
            ff = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                     "intermediate_size": self.intermediate_size,
                                     "names": {"gate_weight": f"{p}.mlp.gate_proj.weight",
                                               "up_weight": f"{p}.mlp.up_proj.weight",
                                               "down_weight": f"{p}.mlp.down_proj.weight"}})
            layers.append(LayerSpec(
                prefix=p, mixer=mixer, feed_forward=ff,
                norms={"mixer": norm(f"{p}.input_layernorm.weight"),
                       "feed_forward": norm(f"{p}.post_attention_layernorm.weight")},
                arrangement="pre_norm"))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.hidden_size,
            vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size,
                                                   "hidden_size": self.hidden_size,
                                                   "names": {"weight": "model.embed_tokens.weight"}}),
            layers=tuple(layers),
            schedule=tuple(RunSpec(i) for i in range(self.num_hidden_layers)),
            final_norm=norm("model.norm.weight"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size,
                                      "hidden_size": self.hidden_size,
                                      "tied": self.tie_word_embeddings,
                                      "names": {"weight": "lm_head.weight",
                                                "tied_to": "model.embed_tokens.weight"}}),
        )
        spec.validate()
        return spec
