"""Typed configuration of the Qwen2 dense decoder, read from ``config.json``.

Takes the place of ``LlamaConfig`` / ``LlamaConfig.from_hf`` in
davidjoyme/flashdecode-cuda (config.py:49-137) but parses the JSON text itself
instead of a transformers config object, and checks the keys the reference
never reads (``hidden_act``, the sliding-window keys) instead of ignoring
them.  No size has a default here except where the reference defines one
(``head_dim`` = hidden/heads, config.py:122; ``tie_word_embeddings`` false,
config.py:67).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """config.json misses a key, or a key has a value the architecture cannot take."""


_REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "vocab_size", "rms_norm_eps", "max_position_embeddings")


@dataclass
class Qwen2Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Optional[Any] = None
    bos_token_id: Optional[int] = None
    # Qwen2 checkpoints carry q/k/v biases without a config key for them; the
    # loader decides from the tensors present (engine/loader.py:29-33 of the
    # reference).  ``attention_bias`` in config.json, when present, must agree.
    attention_bias: Optional[bool] = None
    architecture: str = "Qwen2ForCausalLM"
    extra: Dict[str, Any] = field(default_factory=dict)

    # ------------------------------------------------------------------
    @property
    def num_kv_groups(self) -> int:
        """Query heads per KV head (config.py:75-79 of the reference)."""
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """Sliding window of a layer (keys a query sees, itself included) or
        None: with ``use_sliding_window``, layers from ``max_window_layers`` on."""
        if not self.use_sliding_window:
            return None
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return self.sliding_window if layer >= first else None

    def stop_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]

    # ------------------------------------------------------------------
    @staticmethod
    def _rope(cfg: Dict[str, Any]):
        """(theta, scaling) from flat ``rope_theta`` or ``rope_parameters`` /
        ``rope_scaling`` dictionaries (config.py:80-118 of the reference).
        ``rope_type`` absent or "default" means plain rotation; any other type
        is refused rather than silently ignored."""
        params = cfg.get("rope_parameters")
        if not isinstance(params, dict):
            params = cfg.get("rope_scaling")
        if not isinstance(params, dict):
            params = {}
        theta = cfg.get("rope_theta")
        if theta is None:
            theta = params.get("rope_theta")
        if theta is None:
            raise ConfigError("config.json has no rope_theta (looked at rope_theta, "
                              "rope_parameters.rope_theta, rope_scaling.rope_theta)")
        rope_type = params.get("rope_type") or params.get("type")
        if rope_type not in (None, "default"):
            raise ConfigError(f"rope scaling of type {rope_type!r} is not part of this architecture here")
        return float(theta)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in cfg]
        if missing:
            raise ConfigError(f"config.json misses required keys: {missing}")
        n_q = int(cfg["num_attention_heads"])
        hidden = int(cfg["hidden_size"])
        head_dim = cfg.get("head_dim")
        if head_dim is None:
            if n_q <= 0 or hidden % n_q:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {n_q} "
                                  f"and no head_dim is given")
            head_dim = hidden // n_q
        arch = (cfg.get("architectures") or ["Qwen2ForCausalLM"])[0]
        known = set(cls.__dataclass_fields__) | {"architectures", "rope_parameters", "rope_scaling"}
        out = cls(
            hidden_size=hidden,
            intermediate_size=int(cfg["intermediate_size"]),
            num_hidden_layers=int(cfg["num_hidden_layers"]),
            num_attention_heads=n_q,
            num_key_value_heads=int(cfg["num_key_value_heads"]),
            head_dim=int(head_dim),
            vocab_size=int(cfg["vocab_size"]),
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            rope_theta=cls._rope(cfg),
            max_position_embeddings=int(cfg["max_position_embeddings"]),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            hidden_act=str(cfg.get("hidden_act", "silu")),
            use_sliding_window=bool(cfg.get("use_sliding_window", False)),
            sliding_window=None if cfg.get("sliding_window") is None else int(cfg["sliding_window"]),
            max_window_layers=None if cfg.get("max_window_layers") is None else int(cfg["max_window_layers"]),
            eos_token_id=cfg.get("eos_token_id"),
            bos_token_id=cfg.get("bos_token_id"),
            attention_bias=cfg.get("attention_bias"),
            architecture=arch,
            extra={k: v for k, v in cfg.items() if k not in known},
        )
        out.validate()
        return out

    def validate(self) -> None:
        pos = {k: getattr(self, k) for k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                             "num_attention_heads", "num_key_value_heads", "head_dim",
                                             "vocab_size", "max_position_embeddings")}
        bad = {k: v for k, v in pos.items() if v <= 0}
        if bad:
            raise ConfigError(f"sizes must be positive: {bad}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotate-half position encoding")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act {self.hidden_act!r}: this architecture's feed-forward is SiLU-gated")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("use_sliding_window is set but sliding_window is not a positive number")

    def to_dict(self) -> Dict[str, Any]:
        """A ``config.json`` dictionary that parses back to this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_act": self.hidden_act,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
        }
        for k in ("sliding_window", "max_window_layers", "eos_token_id", "bos_token_id", "attention_bias"):
            if getattr(self, k) is not None:
                d[k] = getattr(self, k)
        for k, v in self.extra.items():
            d.setdefault(k, v)
        return d

    def summary(self) -> str:
        """One line in the manner of ``LlamaConfig.summary`` (config.py:139-145)."""
        return (f"layers={self.num_hidden_layers} hidden={self.hidden_size} "
                f"q_heads={self.num_attention_heads} kv_heads={self.num_key_value_heads} "
                f"(GQA group={self.num_kv_groups}) head_dim={self.head_dim} "
                f"intermediate={self.intermediate_size} vocab={self.vocab_size} "
                f"rope_theta={self.rope_theta} eps={self.rms_norm_eps} "
                f"tied={'yes' if self.tie_word_embeddings else 'no'} "
                f"window={'%s from layer %s' % (self.sliding_window, self.max_window_layers) if self.use_sliding_window else 'off'}")
