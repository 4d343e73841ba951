"""Typed configuration of the Llama architecture, read from config.json.

The keys and their defaults follow the reference's converter
(tools/convert.py:55-80): ``vocab_size``, ``hidden_size``, ``num_hidden_layers``,
``num_attention_heads``, ``num_key_value_heads`` (default: heads), ``head_dim``
(default: hidden // heads), ``intermediate_size``, ``rope_theta`` (10000.0),
``rms_norm_eps`` (1e-6), ``tie_word_embeddings`` (False), ``bos_token_id`` /
``eos_token_id`` (-1; the first element when a list).  The reference rejects any
``rope_scaling`` (tools/convert.py:59-60); here the ``llama3`` rule is accepted and
typed as :class:`RopeScaling`.  The typed fields mirror ``ModelConfig``
(src/model.h:14-31).

No size and no constant of a model lives anywhere else in the package: parts get
them as constructor parameters from this object.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional

from .base import ConfigError, read_config_json  # noqa: F401  (read_config_json is re-exported)


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json for ``rope_type == "llama3"``."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_json(d: dict) -> "RopeScaling":
        kind = d.get("rope_type", d.get("type"))
        if kind != "llama3":  # "default" (no rescaling) is handled by the caller
            raise ConfigError(
                f"rope_scaling of type {kind!r} is not supported (supported: 'llama3')")
        try:
            return RopeScaling(
                rope_type="llama3",
                factor=float(d["factor"]),
                low_freq_factor=float(d["low_freq_factor"]),
                high_freq_factor=float(d["high_freq_factor"]),
                original_max_position_embeddings=int(d["original_max_position_embeddings"]),
            )
        except KeyError as e:
            raise ConfigError(f"rope_scaling lacks the key {e.args[0]!r}") from None


@dataclass(frozen=True)
class LlamaConfig:
    """Hyper-parameters of one Llama / SmolLM2 checkpoint."""

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 2048
    bos_token_id: int = -1
    eos_token_id: int = -1
    rope_scaling: Optional[RopeScaling] = None
    architectures: tuple = ("LlamaForCausalLM",)
    extra: dict = field(default_factory=dict, compare=False)

    architecture_name = "LlamaForCausalLM"

    def __post_init__(self):
        if self.num_key_value_heads is None:
            object.__setattr__(self, "num_key_value_heads", self.num_attention_heads)
        if self.head_dim is None:
            if self.num_attention_heads <= 0 or self.hidden_size % self.num_attention_heads:
                raise ConfigError(
                    "head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        self.validate()

    # derived sizes (src/model.h:29-30)
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def validate(self) -> None:
        pos = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
               "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings")
        for k in pos:
            v = getattr(self, k)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"{k} must be a positive integer, got {v!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta!r}")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps!r}")

    @staticmethod
    def from_json(d: dict) -> "LlamaConfig":
        required = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "intermediate_size")
        missing = [k for k in required if k not in d]
        if missing:
            raise ConfigError("config.json lacks the keys: " + ", ".join(missing))
        eos = d.get("eos_token_id", -1)
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else -1
        bos = d.get("bos_token_id", -1)
        known = set(LlamaConfig.__dataclass_fields__) | {"architectures"}
        scaling = d.get("rope_scaling")
        if scaling and scaling.get("rope_type", scaling.get("type")) == "default":
            scaling = None  # the plain rotary table
        # Options that would change the arithmetic and that this model does not have: the
        # reference's Llama has SiLU only and no biases (src/kernels.cpp:291-298; src/model.cpp:150-164).
        act = d.get("hidden_act", "silu")
        if act not in ("silu", "swish"):
            raise ConfigError(f"hidden_act {act!r} is not supported (the feed-forward is SwiGLU: 'silu')")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"{key} = true is not supported (the projections have no bias)")
        return LlamaConfig(
            vocab_size=d["vocab_size"],
            hidden_size=d["hidden_size"],
            num_hidden_layers=d["num_hidden_layers"],
            num_attention_heads=d["num_attention_heads"],
            intermediate_size=d["intermediate_size"],
            num_key_value_heads=d.get("num_key_value_heads"),
            head_dim=d.get("head_dim"),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            bos_token_id=-1 if bos is None else int(bos),
            eos_token_id=-1 if eos is None else int(eos),
            rope_scaling=RopeScaling.from_json(scaling) if scaling else None,
            architectures=tuple(d.get("architectures", ("LlamaForCausalLM",))),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_json(self) -> dict:
        d = {
            "architectures": list(self.architectures),
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": self.eos_token_id,
            "hidden_act": "silu",
        }
        if self.rope_scaling is not None:
            d["rope_scaling"] = asdict(self.rope_scaling)
        return d
