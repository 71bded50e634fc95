"""LlamaConfig: the typed configuration of LlamaForCausalLM.

Keys, requiredness and defaults follow the reference's ModelConfig
(crates/vllm-models/src/config.rs:11-98): required hidden_size,
num_attention_heads, num_hidden_layers, intermediate_size, vocab_size;
defaults max_position_embeddings 4096, rope_theta 10000.0, rms_norm_eps 1e-5,
num_key_value_heads = num_attention_heads.  Keys the reference cannot read but
the architecture needs are added: head_dim, tie_word_embeddings, rope_scaling
(crates/vllm-models/src/llama/model.rs:49 hard-sets it to None), and
eos_token_id as an integer or a list.  ``hidden_act``, ``attention_bias`` and
``mlp_bias`` are read so that a checkpoint the parts cannot run is refused
here: the feed-forward computes SiLU and nothing else
(crates/vllm-models/src/llama/architecture.rs:82), and no projection adds a bias.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class RopeScaling:
    """rope_scaling of type "llama3"."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_reader(r: KeyReader | None) -> "RopeScaling | None":
        if r is None:
            return None
        kind = r.string("rope_type", None) or r.string("type", None)
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"{r.where}: rope_type {kind!r} is not supported (known: 'llama3', 'default')")
        s = RopeScaling(
            rope_type=kind,
            factor=r.number("factor", positive=True),
            low_freq_factor=r.number("low_freq_factor", positive=True),
            high_freq_factor=r.number("high_freq_factor", positive=True),
            original_max_position_embeddings=r.integer("original_max_position_embeddings", minimum=1),
        )
        if not s.high_freq_factor > s.low_freq_factor:
            raise ConfigError(f"{r.where}: high_freq_factor must exceed low_freq_factor")
        return s


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    num_hidden_layers: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 4096
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    bos_token_id: int | None = None
    eos_token_id: tuple = field(default_factory=tuple)
    torch_dtype: str | None = None

    ARCHITECTURE = "LlamaForCausalLM"

    @staticmethod
    def from_dict(data: dict, where: str = "config.json") -> "LlamaConfig":
        r = KeyReader(data, where)
        archs = data.get("architectures") or [LlamaConfig.ARCHITECTURE]
        hidden = r.integer("hidden_size", minimum=1)
        nh = r.integer("num_attention_heads", minimum=1)
        nkv = r.integer("num_key_value_heads", nh, minimum=1)
        head_dim = r.integer("head_dim", None, minimum=1)
        act = r.string("hidden_act", "silu")
        if act not in ("silu", "swish"):
            raise ConfigError(f"{where}: hidden_act {act!r} is not supported: the feed-forward computes 'silu'")
        for key in ("attention_bias", "mlp_bias"):
            if r.boolean(key, False):
                raise ConfigError(f"{where}: {key} is true, but the projections here add no bias")
        if head_dim is None:
            if hidden % nh:
                raise ConfigError(
                    f"{where}: hidden_size {hidden} is not a multiple of num_attention_heads {nh} "
                    "and no head_dim is given")
            head_dim = hidden // nh
        cfg = LlamaConfig(
            architecture=archs[0],
            hidden_size=hidden,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            intermediate_size=r.integer("intermediate_size", minimum=1),
            vocab_size=r.integer("vocab_size", minimum=1),
            max_position_embeddings=r.integer("max_position_embeddings", 4096, minimum=1),
            rope_theta=r.number("rope_theta", 10000.0, positive=True),
            rope_scaling=RopeScaling.from_reader(r.obj("rope_scaling")),
            rms_norm_eps=r.number("rms_norm_eps", 1e-5, positive=True),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            bos_token_id=r.integer("bos_token_id", None),
            eos_token_id=r.int_list("eos_token_id", ()),
            torch_dtype=r.string("torch_dtype", None),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{where}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"{where}: head_dim {self.head_dim} must be even for rotary embedding")

    def to_dict(self) -> dict:
        """The config.json content that from_dict reads back to this object."""
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "llama"
        if self.rope_scaling is None:
            d["rope_scaling"] = None
        d["eos_token_id"] = list(self.eos_token_id) if self.eos_token_id else None
        if d["torch_dtype"] is None:
            d["torch_dtype"] = "bfloat16"
        return d
