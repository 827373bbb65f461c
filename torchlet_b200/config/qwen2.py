"""Typed configuration of Qwen2.5 dense (``Qwen2ForCausalLM``).

Keys and defaults are those the reference reads
(v10_triton_paged_gqa/model/qwen2_5.py:14-18 rope_theta, :25-36 sizes/eps/bias,
:75 tie_word_embeddings; v10_triton_paged_gqa/layer/gqa.py:26-37 head checks).
Keys the reference never reads are parsed and checked instead of ignored: rope
scaling is refused, the sliding-window keys select a windowed mixer per layer.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, fields
from typing import Optional

from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry

_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "max_position_embeddings",
)


@register_architecture("Qwen2ForCausalLM")
@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    max_position_embeddings: int
    num_key_value_heads: Optional[int] = None  # default: num_attention_heads
    head_dim: Optional[int] = None  # default: hidden_size // num_attention_heads
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    attention_bias: bool = True
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    hidden_act: str = "silu"
    torch_dtype: Optional[str] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None

    architecture = "Qwen2ForCausalLM"

    def __post_init__(self) -> None:
        if self.num_key_value_heads is None:
            object.__setattr__(self, "num_key_value_heads", self.num_attention_heads)
        if self.head_dim is None:
            if self.hidden_size % self.num_attention_heads:
                raise ValueError(
                    f"hidden_size {self.hidden_size} is not divisible by "
                    f"num_attention_heads {self.num_attention_heads} and no head_dim is given"
                )
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        for name in _REQUIRED + ("num_key_value_heads", "head_dim"):
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer, got {value!r}")
        if self.num_key_value_heads > self.num_attention_heads:
            raise ValueError("num_key_value_heads must not exceed num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for split-half rotation")
        if not self.rms_norm_eps > 0:
            raise ValueError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ValueError("rope_theta must be positive")
        if self.hidden_act != "silu":
            raise ValueError(f"hidden_act {self.hidden_act!r} is not supported (SwiGLU needs 'silu')")
        if self.use_sliding_window:
            if not isinstance(self.sliding_window, int) or self.sliding_window <= 0:
                raise ValueError("use_sliding_window needs a positive sliding_window")
            if self.max_window_layers is None:
                object.__setattr__(self, "max_window_layers", 0)
            if not 0 <= self.max_window_layers <= self.num_hidden_layers:
                raise ValueError("max_window_layers must lie in [0, num_hidden_layers]")

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        missing = [key for key in _REQUIRED if key not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if raw.get("rope_scaling") not in (None, {}):
            raise ValueError("rope_scaling is not supported")
        known = {f.name for f in fields(cls)}
        values = {key: raw[key] for key in known if key in raw and raw[key] is not None}
        rope_parameters = raw.get("rope_parameters")
        if isinstance(rope_parameters, dict):
            if rope_parameters.get("rope_type", "default") not in ("default", None):
                raise ValueError("only the default rope_type is supported")
            if "rope_theta" in rope_parameters:
                values["rope_theta"] = rope_parameters["rope_theta"]
        if "torch_dtype" not in values and isinstance(raw.get("dtype"), str):
            values["torch_dtype"] = raw["dtype"]
        eos = raw.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            values["eos_token_id"] = int(eos[0]) if eos else None
        for key in ("rms_norm_eps", "rope_theta"):
            if key in values:
                values[key] = float(values[key])
        return cls(**values)

    def to_dict(self) -> dict:
        out = {key: value for key, value in asdict(self).items() if value is not None}
        out["architectures"] = [self.architecture]
        out["model_type"] = "qwen2"
        return out

    # ------------------------------------------------------------ structure
    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer's mixer: the first ``max_window_layers`` layers see all
        keys, the rest only the last ``sliding_window`` ones, when the window is on."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        feed_forward = PartSpec(
            "swiglu", {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}
        )
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec(
                "attention",
                {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qkv_bias": bool(self.attention_bias),
                    "o_bias": False,
                    "window": self.layer_window(i),
                    "scale": None,  # None: head_dim ** -0.5
                    "positions": PartSpec(
                        "rotary_split_half",
                        {"head_dim": self.head_dim, "theta": float(self.rope_theta)},
                    ),
                },
            )
            layers.append(
                LayerSpec(
                    prefix=f"model.layers.{i}.",
                    block="pre_norm",
                    mixer=mixer,
                    feed_forward=feed_forward,
                    norms=(NormSlot("mixer_norm", norm, "input_layernorm."),
                           NormSlot("feed_forward_norm", norm, "post_attention_layernorm.")),
                    # the checkpoint's names (v10_triton_paged_gqa/layer/transformer_block.py:20-35)
                    mixer_prefix="self_attn.",
                    feed_forward_prefix="mlp.",
                )
            )
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_position_embeddings=self.max_position_embeddings,
            embedding_name="model.embed_tokens.weight",
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=norm,
            final_norm_prefix="model.norm.",
            lm_head_name="lm_head.weight",
            tie_word_embeddings=bool(self.tie_word_embeddings),
        )
        spec.validate()
        return spec
