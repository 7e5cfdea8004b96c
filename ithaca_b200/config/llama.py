"""Typed configuration of the Llama dense decoder, read from ``config.json``.

The reference fills ``HParams`` from GGUF metadata keys inside ``Model::load``
(src/model.h:59-76, src/model.cpp:60-77).  The same numbers are read here from
the keys that a Llama model folder's ``config.json`` carries.  Defaults follow
the reference where it has one: ``num_key_value_heads`` defaults to the head
count (src/model.cpp:64-67), ``head_dim`` to hidden/heads (:71),
``rms_norm_eps`` to 1e-5 (:69), ``rope_theta`` to 10000 (:70),
``max_position_embeddings`` to 4096 (:73).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, need_float as _need_float, need_int as _need_int, token_id_list
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary angles.  ``linear`` divides every
    frequency by ``factor`` (src/model.cpp:231-233).  ``llama3`` divides each
    frequency by a factor that depends on its wavelength; the reference takes
    those per-frequency divisors ready-made from a ``rope_freqs.weight`` tensor
    (src/model.cpp:230, 235), a model folder carries the rule's four numbers."""

    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: 'rope_scaling' must be an object or null, found {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind == "linear":
            f = _need_float(d, "factor")
            if f <= 0:
                raise ConfigError(f"config.json: rope_scaling.factor must be > 0, found {f}")
            return RopeScaling("linear", factor=f)
        if kind == "llama3":
            f = _need_float(d, "factor")
            lo = _need_float(d, "low_freq_factor")
            hi = _need_float(d, "high_freq_factor")
            orig = _need_int(d, "original_max_position_embeddings")
            if f <= 0 or lo <= 0 or hi <= lo:
                raise ConfigError(
                    "config.json: rope_scaling (llama3) needs factor > 0 and 0 < low_freq_factor < high_freq_factor, "
                    f"found factor={f} low={lo} high={hi}")
            return RopeScaling("llama3", f, lo, hi, orig)
        raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (supported: llama3, linear, default)")

    def to_dict(self) -> Dict[str, Any]:
        if self.rope_type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {"rope_type": self.rope_type, "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    sliding_window: Optional[int]
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]
    torch_dtype: str
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures") or [cls.ARCHITECTURE]
        hidden = _need_int(d, "hidden_size")
        heads = _need_int(d, "num_attention_heads")
        kv = _need_int(d, "num_key_value_heads", heads)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        head_dim = _need_int({"head_dim": head_dim}, "head_dim")
        if heads % kv:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even (rotary pairs)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported by this architecture (supported: silu)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key, False):
                raise ConfigError(f"config.json: {key}=true is not supported")
        prf = d.get("partial_rotary_factor", 1.0)
        if prf not in (None, 1, 1.0):
            raise ConfigError(f"config.json: partial_rotary_factor {prf!r} is not supported (the whole head is rotated)")
        eps = _need_float(d, "rms_norm_eps", 1e-5)
        if eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, found {eps}")
        # newer model folders carry the rotary numbers in one object, "rope_parameters": the base beside the scaling rule
        rope = d.get("rope_parameters")
        if rope is not None and not isinstance(rope, dict):
            raise ConfigError(f"config.json: 'rope_parameters' must be an object, found {rope!r}")
        scaling = d.get("rope_scaling") if d.get("rope_scaling") is not None else rope
        theta = _need_float(rope, "rope_theta", 10000.0) if rope and "rope_theta" in rope else _need_float(d, "rope_theta", 10000.0)
        if theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be > 0, found {theta}")
        eos_ids: Tuple[int, ...] = token_id_list(d.get("eos_token_id"), "eos_token_id")
        # The reference never windows the layers of this architecture (only other families get a window,
        # src/model.cpp:147), and folders of window-trained relatives that carry this architecture's name still
        # hold a "sliding_window" number.  So the key alone changes nothing; the window applies only when the
        # folder also says "use_sliding_window": true.
        use_window = d.get("use_sliding_window", False)
        if not isinstance(use_window, bool):
            raise ConfigError(f"config.json: 'use_sliding_window' must be true or false, found {use_window!r}")
        window = _need_int(d, "sliding_window") if use_window and d.get("sliding_window") is not None else None
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"config.json: torch_dtype {dtype!r} is not supported (bfloat16, float32, float16)")
        known = {
            "architectures", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim", "hidden_act",
            "attention_bias", "mlp_bias", "partial_rotary_factor", "rms_norm_eps", "rope_theta", "eos_token_id",
            "sliding_window", "use_sliding_window", "torch_dtype", "dtype", "vocab_size", "num_hidden_layers", "intermediate_size",
            "rope_scaling", "rope_parameters", "max_position_embeddings", "tie_word_embeddings", "bos_token_id",
        }
        return cls(
            architecture=str(archs[0]),
            vocab_size=_need_int(d, "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_need_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            intermediate_size=_need_int(d, "intermediate_size"),
            rms_norm_eps=eps,
            rope_theta=theta,
            rope_scaling=RopeScaling.from_dict(scaling),
            max_position_embeddings=_need_int(d, "max_position_embeddings", 4096),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            sliding_window=window,
            eos_token_ids=eos_ids,
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=dtype,
            extra={k: v for k, v in d.items() if k not in known},
        )

    @classmethod
    def from_json_file(cls, path: str) -> "LlamaConfig":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
            d["use_sliding_window"] = True
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # -- the architecture-neutral description --------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """Layer order per block as the reference runs it: input norm, q/k/v,
        rotary, cache write, attention, output projection, residual, FFN norm,
        SwiGLU, residual (src/model.cpp:1460-1565)."""
        d, nh, nkv, hd, ff = (self.hidden_size, self.num_attention_heads, self.num_key_value_heads,
                              self.head_dim, self.intermediate_size)
        position = PartSpec("rotary", {
            "rotary_dim": hd, "theta": self.rope_theta, "pairing": "half",
            "scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position": self.max_position_embeddings,
        })
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            layers.append(BlockSpec(
                kind="prenorm",
                mixer=PartSpec("attention", {
                    "hidden_size": d, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd,
                    "window": self.sliding_window, "scale": None,
                }, {"q": f"{p}.self_attn.q_proj.weight", "k": f"{p}.self_attn.k_proj.weight",
                    "v": f"{p}.self_attn.v_proj.weight", "o": f"{p}.self_attn.o_proj.weight"}),
                feed_forward=PartSpec("gated_mlp", {
                    "hidden_size": d, "intermediate_size": ff, "activation": "silu",
                }, {"gate": f"{p}.mlp.gate_proj.weight", "up": f"{p}.mlp.up_proj.weight",
                    "down": f"{p}.mlp.down_proj.weight"}),
                norms={
                    "mixer": PartSpec("rmsnorm", {"size": d, "eps": self.rms_norm_eps},
                                      {"weight": f"{p}.input_layernorm.weight"}),
                    "feed_forward": PartSpec("rmsnorm", {"size": d, "eps": self.rms_norm_eps},
                                             {"weight": f"{p}.post_attention_layernorm.weight"}),
                },
                position=position,
            ))
        head_weights = {"weight": "model.embed_tokens.weight" if self.tie_word_embeddings else "lm_head.weight"}
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": d, "scale": 1.0},
                               {"weight": "model.embed_tokens.weight"}),
            layers=tuple(layers),
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=PartSpec("rmsnorm", {"size": d, "eps": self.rms_norm_eps}, {"weight": "model.norm.weight"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": d,
                                      "tied": self.tie_word_embeddings}, head_weights),
            max_position=self.max_position_embeddings,
            stop_token_ids=self.eos_token_ids,
            aliases={"lm_head.weight": "model.embed_tokens.weight"} if self.tie_word_embeddings else {},
        )
