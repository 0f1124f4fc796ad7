"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference parses the same keys into ``SafetensorsLoader::ModelConfig``
(runtime/backends/cuda/inferflux_cuda_executor.h:62-85, parse at
runtime/backends/cuda/inferflux_cuda_executor.cpp:524-604): ``hidden_size``,
``num_hidden_layers``, ``num_attention_heads``, ``num_key_value_heads``,
``head_dim`` (default ``hidden_size / num_attention_heads``),
``intermediate_size``, ``vocab_size``, ``max_position_embeddings``,
``rope_theta`` (default 10000), ``rms_norm_eps`` (default 1e-6),
``model_type`` / ``architectures``, ``hidden_act``, ``torch_dtype``.
It silently keeps defaults when the file cannot be parsed
(inferflux_cuda_executor.cpp:348-351); here every fault is an error.

Keys the reference never reads but the architecture defines
(``tie_word_embeddings``, ``use_sliding_window``, ``sliding_window``,
``max_window_layers``, ``bos_token_id``, ``eos_token_id``) are typed here too.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration."""

    architectures: List[str] = field(default_factory=list)
    model_type: str = ""

    @property
    def architecture(self) -> str:
        if self.architectures:
            return self.architectures[0]
        return self.model_type

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
        return path


def _require_int(d: Dict[str, Any], key: str, minimum: int = 1) -> int:
    if key not in d:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def _opt_number(d: Dict[str, Any], key: str, default: float) -> float:
    v = d.get(key, default)
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """``Qwen2ForCausalLM``: pre-norm RMSNorm decoder, grouped-query attention
    with q/k/v bias, rotate-half rotary positions, SwiGLU feed-forward."""

    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    ARCHITECTURE = "Qwen2ForCausalLM"
    MODEL_TYPE = "qwen2"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2Config":
        archs = d.get("architectures") or []
        if not isinstance(archs, list):
            raise ConfigError("config.json: 'architectures' must be a list")
        model_type = d.get("model_type", "") or ""
        hidden = _require_int(d, "hidden_size")
        heads = _require_int(d, "num_attention_heads")
        # The reference leaves num_key_value_heads at 0 when absent
        # (inferflux_cuda_executor.cpp:537-539); multi-head attention is the
        # meaning of an absent key, so that is the default here.
        kv_heads = _require_int(d, "num_key_value_heads") if "num_key_value_heads" in d else heads
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _require_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by "
                    f"num_attention_heads {heads} and 'head_dim' is not given")
            head_dim = hidden // heads
        rope_scaling = d.get("rope_scaling")
        if rope_scaling not in (None, {}):
            raise ConfigError(
                f"config.json: rope_scaling={rope_scaling!r} is not supported "
                "(only unscaled rotary positions)")
        act = d.get("hidden_act", "silu")
        use_sw = bool(d.get("use_sliding_window", False))
        sw = d.get("sliding_window")
        if sw is not None and (isinstance(sw, bool) or not isinstance(sw, int) or sw < 1):
            raise ConfigError(f"config.json: 'sliding_window' must be a positive integer, got {sw!r}")
        layers = _require_int(d, "num_hidden_layers")
        mwl = d.get("max_window_layers", layers)
        if mwl is None:
            mwl = layers
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architectures=list(archs),
            model_type=model_type,
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_require_int(d, "intermediate_size"),
            vocab_size=_require_int(d, "vocab_size"),
            max_position_embeddings=_require_int(d, "max_position_embeddings"),
            rope_theta=_opt_number(d, "rope_theta", 10000.0),
            rms_norm_eps=_opt_number(d, "rms_norm_eps", 1e-6),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=use_sw,
            sliding_window=sw,
            max_window_layers=int(mwl),
            hidden_act=str(act),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=eos,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary positions")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.rope_theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.use_sliding_window and not self.sliding_window:
            raise ConfigError("use_sliding_window is true but 'sliding_window' is not given")
        if not 0 <= self.max_window_layers:
            raise ConfigError("max_window_layers must be >= 0")

    def window_of_layer(self, layer: int) -> Optional[int]:
        """The attention window of a layer, or None for all keys.

        Layers from ``max_window_layers`` upwards look at the last
        ``sliding_window`` keys (the query's own included) when
        ``use_sliding_window`` is set; the layers below see every key.
        """
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None


def read_config_dict(folder_or_file: str) -> Dict[str, Any]:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    try:
        with open(path) as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def _require_number(d: Dict[str, Any], key: str, where: str = "config.json") -> float:
    if key not in d:
        raise ConfigError(f"{where}: required key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class KunonexLayer:
    """One layer of a Kunonex model: which mixer it has, the mixer's sizes as
    config.json gives them, and the width of its feed-forward (0 = none)."""

    type: str = ""
    mixer: Dict[str, Any] = field(default_factory=dict)
    ff: int = 0
    ff_kind: str = ""


@dataclass(frozen=True)
class KunonexConfig(ModelConfig):
    """``Kunonex``: a decoder whose layers are listed one by one in config.json
    (``layers``: ``type`` = ``mingru`` or ``latent_attention``, the mixer's
    sizes under ``mixer``, the feed-forward under ``mlp`` or null), with a
    stretch of layers (``loop``: ``start``, ``stop``, ``times``) that runs
    several times in a row on the same weights.  Parallel blocks behind one
    layer norm, token shift ahead of the mixer, sinusoidal positions added to
    the embedding, PolyNorm feed-forwards."""

    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    layers: List[KunonexLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0              # 0 = the model has no loop

    ARCHITECTURE = "Kunonex"
    MODEL_TYPE = "kunonex"
    MIXERS = {"mingru": ("width",), "latent_attention": ("heads", "dim", "vdim", "kv_rank", "q_rank", "scale")}
    FF_KINDS = ("dense",)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KunonexConfig":
        width = _require_int(d, "width")
        vocab = _require_int(d, "vocab")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _require_number(norm, "eps", "config.json norm")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"config.json layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = entry.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {sorted(cls.MIXERS)}")
            mixer = entry.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}: 'mixer' must be an object")
            sizes = {}
            for key in cls.MIXERS[kind]:
                if key != "scale":
                    sizes[key] = _require_int(mixer, key)
                elif mixer.get("scale") is None:
                    sizes[key] = float(sizes["dim"]) ** -0.5           # the usual scale where a configuration gives none
                else:
                    sizes[key] = _require_number(mixer, key, where)
            mlp = entry.get("mlp")
            ff, ff_kind = 0, ""
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{where}: 'mlp' must be an object or null")
                ff_kind = mlp.get("kind")
                if ff_kind not in cls.FF_KINDS:
                    raise ConfigError(f"{where}: mlp kind {ff_kind!r} is not one of {list(cls.FF_KINDS)}")
                ff = _require_int(mlp, "ff")
            layers.append(KunonexLayer(type=kind, mixer=sizes, ff=ff, ff_kind=ff_kind or ""))
        start = stop = times = 0
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object or null")
            start, stop = _require_int(loop, "start", 0), _require_int(loop, "stop", 0)
            times = _require_int(loop, "times", 1)
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
        arch = d.get("architecture") or (d.get("architectures") or [cls.ARCHITECTURE])[0]
        cfg = cls(architectures=[str(arch)], model_type=str(d.get("model_type", "") or cls.MODEL_TYPE), width=width,
                  vocab=vocab, norm_eps=eps, logit_scale=_opt_number(d, "logit_scale", 1.0), layers=layers,
                  loop_start=start, loop_stop=stop, loop_times=times)
        if cfg.norm_eps <= 0:
            raise ConfigError(f"norm eps must be positive, got {cfg.norm_eps}")
        return cfg

    # what Engine and the command line read of any model's configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> Optional[int]:
        return None

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration was read from (its own keys)."""
        out: Dict[str, Any] = {
            "architecture": self.architecture, "width": self.width, "vocab": self.vocab,
            "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
            "layers": [{"type": l.type, "mixer": dict(l.mixer),
                        "mlp": {"kind": l.ff_kind, "ff": l.ff} if l.ff else None} for l in self.layers]}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
