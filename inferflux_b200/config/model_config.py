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


def _sub(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None and optional:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclass(frozen=True)
class PemoraxLayer:
    """One layer of a Pemorax model as config.json gives it: the mixer's sizes and constants (checked, defaults
    filled in) and its feed-forward (``None`` = none; ``kind`` ``dense`` with ``ff``, or ``moe`` with ``ff`` of
    one expert, ``experts`` and ``top``)."""

    type: str = ""
    mixer: Dict[str, Any] = field(default_factory=dict)
    mlp: Optional[Dict[str, Any]] = None


@dataclass(frozen=True)
class PemoraxConfig(ModelConfig):
    """``Pemorax``: a decoder whose layers are listed one by one in config.json (``layers``: ``type``, the
    mixer's sizes under ``mixer``, the feed-forward under ``mlp`` or null).  Every sublayer sits between two
    RMS norms.  The mixer ``parallel`` runs a pair of mixers on one input: ``left`` grouped-query
    attention (short convolution on q, k, v, interleaved rotary positions with an optional frequency scaling,
    capped scores, a window that keeps the first tokens, a sink in the softmax, an output gate) and ``right``
    retention (rotate-half positions, a fixed decay per head, a per-head unit norm, a silu gate); their normed
    outputs are averaged.  Feed-forwards are dense (gelu) or routed experts (gated silu)."""

    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    layers: List[PemoraxLayer] = field(default_factory=list)

    ARCHITECTURE = "Pemorax"
    MODEL_TYPE = "pemorax"

    @staticmethod
    def _rot(d: Dict[str, Any], where: str, dim: int) -> Dict[str, Any]:
        rot = _sub(d, "rot", where, optional=True)
        if rot is None:
            return {"dims": 0, "base": 10000.0, "scaling": None}
        dims = _require_int(rot, "dims", 0)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {dim}")
        out = {"dims": dims, "base": _require_number(rot, "base", where + " rot"), "scaling": None}
        if out["base"] <= 1.0:
            raise ConfigError(f"{where}: rot.base must be above 1")
        sc = _sub(rot, "scaling", where + " rot", optional=True)
        if sc is not None:
            out["scaling"] = {k: _require_number(sc, k, where + " rot.scaling") for k in ("factor", "original", "fast", "slow")}
            if min(out["scaling"].values()) <= 0:
                raise ConfigError(f"{where}: the numbers of rot.scaling must be positive")
        return out

    @classmethod
    def _left(cls, m: Dict[str, Any], where: str) -> Dict[str, Any]:
        heads, dim = _require_int(m, "heads"), _require_int(m, "dim")
        out = {"heads": heads, "kv_heads": _require_int(m, "kv_heads") if m.get("kv_heads") is not None else heads,
               "dim": dim, "vdim": _require_int(m, "vdim") if m.get("vdim") is not None else dim,
               "conv": _require_int(m, "conv", 1) if m.get("conv") is not None else 0,
               "scale": _require_number(m, "scale", where) if m.get("scale") is not None else float(dim) ** -0.5,
               "softcap": _require_number(m, "softcap", where) if m.get("softcap") is not None else None,
               "rot": cls._rot(m, where, dim), "mask": None}
        if heads % out["kv_heads"]:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {out['kv_heads']}")
        if out["conv"] > 16:
            raise ConfigError(f"{where}: a convolution of {out['conv']} taps is not supported (at most 16)")
        if out["softcap"] is not None and out["softcap"] <= 0:
            raise ConfigError(f"{where}: softcap must be positive")
        mask = _sub(m, "mask", where, optional=True)
        if mask is not None:
            out["mask"] = {"size": _require_int(mask, "size"),
                           "keep_first": _require_int(mask, "keep_first", 0) if mask.get("keep_first") is not None else 0}
        return out

    @classmethod
    def _right(cls, m: Dict[str, Any], where: str) -> Dict[str, Any]:
        heads, dim = _require_int(m, "heads"), _require_int(m, "dim")
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or any(
                isinstance(x, bool) or not isinstance(x, (int, float)) or not 0.0 < float(x) <= 1.0 for x in decay):
            raise ConfigError(f"{where}: 'decay' must list one number in (0, 1] for each of the {heads} heads")
        return {"heads": heads, "dim": dim, "vdim": _require_int(m, "vdim") if m.get("vdim") is not None else dim,
                "decay": [float(x) for x in decay], "rot": cls._rot(m, where, dim)}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PemoraxConfig":
        width, vocab = _require_int(d, "width"), _require_int(d, "vocab")
        eps = _require_number(_sub(d, "norm", "config.json"), "eps", "config.json norm")
        if eps <= 0:
            raise ConfigError(f"norm eps must be positive, got {eps}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"config.json layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = entry.get("type")
            if kind != "parallel":
                raise ConfigError(f"{where}: type {kind!r} is not one of ['parallel']")
            mixer = _sub(entry, "mixer", where)
            sizes = {"left": cls._left(_sub(mixer, "left", where + " mixer"), where + " mixer.left"),
                     "right": cls._right(_sub(mixer, "right", where + " mixer"), where + " mixer.right")}
            mlp = _sub(entry, "mlp", where, optional=True)
            ff = None
            if mlp is not None:
                ff_kind = mlp.get("kind")
                if ff_kind == "dense":
                    ff = {"kind": "dense", "ff": _require_int(mlp, "ff")}
                elif ff_kind == "moe":
                    router = _sub(mlp, "router", where + " mlp")
                    ff = {"kind": "moe", "ff": _require_int(_sub(mlp, "expert", where + " mlp"), "ff"),
                          "experts": _require_int(router, "experts"), "top": _require_int(router, "top")}
                    if ff["top"] > ff["experts"]:
                        raise ConfigError(f"{where}: router.top {ff['top']} exceeds router.experts {ff['experts']}")
                else:
                    raise ConfigError(f"{where}: mlp kind {ff_kind!r} is not one of ['dense', 'moe']")
            layers.append(PemoraxLayer(type=kind, mixer=sizes, mlp=ff))
        arch = d.get("architecture") or (d.get("architectures") or [cls.ARCHITECTURE])[0]
        return cls(architectures=[str(arch)], model_type=str(d.get("model_type", "") or cls.MODEL_TYPE), width=width,
                   vocab=vocab, norm_eps=eps, layers=layers)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> Optional[int]:
        return None

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration was read from (its own keys)."""
        def rot(r):
            if not r["dims"]:
                return None
            out = {"dims": r["dims"], "base": r["base"]}
            if r["scaling"]:
                out["scaling"] = dict(r["scaling"])
            return out

        def strip(m):
            return {k: v for k, v in m.items() if v is not None}
        layers = []
        for l in self.layers:
            left, right = dict(l.mixer["left"]), dict(l.mixer["right"])
            left["rot"], right["rot"] = rot(left["rot"]), rot(right["rot"])
            if not left["conv"]:
                left["conv"] = None
            mlp = None
            if l.mlp and l.mlp["kind"] == "dense":
                mlp = {"kind": "dense", "ff": l.mlp["ff"]}
            elif l.mlp:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp["ff"]}, "router": {"experts": l.mlp["experts"], "top": l.mlp["top"]}}
            layers.append({"type": l.type, "mixer": {"left": strip(left), "right": strip(right)}, "mlp": mlp})
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                "norm": {"eps": self.norm_eps}, "layers": layers}


@dataclass(frozen=True)
class TekosunLayer:
    """One layer of a Tekosun model as config.json gives it: ``type`` (which mixer), the mixer's sizes and
    constants (checked, defaults filled in) and its feed-forward (``None`` = none; else the experts' and the
    shared expert's sizes and the router's constants)."""

    type: str = ""
    mixer: Dict[str, Any] = field(default_factory=dict)
    mlp: Optional[Dict[str, Any]] = None


@dataclass(frozen=True)
class TekosunConfig(ModelConfig):
    """``Tekosun``: a decoder whose layers are listed one by one in config.json (``layers``: ``type``, the mixer's
    sizes under ``mixer``, the feed-forward under ``mlp`` or null).  The embedding is multiplied by
    ``embedding.scale``.  A sublayer reads the stream itself; an RMS norm sits behind it.  Mixers: ``mamba2`` (a
    selective state-space layer), ``general_delta`` (linear attention by the generalized delta rule) and
    ``attention`` (grouped-query attention with a norm over the whole query and key projections, rotary positions
    with an optional frequency scaling, a unit norm on every value head, an optional sliding window and an optional
    blend of the values with those of the first such layer).  The feed-forward is a mixture of squared-relu
    experts with a softmax router over all experts and a shared expert."""

    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    layers: List[TekosunLayer] = field(default_factory=list)

    ARCHITECTURE = "Tekosun"
    MODEL_TYPE = "tekosun"
    MIXERS = ("mamba2", "general_delta", "attention")

    @staticmethod
    def _opt_int(m: Dict[str, Any], key: str, default: int, minimum: int = 1) -> int:
        return _require_int(m, key, minimum) if m.get(key) is not None else default

    @classmethod
    def _mamba2(cls, m: Dict[str, Any], where: str) -> Dict[str, Any]:
        out = {"heads": _require_int(m, "heads"), "vdim": _require_int(m, "vdim"), "state": _require_int(m, "state"),
               "groups": cls._opt_int(m, "groups", 1), "conv": _require_int(m, "conv"),
               "norm_groups": cls._opt_int(m, "norm_groups", 1)}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"{where}: heads {out['heads']} is not a multiple of groups {out['groups']}")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"{where}: heads * vdim is not a multiple of norm_groups {out['norm_groups']}")
        if out["conv"] > 16:
            raise ConfigError(f"{where}: a convolution of {out['conv']} taps is not supported (at most 16)")
        if out["state"] > 512:
            raise ConfigError(f"{where}: a state of {out['state']} rows is not supported (at most 512)")
        return out

    @classmethod
    def _general_delta(cls, m: Dict[str, Any], where: str) -> Dict[str, Any]:
        out = {"heads": _require_int(m, "heads"), "dim": _require_int(m, "dim"),
               "decay_rank": cls._opt_int(m, "decay_rank", 0)}      # 0: the stored tensor's shape gives it
        if out["dim"] > 512:
            raise ConfigError(f"{where}: dim {out['dim']} is not supported (at most 512)")
        return out

    @classmethod
    def _attention(cls, m: Dict[str, Any], where: str) -> Dict[str, Any]:
        heads, dim = _require_int(m, "heads"), _require_int(m, "dim")
        out = {"heads": heads, "kv_heads": cls._opt_int(m, "kv_heads", heads), "dim": dim, "vdim": cls._opt_int(m, "vdim", dim),
               "scale": _require_number(m, "scale", where) if m.get("scale") is not None else float(dim) ** -0.5,
               "v_mix": bool(m.get("v_mix") or False), "window": None, "rot": {"dims": 0, "base": 10000.0, "scaling": None}}
        if heads % out["kv_heads"]:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {out['kv_heads']}")
        if dim > 256 or out["vdim"] > 256:
            raise ConfigError(f"{where}: dim and vdim must be at most 256")
        mask = _sub(m, "mask", where, optional=True)
        if mask is not None and mask.get("size") is not None:
            out["window"] = _require_int(mask, "size")
        rot = _sub(m, "rot", where, optional=True)
        if rot is not None and rot.get("dims"):
            dims = _require_int(rot, "dims")
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {dim}")
            base = _require_number(rot, "base", where + " rot")
            if base <= 1.0:
                raise ConfigError(f"{where}: rot.base must be above 1")
            out["rot"] = {"dims": dims, "base": base, "scaling": None}
            sc = _sub(rot, "scaling", where + " rot", optional=True)
            if sc is not None:
                out["rot"]["scaling"] = {k: _require_number(sc, k, where + " rot.scaling") for k in ("factor", "low", "high", "original")}
                s = out["rot"]["scaling"]
                if min(s.values()) <= 0 or s["high"] == s["low"]:
                    raise ConfigError(f"{where}: the numbers of rot.scaling must be positive, high and low different")
        return out

    @classmethod
    def _mlp(cls, mlp: Dict[str, Any], where: str) -> Dict[str, Any]:
        kind = mlp.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}: mlp kind {kind!r} is not one of ['moe']")
        router = _sub(mlp, "router", where)
        out = {"kind": "moe", "ff": _require_int(_sub(mlp, "expert", where), "ff"), "experts": _require_int(router, "experts"),
               "top": _require_int(router, "top"),
               "scale": _require_number(router, "scale", where + " router") if router.get("scale") is not None else 1.0,
               "shared_ff": None}
        if out["top"] > out["experts"]:
            raise ConfigError(f"{where}: router.top {out['top']} exceeds router.experts {out['experts']}")
        if out["top"] > 64:
            raise ConfigError(f"{where}: router.top {out['top']} is not supported (at most 64)")
        shared = _sub(mlp, "shared", where, optional=True)
        if shared is not None:
            out["shared_ff"] = _require_int(shared, "ff")
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TekosunConfig":
        width, vocab = _require_int(d, "width"), _require_int(d, "vocab")
        eps = _require_number(_sub(d, "norm", "config.json"), "eps", "config.json norm")
        if eps <= 0:
            raise ConfigError(f"norm eps must be positive, got {eps}")
        emb = _sub(d, "embedding", "config.json", optional=True) or {}
        scale = _require_number(emb, "scale", "config.json embedding") if emb.get("scale") is not None else 1.0
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers, first_mix = [], None
        for i, entry in enumerate(raw):
            where = f"config.json layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = entry.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {list(cls.MIXERS)}")
            mixer = getattr(cls, "_" + kind)(_sub(entry, "mixer", where), where + " mixer")
            if kind == "attention" and mixer["v_mix"]:
                sizes = (mixer["kv_heads"], mixer["vdim"])
                if first_mix is None:
                    first_mix = sizes
                elif sizes != first_mix:
                    raise ConfigError(f"{where}: a layer with v_mix has kv_heads, vdim {sizes}, the first such layer {first_mix}")
            mlp = _sub(entry, "mlp", where, optional=True)
            layers.append(TekosunLayer(type=kind, mixer=mixer, mlp=cls._mlp(mlp, where + " mlp") if mlp is not None else None))
        arch = d.get("architecture") or (d.get("architectures") or [cls.ARCHITECTURE])[0]
        return cls(architectures=[str(arch)], model_type=str(d.get("model_type", "") or cls.MODEL_TYPE), width=width,
                   vocab=vocab, norm_eps=eps, embedding_scale=scale, layers=layers)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> Optional[int]:
        return None

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration was read from (its own keys)."""
        layers = []
        for l in self.layers:
            m = dict(l.mixer)
            if l.type == "attention":
                rot, window = m.pop("rot"), m.pop("window")
                if rot["dims"]:
                    m["rot"] = {k: v for k, v in rot.items() if v is not None}
                if window:
                    m["mask"] = {"size": window}
            elif l.type == "general_delta" and not m["decay_rank"]:
                m.pop("decay_rank")
            mlp = None
            if l.mlp:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp["ff"]},
                       "router": {"experts": l.mlp["experts"], "top": l.mlp["top"], "scale": l.mlp["scale"]}}
                if l.mlp["shared_ff"]:
                    mlp["shared"] = {"ff": l.mlp["shared_ff"]}
            layers.append({"type": l.type, "mixer": m, "mlp": mlp})
        return {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "layers": layers}


@dataclass(frozen=True)
class MalazenLayer:
    """One layer of a Malazen model as config.json gives it: the mixer's sizes and constants (checked, defaults
    filled in) and its feed-forward (``None`` = none; ``kind`` ``dense`` with ``ff`` and ``limit``)."""

    type: str = ""
    mixer: Dict[str, Any] = field(default_factory=dict)
    mlp: Optional[Dict[str, Any]] = None


@dataclass(frozen=True)
class MalazenConfig(ModelConfig):
    """``Malazen``: a decoder whose layers are listed one by one in config.json (``layers``: ``type``, the mixer's
    sizes under ``mixer``, the feed-forward under ``mlp`` or null), pre-norm with an RMS norm taken over
    ``norm.groups`` equal parts of the row.  The mixer ``parallel`` is a weighted sum of a pair of mixers on one
    input: ``left`` grouped-query attention without rotation (biases, a query that grows with the logarithm of its
    position, a score that loses a logarithm of the distance) and ``right`` gated linear attention (a decay per key
    channel from a small projection, a normed and silu-gated output).  The mixer ``latent_attention`` keeps one
    normed latent and one rotated key part per token (neighbouring pairs rotate, frequencies optionally stretched),
    attends within a window and has a learned sink per head.  Feed-forwards are gated with clamped inputs.  A
    stretch of layers (``loop``: ``start``, ``stop``, ``times``) may run several times in a row on the same
    weights, the embedding's output being added to the stream ahead of every pass but the first.  The output head
    is the embedding table."""

    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    norm_groups: int = 1
    layers: List[MalazenLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0              # 0 = the model has no loop

    ARCHITECTURE = "Malazen"
    MODEL_TYPE = "malazen"

    @staticmethod
    def _left(m: Dict[str, Any], where: str) -> Dict[str, Any]:
        heads, dim = _require_int(m, "heads"), _require_int(m, "dim")
        out = {"heads": heads, "kv_heads": _require_int(m, "kv_heads") if m.get("kv_heads") is not None else heads,
               "dim": dim, "vdim": _require_int(m, "vdim") if m.get("vdim") is not None else dim,
               "scale": _require_number(m, "scale", where) if m.get("scale") is not None else float(dim) ** -0.5,
               "q_temp": None}
        if heads % out["kv_heads"]:
            raise ConfigError(f"{where}: heads {heads} is not a multiple of kv_heads {out['kv_heads']}")
        qt = _sub(m, "q_temp", where, optional=True)
        if qt is not None:
            out["q_temp"] = {"coef": _require_number(qt, "coef", where + " q_temp"), "every": _require_int(qt, "every")}
        return out

    @staticmethod
    def _right(m: Dict[str, Any], where: str) -> Dict[str, Any]:
        heads, dim = _require_int(m, "heads"), _require_int(m, "dim")
        tau = _require_number(m, "tau", where)
        if tau <= 0:
            raise ConfigError(f"{where}: tau must be positive")
        return {"heads": heads, "dim": dim, "vdim": _require_int(m, "vdim") if m.get("vdim") is not None else dim, "tau": tau}

    @staticmethod
    def _latent(m: Dict[str, Any], where: str) -> Dict[str, Any]:
        dim, rot_dim = _require_int(m, "dim"), _require_int(m, "rot_dim", 0) if m.get("rot_dim") is not None else 0
        out = {"heads": _require_int(m, "heads"), "dim": dim, "rot_dim": rot_dim, "vdim": _require_int(m, "vdim"),
               "kv_rank": _require_int(m, "kv_rank"),
               "scale": _require_number(m, "scale", where) if m.get("scale") is not None else float(dim + rot_dim) ** -0.5,
               "window": 0, "rot": None}
        mask = _sub(m, "mask", where, optional=True)
        if mask is not None:
            out["window"] = _require_int(mask, "size")
        if rot_dim:
            out["rot"] = PemoraxConfig._rot(m, where, rot_dim)
            if out["rot"]["dims"] != rot_dim:
                raise ConfigError(f"{where}: rot.dims {out['rot']['dims']} must equal rot_dim {rot_dim}")
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MalazenConfig":
        width, vocab = _require_int(d, "width"), _require_int(d, "vocab")
        norm = _sub(d, "norm", "config.json")
        eps = _require_number(norm, "eps", "config.json norm")
        groups = _require_int(norm, "groups") if norm.get("groups") is not None else 1
        if eps <= 0:
            raise ConfigError(f"norm eps must be positive, got {eps}")
        if width % groups:
            raise ConfigError(f"norm.groups {groups} does not divide the width {width}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw):
            where = f"config.json layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where}: must be an object")
            kind = entry.get("type")
            mixer = _sub(entry, "mixer", where)
            if kind == "parallel":
                sizes = {"left": cls._left(_sub(mixer, "left", where + " mixer"), where + " mixer.left"),
                         "right": cls._right(_sub(mixer, "right", where + " mixer"), where + " mixer.right"),
                         "left_scale": _opt_number(mixer, "left_scale", 1.0), "right_scale": _opt_number(mixer, "right_scale", 1.0)}
            elif kind == "latent_attention":
                sizes = cls._latent(mixer, where + " mixer")
            else:
                raise ConfigError(f"{where}: type {kind!r} is not one of ['latent_attention', 'parallel']")
            mlp = _sub(entry, "mlp", where, optional=True)
            ff = None
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}: mlp kind {mlp.get('kind')!r} is not one of ['dense']")
                ff = {"kind": "dense", "ff": _require_int(mlp, "ff"), "limit": _require_number(mlp, "limit", where + " mlp")}
                if ff["limit"] <= 0:
                    raise ConfigError(f"{where}: mlp limit must be positive")
            layers.append(MalazenLayer(type=kind, mixer=sizes, mlp=ff))
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
        return cls(architectures=[str(arch)], model_type=str(d.get("model_type", "") or cls.MODEL_TYPE), width=width,
                   vocab=vocab, norm_eps=eps, norm_groups=groups, layers=layers, loop_start=start, loop_stop=stop,
                   loop_times=times)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> Optional[int]:
        return None

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration was read from (its own keys)."""
        layers = []
        for l in self.layers:
            m = {k: (dict(v) if isinstance(v, dict) else v) for k, v in l.mixer.items()}
            if l.type == "parallel":
                if m["left"]["q_temp"] is None:
                    m["left"].pop("q_temp")
            else:
                window, rot = m.pop("window"), m.pop("rot")
                if window:
                    m["mask"] = {"size": window}
                if rot:
                    m["rot"] = {k: v for k, v in rot.items() if v is not None}
            layers.append({"type": l.type, "mixer": m, "mlp": dict(l.mlp) if l.mlp else None})
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": layers}
        if self.loop_times:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
