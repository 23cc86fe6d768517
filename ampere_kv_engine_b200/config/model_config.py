"""Typed model configurations read from an architecture's own config.json keys.

The reference has no configuration code of its own: it reads attributes of the object the
checkpoint loader builds (ampere_kv/runner.py:33-44: ``head_dim``, ``rope_theta``,
``hidden_act``, per-layer ``sliding_window``, per-norm ``variance_epsilon``; runner.py:321
``num_key_value_heads``; runner.py:331 ``eos_token_id``).  Here every such constant is a
field of a dataclass parsed from config.json; no size stands anywhere else in the code.
"""

from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, fields
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, of the wrong type, or asks for something unsupported."""


def _require(d: dict, key: str, kind):
    if key not in d:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return _typed(d, key, kind)


def _typed(d: dict, key: str, kind):
    value = d[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if kind is int and isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config.json: key '{key}' must be {kind.__name__}, got {value!r}")
    return value


def _optional(d: dict, key: str, kind, default):
    if key not in d or d[key] is None:
        return default
    return _typed(d, key, kind)


@dataclass(frozen=True)
class Qwen3Config:
    """config.json of ``Qwen3ForCausalLM`` (dense decoder).

    Field names are the checkpoint's own keys.  ``head_dim`` is explicit and need not equal
    ``hidden_size // num_attention_heads`` (the reference derives head counts from the
    projection widths, ampere_kv/runner.py:69).
    """

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    layer_types: tuple[str, ...] | None = None
    eos_token_id: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("Qwen3ForCausalLM",)

    ARCHITECTURE = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen3Config":
        heads = _require(d, "num_attention_heads", int)
        hidden = _require(d, "hidden_size", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: 'num_attention_heads' and 'hidden_size' must be positive")
        eos = d.get("eos_token_id")
        if eos is None:
            eos = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos = tuple(eos)
        else:
            raise ConfigError(f"config.json: key 'eos_token_id' must be an int or a list of ints, got {eos!r}")
        layer_types = d.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, (list, tuple)) or not all(isinstance(t, str) for t in layer_types):
                raise ConfigError("config.json: key 'layer_types' must be a list of strings")
            layer_types = tuple(layer_types)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"
        arch = d.get("architectures") or (cls.ARCHITECTURE,)
        cfg = cls(
            vocab_size=_require(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_require(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_optional(d, "num_key_value_heads", int, heads),
            head_dim=_optional(d, "head_dim", int, hidden // heads),
            intermediate_size=_require(d, "intermediate_size", int),
            rope_theta=_optional(d, "rope_theta", float, 10000.0),
            rms_norm_eps=_optional(d, "rms_norm_eps", float, 1e-6),
            max_position_embeddings=_optional(d, "max_position_embeddings", int, 32768),
            tie_word_embeddings=_optional(d, "tie_word_embeddings", bool, False),
            hidden_act=_optional(d, "hidden_act", str, "silu"),
            attention_bias=_optional(d, "attention_bias", bool, False),
            use_sliding_window=_optional(d, "use_sliding_window", bool, False),
            sliding_window=_optional(d, "sliding_window", int, None),
            max_window_layers=_optional(d, "max_window_layers", int, None),
            layer_types=layer_types,
            eos_token_id=eos,
            torch_dtype=str(dtype),
            architectures=tuple(arch),
        )
        cfg.validate(d)
        return cfg

    def validate(self, raw: dict | None = None) -> None:
        for name in ("vocab_size", "num_hidden_layers", "num_key_value_heads", "head_dim", "intermediate_size",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: key '{name}' must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' ({self.num_attention_heads}) must be a multiple of "
                f"'num_key_value_heads' ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' must be even for rotate-half RoPE, got {self.head_dim}")
        if self.hidden_act != "silu":
            # the reference refuses anything but SiLU (ampere_kv/runner.py:39-40)
            raise ConfigError(f"config.json: 'hidden_act' must be 'silu', got {self.hidden_act!r}")
        if self.rope_theta <= 0 or self.rms_norm_eps <= 0:
            raise ConfigError("config.json: 'rope_theta' and 'rms_norm_eps' must be positive")
        if raw is not None and raw.get("rope_scaling") not in (None, {}):
            scaling = raw["rope_scaling"]
            kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                # the reference assumes rope_scaling is empty (ampere_kv/runner.py:83)
                raise ConfigError(f"config.json: 'rope_scaling' {kind!r} is not supported (only none/default)")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config.json: 'use_sliding_window' is true but 'sliding_window' is not a positive int")
        if self.layer_types is not None:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            bad = sorted(set(self.layer_types) - {"full_attention", "sliding_attention"})
            if bad:
                raise ConfigError(f"config.json: 'layer_types' holds unknown kinds {bad}")

    def window_of_layer(self, index: int) -> int | None:
        """Number of keys (the query's own included) layer ``index`` attends to, or None for all."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        if self.layer_types is not None:
            slides = self.layer_types[index] == "sliding_attention"
        else:
            first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
            slides = index >= first
        return self.sliding_window if slides else None

    def to_dict(self) -> dict[str, Any]:
        out = {}
        for f in fields(self):
            value = getattr(self, f.name)
            if isinstance(value, tuple):
                value = list(value)
            out[f.name] = value
        if len(out["eos_token_id"]) == 0:
            out["eos_token_id"] = None
        elif len(out["eos_token_id"]) == 1:
            out["eos_token_id"] = out["eos_token_id"][0]
        out["model_type"] = "qwen3"
        return out


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as handle:
        try:
            raw = json.load(handle)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    # The reference stops on ``model.generation_config.eos_token_id`` (ampere_kv/runner.py:331): the ids of
    # generation_config.json where that file carries them (a published checkpoint lists more ids there than in
    # config.json), else config.json's own.
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen_path):
        with open(gen_path, "r", encoding="utf-8") as handle:
            try:
                gen = json.load(handle)
            except json.JSONDecodeError as exc:
                raise ConfigError(f"{gen_path}: not valid JSON ({exc})") from exc
        if isinstance(gen, dict) and gen.get("eos_token_id") is not None:
            raw["eos_token_id"] = gen["eos_token_id"]
    return raw


def _section(d: dict, key: str, where: str) -> dict:
    if key not in d or not isinstance(d[key], dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return d[key]


def _sized(d: dict, key: str, where: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json: {where}required key '{key}' is missing")
    value = d[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {value!r}")
    return value


def _number(d: dict, key: str, where: str) -> float:
    if key not in d:
        raise ConfigError(f"config.json: {where}required key '{key}' is missing")
    value = d[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class SukalornLayer:
    """One entry of ``layers``: the mixer's ``type``, its sizes and constants as config.json gives them, and the
    feed-forward (None: the layer has none)."""

    type: str
    mixer: dict
    mlp: dict | None

    MIXERS = ("attention", "latent_attention")


@dataclass(frozen=True)
class SukalornConfig:
    """config.json of the ``Sukalorn`` decoder: ``vocab``, ``width``, ``norm.eps`` and a list of layers, each naming
    its mixer (``attention``: grouped queries with unit-norm q/k, capped and distance-biased scores, blocks of
    positions, blended values and a gate per head; ``latent_attention``: low-rank query and key/value latents with a
    shared rotated key part) and its dense feed-forward.  Every size and constant is read from here."""

    vocab: int
    width: int
    norm_eps: float
    layers: tuple[SukalornLayer, ...]
    max_position_embeddings: int = 1 << 20
    eos_token_id: tuple[int, ...] = ()
    architectures: tuple[str, ...] = ("Sukalorn",)

    ARCHITECTURE = "Sukalorn"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "SukalornConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, dict) or entry.get("type") not in SukalornLayer.MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {list(SukalornLayer.MIXERS)}, "
                                  f"got {entry.get('type') if isinstance(entry, dict) else entry!r}")
            mixer = _section(entry, "mixer", where)
            where_m = where + "mixer: "
            for key in ("heads", "dim", "vdim"):
                _sized(mixer, key, where_m)
            _number(mixer, "scale", where_m)
            if entry["type"] == "attention":
                kv = _sized(mixer, "kv_heads", where_m)
                if mixer["heads"] % kv:
                    raise ConfigError(f"config.json: {where_m}'heads' ({mixer['heads']}) must be a multiple of "
                                      f"'kv_heads' ({kv})")
                if mixer.get("softcap") is not None and _number(mixer, "softcap", where_m) <= 0:
                    raise ConfigError(f"config.json: {where_m}'softcap' must be positive")
                if mixer.get("mask") is not None:
                    _sized(_section(mixer, "mask", where_m), "size", where_m + "mask: ")
            else:
                for key in ("q_rank", "kv_rank", "rot_dim"):
                    _sized(mixer, key, where_m)
                rot = _section(mixer, "rot", where_m)
                dims = _sized(rot, "dims", where_m + "rot: ")
                if _number(rot, "base", where_m + "rot: ") <= 0:
                    raise ConfigError(f"config.json: {where_m}rot: 'base' must be positive")
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"config.json: {where_m}rot: 'dims' must be even and at most 'rot_dim' "
                                      f"({mixer['rot_dim']}), got {dims}")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}'mlp' must be an object or null")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp: 'kind' must be 'dense', got {mlp.get('kind')!r}")
                _sized(mlp, "ff", where + "mlp: ")
            layers.append(SukalornLayer(entry["type"], dict(mixer), None if mlp is None else dict(mlp)))
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        cfg = cls(
            vocab=_sized(d, "vocab", ""),
            width=_sized(d, "width", ""),
            norm_eps=_number(_section(d, "norm", ""), "eps", "norm: "),
            layers=tuple(layers),
            max_position_embeddings=_optional(d, "max_position_embeddings", int, 1 << 20),
            eos_token_id=eos,
        )
        if cfg.norm_eps <= 0:
            raise ConfigError("config.json: norm: 'eps' must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.mlp is None else dict(l.mlp)}
                          for l in self.layers]}
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


@dataclass(frozen=True)
class ZifuzenLayer:
    """One entry of ``layers``: the mixer's ``type``, its sizes and constants as config.json gives them, and the
    feed-forward (None: the layer has none)."""

    type: str
    mixer: dict
    mlp: dict | None

    #: both delta types are the gated delta rule
    MIXERS = ("attention", "delta", "delta_2")


@dataclass(frozen=True)
class ZifuzenConfig:
    """config.json of the ``Zifuzen`` decoder: ``vocab``, ``width``, ``max_positions`` (rows of the learned
    position table), ``embedding.scale``, ``norm.eps``, ``logit_softcap`` and a list of layers.  A layer names its
    mixer (``attention``: grouped queries with a weighted RMS norm on queries and keys, no rotation, optionally the
    keys and values of an earlier layer, ``kv_from``; ``delta`` / ``delta_2``: the gated delta rule behind short
    convolutions) and its feed-forward (``dense`` with biases and tanh GELU, ``moe`` with a sigmoid router over groups
    of experts and an optional shared expert, or none).  Every size and constant is read from here."""

    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float | None
    layers: tuple[ZifuzenLayer, ...]
    eos_token_id: tuple[int, ...] = ()
    architectures: tuple[str, ...] = ("Zifuzen",)

    ARCHITECTURE = "Zifuzen"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @staticmethod
    def _check_expert(d: dict, where: str) -> None:
        _sized(d, "ff", where)
        if _number(d, "limit", where) <= 0:
            raise ConfigError(f"config.json: {where}'limit' must be positive")

    @classmethod
    def _check_mlp(cls, mlp: dict, where: str) -> None:
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _sized(mlp, "ff", where)
            return
        if kind != "moe":
            raise ConfigError(f"config.json: {where}'kind' must be 'dense' or 'moe', got {kind!r}")
        cls._check_expert(_section(mlp, "expert", where), where + "expert: ")
        router = _section(mlp, "router", where)
        where_r = where + "router: "
        experts, top = _sized(router, "experts", where_r), _sized(router, "top", where_r)
        _number(router, "scale", where_r)
        count = keep = 1
        if router.get("groups") is not None:
            groups = _section(router, "groups", where_r)
            count, keep = _sized(groups, "count", where_r + "groups: "), _sized(groups, "keep", where_r + "groups: ")
        if experts % count or keep > count:
            raise ConfigError(f"config.json: {where_r}groups: 'count' ({count}) must divide 'experts' ({experts}) and "
                              f"'keep' ({keep}) must not exceed it")
        if top > keep * (experts // count):
            raise ConfigError(f"config.json: {where_r}'top' ({top}) is more than the {keep} kept groups of "
                              f"{experts // count} experts hold")
        if mlp.get("shared") is not None:
            cls._check_expert(_section(mlp, "shared", where), where + "shared: ")

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ZifuzenConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, dict) or entry.get("type") not in ZifuzenLayer.MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {list(ZifuzenLayer.MIXERS)}, "
                                  f"got {entry.get('type') if isinstance(entry, dict) else entry!r}")
            mixer = _section(entry, "mixer", where)
            where_m = where + "mixer: "
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _sized(mixer, key, where_m)
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"config.json: {where_m}'heads' ({mixer['heads']}) must be a multiple of "
                                  f"'kv_heads' ({mixer['kv_heads']})")
            if entry["type"] == "attention":
                _number(mixer, "scale", where_m)
                source = mixer.get("kv_from")
                if source is not None:
                    ok = isinstance(source, int) and not isinstance(source, bool) and 0 <= source < i
                    other = layers[source] if ok else None
                    if other is None or other.type != "attention" or other.mixer.get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where_m}'kv_from' must name an earlier attention layer that "
                                          f"has keys and values of its own, got {source!r}")
                    if any(other.mixer[k] != mixer[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"config.json: {where_m}'kv_from': layer {source} keeps keys and values of "
                                          f"another shape")
            else:
                _sized(mixer, "conv", where_m)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}'mlp' must be an object or null")
                cls._check_mlp(mlp, where + "mlp: ")
            layers.append(ZifuzenLayer(entry["type"], dict(mixer), None if mlp is None else copy.deepcopy(mlp)))
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        cap = d.get("logit_softcap")
        cfg = cls(
            vocab=_sized(d, "vocab", ""),
            width=_sized(d, "width", ""),
            max_positions=_sized(d, "max_positions", ""),
            embedding_scale=_number(_section(d, "embedding", ""), "scale", "embedding: "),
            norm_eps=_number(_section(d, "norm", ""), "eps", "norm: "),
            logit_softcap=None if cap is None else _number(d, "logit_softcap", ""),
            layers=tuple(layers),
            eos_token_id=eos,
        )
        if cfg.norm_eps <= 0:
            raise ConfigError("config.json: norm: 'eps' must be positive")
        if cfg.logit_softcap is not None and cfg.logit_softcap <= 0:
            raise ConfigError("config.json: 'logit_softcap' must be positive (or null for none)")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
               "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap,
               "layers": [{"type": l.type, "mixer": dict(l.mixer), "mlp": None if l.mlp is None else copy.deepcopy(l.mlp)}
                          for l in self.layers]}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


@dataclass(frozen=True)
class RenadraLayer:
    """One entry of ``layers``: the mixer's ``type``, its sizes and constants as config.json gives them, and the
    feed-forward (None: the layer has none)."""

    type: str
    mixer: dict
    mlp: dict | None

    MIXERS = ("attention", "hgrn2", "parallel")


@dataclass(frozen=True)
class RenadraConfig:
    """config.json of the ``Renadra`` decoder: ``vocab``, ``width``, ``norm.eps``, ``embedding`` (``scale`` and an
    optional ``bigram`` table: ``buckets``, ``mul_prev``, ``mul_cur``), a list of layers and an optional ``loop``
    (``start``, ``stop``, ``times``: the run of layers [start, stop) is walked ``times`` times on one set of weights).
    A layer names its mixer (``attention``: rotated queries and keys in neighbouring pairs, unit-RMS values, a window,
    softmax; ``hgrn2``: a matrix memory per head that writes to a row with one minus its forget gate; ``parallel``: a
    ``left`` attention without a softmax whose values are its unrotated keys, beside a ``right`` linear attention with
    a constant decay per head) and its dense feed-forward (or null).  Every size and constant is read from here."""

    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: dict | None
    layers: tuple[RenadraLayer, ...]
    loop: dict | None = None
    max_position_embeddings: int = 1 << 20
    eos_token_id: tuple[int, ...] = ()
    architectures: tuple[str, ...] = ("Renadra",)

    ARCHITECTURE = "Renadra"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def _check_rot(m: dict, where: str, dim: int) -> None:
        rot = _section(m, "rot", where)
        where_r = where + "rot: "
        dims = _sized(rot, "dims", where_r)
        if _number(rot, "base", where_r) <= 1:
            raise ConfigError(f"config.json: {where_r}'base' must be above 1")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where_r}'dims' must be even and at most 'dim' ({dim}), got {dims}")
        if rot.get("scaling") is not None:
            s = _section(rot, "scaling", where_r)
            for key in ("factor", "original", "fast", "slow"):
                if _number(s, key, where_r + "scaling: ") <= 0:
                    raise ConfigError(f"config.json: {where_r}scaling: '{key}' must be positive")

    @classmethod
    def _check_attention(cls, m: dict, where: str, left: bool) -> None:
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _sized(m, key, where)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {where}'heads' ({m['heads']}) must be a multiple of 'kv_heads' "
                              f"({m['kv_heads']})")
        _number(m, "scale", where)
        cls._check_rot(m, where, m["dim"])
        mask = _section(m, "mask", where)
        _sized(mask, "size", where + "mask: ")
        keep = mask.get("keep_first") or 0
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            raise ConfigError(f"config.json: {where}mask: 'keep_first' must be a non-negative integer, got {keep!r}")
        if m.get("softcap") is not None and _number(m, "softcap", where) <= 0:
            raise ConfigError(f"config.json: {where}'softcap' must be positive")
        if left and m["vdim"] != m["dim"]:
            raise ConfigError(f"config.json: {where}'vdim' ({m['vdim']}) must equal 'dim' ({m['dim']}): the values "
                              f"are the keys")

    @staticmethod
    def _check_memory(m: dict, where: str, decay: bool) -> None:
        for key in ("heads", "dim", "vdim"):
            _sized(m, key, where)
        if decay:
            rates = m.get("decay")
            if not isinstance(rates, (list, tuple)) or len(rates) != m["heads"] or not all(
                    isinstance(r, (int, float)) and not isinstance(r, bool) and 0 <= r <= 1 for r in rates):
                raise ConfigError(f"config.json: {where}'decay' must list a number between 0 and 1 for each of the "
                                  f"{m['heads']} heads")

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "RenadraConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, dict) or entry.get("type") not in RenadraLayer.MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {list(RenadraLayer.MIXERS)}, "
                                  f"got {entry.get('type') if isinstance(entry, dict) else entry!r}")
            mixer = _section(entry, "mixer", where)
            where_m = where + "mixer: "
            if entry["type"] == "attention":
                cls._check_attention(mixer, where_m, left=False)
            elif entry["type"] == "hgrn2":
                cls._check_memory(mixer, where_m, decay=False)
            else:
                cls._check_attention(_section(mixer, "left", where_m), where_m + "left: ", left=True)
                cls._check_memory(_section(mixer, "right", where_m), where_m + "right: ", decay=True)
                _number(mixer, "left_scale", where_m)
                _number(mixer, "right_scale", where_m)
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}'mlp' must be an object or null")
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp: 'kind' must be 'dense', got {mlp.get('kind')!r}")
                _sized(mlp, "ff", where + "mlp: ")
            layers.append(RenadraLayer(entry["type"], copy.deepcopy(mixer), None if mlp is None else copy.deepcopy(mlp)))
        embedding = _section(d, "embedding", "")
        bigram = embedding.get("bigram")
        if bigram is not None:
            bigram = _section(embedding, "bigram", "embedding: ")
            _sized(bigram, "buckets", "embedding: bigram: ")
            for key in ("mul_prev", "mul_cur"):
                if isinstance(bigram.get(key), bool) or not isinstance(bigram.get(key), int) or bigram[key] < 0:
                    raise ConfigError(f"config.json: embedding: bigram: '{key}' must be a non-negative integer, "
                                      f"got {bigram.get(key)!r}")
            bigram = dict(bigram)
        loop = d.get("loop")
        if loop is not None:
            loop = _section(d, "loop", "")
            times = _sized(loop, "times", "loop: ")
            start, stop = loop.get("start"), loop.get("stop")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop)) or \
                    not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop: 'start' and 'stop' must satisfy 0 <= start < stop <= "
                                  f"{len(layers)}, got {start!r} and {stop!r}")
            loop = {"start": start, "stop": stop, "times": times}
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        cfg = cls(
            vocab=_sized(d, "vocab", ""),
            width=_sized(d, "width", ""),
            norm_eps=_number(_section(d, "norm", ""), "eps", "norm: "),
            embedding_scale=_number(embedding, "scale", "embedding: "),
            bigram=bigram,
            layers=tuple(layers),
            loop=loop,
            max_position_embeddings=_optional(d, "max_position_embeddings", int, 1 << 20),
            eos_token_id=eos,
        )
        if cfg.norm_eps <= 0:
            raise ConfigError("config.json: norm: 'eps' must be positive")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        embedding: dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = dict(self.bigram)
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": embedding,
               "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer),
                           "mlp": None if l.mlp is None else copy.deepcopy(l.mlp)} for l in self.layers]}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out


@dataclass(frozen=True)
class ZavizenLayer:
    """One layer of a Zavizen model as config.json gives it: ``type`` names the mixer, ``mixer`` holds its sizes and
    constants, ``mlp`` the feed-forward's (None: the layer has none)."""

    type: str
    mixer: dict
    mlp: dict | None

    MIXERS = ("parallel", "mamba2")


@dataclass(frozen=True)
class ZavizenConfig:
    """config.json of the ``Zavizen`` decoder: ``vocab``, ``width``, ``norm.eps``, ``streams`` (copies of the residual
    stream), a list of layers and an optional ``loop`` (``start``, ``stop``, ``times``: the run of layers [start, stop)
    is walked ``times`` times on one set of weights).  A layer names its mixer (``parallel``: a ``left`` softmax
    attention with ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` beside a ``right`` retention with
    ``heads``, ``dim``, ``vdim``, ``decay``, ``rot``; ``mamba2``: ``heads``, ``vdim``, ``state``, ``groups``, ``conv``,
    ``norm_groups``) and its feed-forward (``kind`` ``dense`` with ``ff``, or ``moe`` with ``expert.ff``, ``router``
    (``experts``, ``top``, ``scale``, optional ``groups`` with ``count`` and ``keep``) and an optional ``shared.ff``;
    or null).  Every size and constant is read from here."""

    vocab: int
    width: int
    norm_eps: float
    streams: int
    layers: tuple[ZavizenLayer, ...]
    loop: dict | None = None
    max_position_embeddings: int = 1 << 20
    eos_token_id: tuple[int, ...] = ()
    architectures: tuple[str, ...] = ("Zavizen",)

    ARCHITECTURE = "Zavizen"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def _check_rot(m: dict, where: str, dim: int) -> None:
        rot = _section(m, "rot", where)
        where_r = where + "rot: "
        dims = _sized(rot, "dims", where_r)
        if _number(rot, "base", where_r) <= 1:
            raise ConfigError(f"config.json: {where_r}'base' must be above 1")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where_r}'dims' must be even and at most 'dim' ({dim}), got {dims}")
        if rot.get("scaling") is not None:
            if _number(_section(rot, "scaling", where_r), "factor", where_r + "scaling: ") <= 0:
                raise ConfigError(f"config.json: {where_r}scaling: 'factor' must be positive")

    @classmethod
    def _check_mixer(cls, kind: str, m: dict, where: str) -> None:
        if kind == "mamba2":
            for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                _sized(m, key, where)
            if m["heads"] % m["groups"]:
                raise ConfigError(f"config.json: {where}'heads' ({m['heads']}) must be a multiple of 'groups' "
                                  f"({m['groups']})")
            if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                raise ConfigError(f"config.json: {where}'norm_groups' ({m['norm_groups']}) must divide heads * vdim "
                                  f"({m['heads'] * m['vdim']})")
            return
        left, right = _section(m, "left", where), _section(m, "right", where)
        wl, wr = where + "left: ", where + "right: "
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _sized(left, key, wl)
        if left["heads"] % left["kv_heads"]:
            raise ConfigError(f"config.json: {wl}'heads' ({left['heads']}) must be a multiple of 'kv_heads' "
                              f"({left['kv_heads']})")
        _number(left, "scale", wl)
        cls._check_rot(left, wl, left["dim"])
        for key in ("heads", "dim", "vdim"):
            _sized(right, key, wr)
        cls._check_rot(right, wr, right["dim"])
        rates = right.get("decay")
        if not isinstance(rates, (list, tuple)) or len(rates) != right["heads"] or not all(
                isinstance(r, (int, float)) and not isinstance(r, bool) and 0 <= r <= 1 for r in rates):
            raise ConfigError(f"config.json: {wr}'decay' must list a number between 0 and 1 for each of the "
                              f"{right['heads']} heads")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _sized(mlp, "ff", where)
            return
        if kind != "moe":
            raise ConfigError(f"config.json: {where}'kind' must be 'dense' or 'moe', got {kind!r}")
        _sized(_section(mlp, "expert", where), "ff", where + "expert: ")
        router, where_r = _section(mlp, "router", where), where + "router: "
        experts, top = _sized(router, "experts", where_r), _sized(router, "top", where_r)
        _number(router, "scale", where_r)
        count, keep = 1, 1
        if router.get("groups") is not None:
            groups = _section(router, "groups", where_r)
            count, keep = _sized(groups, "count", where_r + "groups: "), _sized(groups, "keep", where_r + "groups: ")
        if experts % count or keep > count:
            raise ConfigError(f"config.json: {where_r}{experts} experts do not form {count} equal groups of which "
                              f"{keep} are kept")
        if top > keep * (experts // count):
            raise ConfigError(f"config.json: {where_r}'top' ({top}) is more than the kept groups hold")
        if mlp.get("shared") is not None:
            _sized(_section(mlp, "shared", where), "ff", where + "shared: ")

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ZavizenConfig":
        layers_raw = d.get("layers")
        if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]: "
            if not isinstance(entry, dict) or entry.get("type") not in ZavizenLayer.MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {list(ZavizenLayer.MIXERS)}, "
                                  f"got {entry.get('type') if isinstance(entry, dict) else entry!r}")
            mixer = _section(entry, "mixer", where)
            cls._check_mixer(entry["type"], mixer, where + "mixer: ")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}'mlp' must be an object or null")
                cls._check_mlp(mlp, where + "mlp: ")
            layers.append(ZavizenLayer(entry["type"], copy.deepcopy(mixer), None if mlp is None else copy.deepcopy(mlp)))
        loop = d.get("loop")
        if loop is not None:
            loop = _section(d, "loop", "")
            times = _sized(loop, "times", "loop: ")
            start, stop = loop.get("start"), loop.get("stop")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop)) or \
                    not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop: 'start' and 'stop' must satisfy 0 <= start < stop <= "
                                  f"{len(layers)}, got {start!r} and {stop!r}")
            loop = {"start": start, "stop": stop, "times": times}
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        cfg = cls(
            vocab=_sized(d, "vocab", ""),
            width=_sized(d, "width", ""),
            norm_eps=_number(_section(d, "norm", ""), "eps", "norm: "),
            streams=_sized(d, "streams", ""),
            layers=tuple(layers),
            loop=loop,
            max_position_embeddings=_optional(d, "max_position_embeddings", int, 1 << 20),
            eos_token_id=eos,
        )
        if cfg.norm_eps <= 0:
            raise ConfigError("config.json: norm: 'eps' must be positive")
        if cfg.streams > 8:
            raise ConfigError(f"config.json: 'streams' must be at most 8, got {cfg.streams}")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "streams": self.streams,
               "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer),
                           "mlp": None if l.mlp is None else copy.deepcopy(l.mlp)} for l in self.layers]}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
