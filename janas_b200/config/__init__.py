"""Configuration: typed per-architecture classes, the neutral ``ModelSpec`` they
produce, and the registry that finds the class for a ``config.json``.

The reading, checking and the registry are the library's (``config/qwen3.cpp``,
``config/registry.cpp``, ``config/spec.cpp``); the classes here hold what it
returns.  A ``ModelSpec`` can also be put together by hand from ``PartSpec``s of
registered parts and opened directly (``janas_b200.engine.Engine.from_spec``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple

from .. import lib


class ConfigError(ValueError):
    """A configuration that cannot be built: a missing key, a wrong value."""

    def __init__(self, message: str, code: int = lib.EOPEN):
        super().__init__(message)
        self.code = code


def _call(method: str, **args):
    try:
        return lib.call(method, **args)
    except lib.LLMError as e:
        raise ConfigError(str(e), e.code) from None


def _plain(v: Any) -> Any:
    """Parameters as JSON holds them (tuples become lists, parts become objects)."""
    if isinstance(v, PartSpec):
        return v.to_json()
    if isinstance(v, Mapping):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __hash__(self) -> int:
        return hash((self.kind, json.dumps(_plain(self.params), sort_keys=True)))

    def to_json(self) -> Dict[str, Any]:
        return {"kind": self.kind, "params": _plain(self.params)}

    @staticmethod
    def from_json(d: Mapping[str, Any]) -> "PartSpec":
        params = {k: (PartSpec.from_json(v) if isinstance(v, dict) and set(v) == {"kind", "params"}
                      else v) for k, v in (d.get("params") or {}).items()}
        return PartSpec(d["kind"], params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged and where its tensors are found."""

    block: str
    mixer: PartSpec
    feed_forward: Optional[PartSpec]        # None: the layer has no feed-forward (and no ffn_norm)
    mixer_norm: Optional[PartSpec]          # None: the arrangement's sublayers read the residual stream itself
    ffn_norm: Optional[PartSpec]
    prefix: str
    mixer_name: str = "self_attn"
    ffn_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    ffn_norm_name: str = "post_attention_layernorm"
    # norms on the sublayers' results, for the arrangements that have them
    post_mixer_norm: Optional[PartSpec] = None
    post_ffn_norm: Optional[PartSpec] = None
    post_mixer_norm_name: str = "post_mixer_norm"
    post_ffn_norm_name: str = "post_ffn_norm"
    # the arrangement's own constants and the names of tensors it owns
    block_params: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:
        return hash((self.block, self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm,
                     self.prefix, json.dumps(_plain(self.block_params), sort_keys=True)))

    def to_json(self) -> Dict[str, Any]:
        none = {"kind": "", "params": {}}
        d = {"block": self.block, "mixer": self.mixer.to_json(),
             "feed_forward": self.feed_forward.to_json() if self.feed_forward else none,
             "mixer_norm": self.mixer_norm.to_json() if self.mixer_norm else none,
             "ffn_norm": self.ffn_norm.to_json() if self.ffn_norm else none,
             "prefix": self.prefix, "mixer_name": self.mixer_name, "ffn_name": self.ffn_name,
             "mixer_norm_name": self.mixer_norm_name, "ffn_norm_name": self.ffn_norm_name,
             "post_mixer_norm_name": self.post_mixer_norm_name,
             "post_ffn_norm_name": self.post_ffn_norm_name}
        if self.post_mixer_norm:
            d["post_mixer_norm"] = self.post_mixer_norm.to_json()
        if self.post_ffn_norm:
            d["post_ffn_norm"] = self.post_ffn_norm.to_json()
        if self.block_params:
            d["block_params"] = _plain(self.block_params)
        return d

    @staticmethod
    def from_json(l: Mapping[str, Any]) -> "LayerSpec":
        def part(key):
            v = l.get(key)
            return PartSpec.from_json(v) if v and v.get("kind") else None
        return LayerSpec(
            l["block"], PartSpec.from_json(l["mixer"]), part("feed_forward"),
            part("mixer_norm"), part("ffn_norm"), l["prefix"],
            l["mixer_name"], l["ffn_name"], l["mixer_norm_name"], l["ffn_norm_name"],
            part("post_mixer_norm"), part("post_ffn_norm"),
            l.get("post_mixer_norm_name", "post_mixer_norm"),
            l.get("post_ffn_norm_name", "post_ffn_norm"), l.get("block_params") or {})


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run ``layer`` (its weights).  With ``cache_of``
    set (the index of an earlier entry) the entry's mixer writes nothing and reads
    that entry's cache."""

    layer: int
    cache_of: Optional[int] = None
    # before this entry the embedding output is added to the residual stream once more
    add_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    tie_embeddings: bool
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
    position_table_name: str = ""      # a table of learned position vectors; "": none
    logit_scale: float = 1.0
    embedding_scale: float = 1.0       # a factor on the embedding rows (a tied head reads the table without it)
    embedding_norm: Optional[PartSpec] = None      # a norm on the embedding rows
    embedding_norm_name: str = "model.embed_norm"
    token_table_name: str = ""         # a second table of vectors per token that the layers' blocks read; "": none
    token_table_width: int = 0

    def to_json(self) -> Dict[str, Any]:
        d = {
            "architecture": self.architecture, "hidden_size": self.hidden_size,
            "vocab_size": self.vocab_size, "max_positions": self.max_positions,
            "layers": [l.to_json() for l in self.layers],
            "run_order": [dict({"layer": e.layer, "cache_of": e.cache_of},
                               **({"add_embedding": True} if e.add_embedding else {}))
                          for e in self.run_order],
            "final_norm": self.final_norm.to_json(), "tie_embeddings": self.tie_embeddings,
            "embedding_name": self.embedding_name, "final_norm_name": self.final_norm_name,
            "head_name": self.head_name}
        if self.position_table_name:
            d["position_table_name"] = self.position_table_name
        if self.logit_scale != 1.0:
            d["logit_scale"] = self.logit_scale
        if self.embedding_scale != 1.0:
            d["embedding_scale"] = self.embedding_scale
        if self.token_table_name:
            d["token_table_name"] = self.token_table_name
            d["token_table_width"] = self.token_table_width
        if self.embedding_norm:
            d["embedding_norm"] = self.embedding_norm.to_json()
            d["embedding_norm_name"] = self.embedding_norm_name
        return d

    @staticmethod
    def from_json(d: Mapping[str, Any]) -> "ModelSpec":
        layers = tuple(LayerSpec.from_json(l) for l in d["layers"])
        return ModelSpec(
            position_table_name=d.get("position_table_name", ""),
            logit_scale=d.get("logit_scale", 1.0),
            embedding_scale=d.get("embedding_scale", 1.0),
            token_table_name=d.get("token_table_name", ""),
            token_table_width=d.get("token_table_width", 0),
            embedding_norm=PartSpec.from_json(d["embedding_norm"]) if d.get("embedding_norm") else None,
            embedding_norm_name=d.get("embedding_norm_name", "model.embed_norm"),
            architecture=d["architecture"], hidden_size=d["hidden_size"],
            vocab_size=d["vocab_size"], max_positions=d["max_positions"], layers=layers,
            run_order=tuple(RunEntry(e["layer"], e["cache_of"], bool(e.get("add_embedding", False)))
                            for e in d["run_order"]),
            final_norm=PartSpec.from_json(d["final_norm"]), tie_embeddings=d["tie_embeddings"],
            embedding_name=d["embedding_name"], final_norm_name=d["final_norm_name"],
            head_name=d["head_name"])

    def validate(self) -> None:
        _call("spec.validate", spec=self.to_json())


@dataclass(frozen=True)
class Qwen3Config:
    """The Qwen3 dense decoder's ``config.json`` keys, as the library read them."""

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
    tie_word_embeddings: bool = False
    layer_types: Tuple[str, ...] = ()
    sliding_window: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)


@dataclass(frozen=True)
class ZuzelornConfig:
    """The Zuzelorn decoder's ``config.json`` keys, as the library read them."""
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[Mapping[str, Any], ...]     # each: type, mixer {...}, mlp {...} or None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Zuzelorn"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZuzelornConfig":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)

    def __hash__(self) -> int:
        return hash(json.dumps(self.to_dict(), sort_keys=True))


@dataclass(frozen=True)
class DunavikConfig:
    """The Dunavik decoder's ``config.json`` keys, as the library read them."""
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    loop: Mapping[str, int]                   # start, stop, times
    layers: Tuple[Mapping[str, Any], ...]     # each: type, mixer {...}, mlp {...} or None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Dunavik"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DunavikConfig":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)

    def __hash__(self) -> int:
        return hash(json.dumps(self.to_dict(), sort_keys=True))


@dataclass(frozen=True)
class KefesunConfig:
    """The Kefesun decoder's ``config.json`` keys, as the library read them."""
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    taps: int                                 # canon.taps; 0: no convolution in front of the sublayers
    layers: Tuple[Mapping[str, Any], ...]     # each: type, mixer {...}, mlp {...} or None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Kefesun"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "KefesunConfig":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)

    def __hash__(self) -> int:
        return hash(json.dumps(self.to_dict(), sort_keys=True))


@dataclass(frozen=True)
class MunisunConfig:
    """The Munisun decoder's ``config.json`` keys, as the library read them."""
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    side_dim: int                             # token_side.dim; 0: no per-layer input of the token itself
    layers: Tuple[Mapping[str, Any], ...]     # each: type, mixer {left, right, ...}, mlp {...} or None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Munisun"
    _json: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)
    _spec: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MunisunConfig":
        return _wrap(_call("config.parse", config=dict(d)))

    def to_dict(self) -> Dict[str, Any]:
        return dict(self._json)

    def to_model_spec(self) -> ModelSpec:
        return ModelSpec.from_json(self._spec)

    def __hash__(self) -> int:
        return hash(json.dumps(self.to_dict(), sort_keys=True))


def _wrap(r: Mapping[str, Any]):
    c = r["config"]
    if r["architecture"] == "Munisun":
        return MunisunConfig(
            vocab=c["vocab"], width=c["width"], norm_eps=c["norm"]["eps"],
            embedding_scale=c["embedding"]["scale"], side_dim=(c.get("token_side") or {}).get("dim", 0),
            layers=tuple(c["layers"]), eos_token_ids=tuple(r["eos_token_ids"]), _json=c, _spec=r["spec"])
    if r["architecture"] == "Kefesun":
        return KefesunConfig(
            vocab=c["vocab"], width=c["width"], norm_eps=c["norm"]["eps"],
            embedding_scale=c["embedding"]["scale"], taps=(c.get("canon") or {}).get("taps", 0),
            layers=tuple(c["layers"]), eos_token_ids=tuple(r["eos_token_ids"]), _json=c, _spec=r["spec"])
    if r["architecture"] == "Dunavik":
        return DunavikConfig(
            vocab=c["vocab"], width=c["width"], norm_eps=c["norm"]["eps"],
            residual_mult=c["residual_mult"], loop=dict(c["loop"]), layers=tuple(c["layers"]),
            eos_token_ids=tuple(r["eos_token_ids"]), _json=c, _spec=r["spec"])
    if r["architecture"] == "Zuzelorn":
        return ZuzelornConfig(
            vocab=c["vocab"], width=c["width"], max_positions=c["max_positions"],
            norm_eps=c["norm"]["eps"], logit_scale=c["logit_scale"], layers=tuple(c["layers"]),
            eos_token_ids=tuple(r["eos_token_ids"]), _json=c, _spec=r["spec"])
    if r["architecture"] != "Qwen3ForCausalLM" and c.get("model_type") != "qwen3":
        raise ConfigError(f"no Python class for architecture {r['architecture']!r}")
    n = c["num_hidden_layers"]
    return Qwen3Config(
        vocab_size=c["vocab_size"], hidden_size=c["hidden_size"],
        intermediate_size=c["intermediate_size"], num_hidden_layers=n,
        num_attention_heads=c["num_attention_heads"],
        num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
        max_position_embeddings=c["max_position_embeddings"], rms_norm_eps=c["rms_norm_eps"],
        rope_theta=c["rope_theta"], tie_word_embeddings=c["tie_word_embeddings"],
        layer_types=tuple(c.get("layer_types") or ["full_attention"] * n),
        sliding_window=c.get("sliding_window"), eos_token_ids=tuple(r["eos_token_ids"]),
        architecture=r["architecture"], _json=c, _spec=r["spec"])


def known_architectures() -> list:
    return sorted(_call("config.known")["architectures"])


def config_from_dict(d: Mapping[str, Any]):
    """The typed configuration for a ``config.json`` given as a dictionary."""
    return _wrap(_call("config.parse", config=dict(d)))


def config_from_dir(model_dir: str):
    """The typed configuration of the model folder ``model_dir``."""
    return _wrap(_call("config.from_dir", dir=str(model_dir)))


__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "ZuzelornConfig", "DunavikConfig", "KefesunConfig", "MunisunConfig", "config_from_dict", "config_from_dir", "known_architectures"]
