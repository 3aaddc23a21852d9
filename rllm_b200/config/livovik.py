"""Typed configuration of the Livovik design, read from its own config.json keys.

A Livovik model is a list of post-norm layers: x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)).
The mixer is grouped-query attention with a per-head norm of queries and keys, a rotation of part of each
head, a block mask, a sink in the softmax and an output gate; the feed-forward is dense (relu squared),
a mixture of gated experts with sigmoid scores and an optional shared expert, or absent. A layer may run on
another layer's tensors. config.json gives every size and every constant; nothing here assumes a value. Keys:

    architecture            "Livovik"
    vocab, width            sizes of the embedding table and of the output matrix
    norm.eps                eps of every RMS norm
    postln_alpha            factor on the stream where a sublayer's output is added
    layers[i].type          "attention"
    layers[i].mixer         {heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, low, high,
                            original} or absent} or absent, mask {size} or absent}
    layers[i].mlp           null, {kind "dense", ff}, or {kind "moe", expert {ff}, router {experts, top},
                            shared {ff} or absent}
    layers[i].weights_of    absent, or the layer whose tensors this one runs on
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, ModelConfig, require_float, require_int
from .llama import RopeScaling


def _obj(raw: dict, key: str, where: str, optional: bool = False):
    v = raw.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"{where} lacks required key {key!r}")
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {key!r} must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                      # query/key size per head
    vdim: int                     # value size per head
    scale: float                  # factor on the scores
    rot_dims: int = 0             # how many of a head's dimensions are rotated (0: none)
    rot_base: float = 10000.0
    rot_scaling: RopeScaling | None = None
    chunk: int | None = None      # a query sees only its own block of this many positions; None: all before it

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "SinkAttentionConfig":
        rot = _obj(m, "rot", where, optional=True)
        mask = _obj(m, "mask", where, optional=True)
        dims, base, scaling = 0, 10000.0, None
        if rot is not None:
            dims, base = require_int(rot, "dims", minimum=0), require_float(rot, "base")
            sc = _obj(rot, "scaling", where + ".rot", optional=True)
            if sc is not None:
                orig = require_float(sc, "original")
                scaling = RopeScaling("llama3", require_float(sc, "factor"), require_float(sc, "low"),
                                      require_float(sc, "high"), int(orig) if orig == int(orig) else orig)
                if scaling.factor <= 0 or scaling.high_freq_factor <= scaling.low_freq_factor:
                    raise ConfigError(f"{where}.rot.scaling: factor must be positive and high above low")
        c = cls(require_int(m, "heads"), require_int(m, "kv_heads"), require_int(m, "dim"), require_int(m, "vdim"),
                require_float(m, "scale"), dims, base, scaling, None if mask is None else require_int(mask, "size"))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{where}: {c.heads} heads do not divide over {c.kv_heads} kv_heads")
        if c.rot_dims % 2 or c.rot_dims > c.dim:
            raise ConfigError(f"{where}: rot.dims {c.rot_dims} must be even and at most dim {c.dim}")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                s = self.rot_scaling
                d["rot"]["scaling"] = {"factor": s.factor, "low": s.low_freq_factor, "high": s.high_freq_factor,
                                       "original": s.original_max_position_embeddings}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class LivovikMLP:
    kind: str                     # "dense" or "moe"
    ff: int                       # inner size (of one expert for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None  # inner size of the expert every token uses; None: there is none

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LivovikMLP":
        kind = m.get("kind")
        if kind == "dense":
            return cls("dense", require_int(m, "ff"))
        if kind == "moe":
            router = _obj(m, "router", where)
            shared = _obj(m, "shared", where, optional=True)
            c = cls("moe", require_int(_obj(m, "expert", where), "ff"), require_int(router, "experts"),
                    require_int(router, "top"), None if shared is None else require_int(shared, "ff"))
            if c.top > c.experts:
                raise ConfigError(f"{where}: top {c.top} exceeds the {c.experts} experts")
            return c
        raise ConfigError(f"{where}: feed-forward kind {kind!r} is not known (known: 'dense', 'moe')")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class LivovikLayer:
    type: str
    mixer: SinkAttentionConfig
    mlp: LivovikMLP | None
    weights_of: int | None = None     # the layer whose tensors this one runs on


@dataclass(frozen=True)
class LivovikConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: tuple
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LivovikConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            if isinstance(L, dict) and L.get("weights_of") is not None:
                # an entry that names another layer's tensors may leave out what it shares with that layer
                j, seen = L["weights_of"], {i}
                while isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(layers_raw) and j not in seen \
                        and isinstance(layers_raw[j], dict):
                    seen.add(j)
                    L = {**{k: v for k, v in layers_raw[j].items() if k != "weights_of"}, **L}
                    j = layers_raw[j].get("weights_of")
            if not isinstance(L, dict) or L.get("type") != "attention":
                raise ConfigError(f"{where}: 'type' must be 'attention', got {L.get('type') if isinstance(L, dict) else L!r}")
            mixer = SinkAttentionConfig.from_dict(_obj(L, "mixer", where), where + ".mixer")
            mlp = L.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            src = L.get("weights_of")
            if src is not None:
                src = require_int(L, "weights_of", minimum=0)
                if src >= len(layers_raw) or src == i:
                    raise ConfigError(f"{where}: weights_of {src} names no other layer")
            layers.append(LivovikLayer("attention", mixer, None if mlp is None else LivovikMLP.from_dict(mlp, where + ".mlp"),
                                       src))
        cfg = cls(require_int(raw, "vocab"), require_int(raw, "width"),
                  require_float(_obj(raw, "norm", "config.json"), "eps"), require_float(raw, "postln_alpha"),
                  tuple(layers), cls._eos(raw))
        for i, L in enumerate(layers):
            if L.weights_of is not None:
                j = cfg.owner(i)
                if (layers[j].mixer, layers[j].mlp) != (L.mixer, L.mlp):
                    raise ConfigError(f"layers[{i}] runs on layer {j}'s tensors but differs from it")
        return cfg

    @staticmethod
    def _eos(raw) -> tuple:
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        return tuple(int(e) for e in eos)

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs on (itself, if it has its own)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}]: weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def to_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            d = {"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
            if L.weights_of is not None:
                d["weights_of"] = L.weights_of
            layers.append(d)
        d = {"architecture": "Livovik", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "postln_alpha": self.postln_alpha, "layers": layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
