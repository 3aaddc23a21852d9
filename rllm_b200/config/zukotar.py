"""Typed configuration of the Zukotar design, read from its own config.json keys.

A Zukotar model is a list of layers, each with a mixer (`latent_attention` or `gla`) and a routed
feed-forward or none, of which a stretch may run several times with the same weights (`loop`).
config.json gives every size and every constant: nothing here assumes a value. Keys:

    architecture            "Zukotar"
    vocab, width            sizes of the embedding table
    embedding.scale         factor on the embedded rows
    norm.eps                eps of every RMS norm
    layers[i].type          the mixer's kind
    layers[i].mixer         its sizes: latent_attention {heads, dim, rot_dim, vdim, kv_rank, scale,
                            rot {base, dims}, mask {size} or absent}; gla {heads, dim, vdim, tau; optionally decay_rank, which a
                            checkpoint's tensors give otherwise}
    layers[i].mlp           null, or {kind "moe", expert {ff}, router {experts, top, groups {count, keep}
                            or absent}}
    loop                    absent/null, or {start, stop, times}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, ModelConfig, require_float, require_int


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
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query/key dimensions per head
    rot_dim: int             # rotated query/key dimensions per head (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float             # factor on the scores
    rot_base: float
    rot_dims: int            # how many of the rot_dim dimensions are rotated
    window: int | None       # a query sees itself and the window - 1 positions before it; None: all

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LatentAttentionConfig":
        rot = _obj(m, "rot", where)
        mask = _obj(m, "mask", where, optional=True)
        c = cls(require_int(m, "heads"), require_int(m, "dim"), require_int(m, "rot_dim", minimum=0),
                require_int(m, "vdim"), require_int(m, "kv_rank"), require_float(m, "scale"),
                require_float(rot, "base"), require_int(rot, "dims", minimum=0),
                None if mask is None else require_int(mask, "size"))
        if c.rot_dims > c.rot_dim or c.rot_dims % 2:
            raise ConfigError(f"{where}: rot.dims {c.rot_dims} must be even and at most rot_dim {c.rot_dim}")
        return c

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
             "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class GLAConfig:
    heads: int
    dim: int                 # key channels per head
    vdim: int
    tau: float               # the decay is sigmoid(z) ^ (1 / tau)
    decay_rank: int | None = None    # rows of the decay's first projection; None: the checkpoint's tensor says

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "GLAConfig":
        c = cls(require_int(m, "heads"), require_int(m, "dim"), require_int(m, "vdim"), require_float(m, "tau"),
                None if m.get("decay_rank") is None else require_int(m, "decay_rank"))
        if not c.tau > 0:
            raise ConfigError(f"{where}: tau must be positive, got {c.tau}")
        return c

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class MoEConfig:
    ff: int
    experts: int
    top: int
    groups: int = 1          # experts form `groups` equal groups of neighbours
    keep: int = 1            # only experts of the best `keep` groups can be chosen

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "MoEConfig":
        kind = m.get("kind")
        if kind != "moe":
            raise ConfigError(f"{where}: feed-forward kind {kind!r} is not known (known: 'moe')")
        router = _obj(m, "router", where)
        groups = _obj(router, "groups", where, optional=True)
        c = cls(require_int(_obj(m, "expert", where), "ff"), require_int(router, "experts"), require_int(router, "top"),
                1 if groups is None else require_int(groups, "count"),
                1 if groups is None else require_int(groups, "keep"))
        if c.experts % c.groups or c.keep > c.groups:
            raise ConfigError(f"{where}: {c.experts} experts do not form {c.groups} equal groups of which {c.keep} are kept")
        if c.top > c.experts // c.groups * c.keep:
            raise ConfigError(f"{where}: top {c.top} exceeds the experts of the kept groups")
        return c

    def to_dict(self) -> dict:
        r: dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            r["groups"] = {"count": self.groups, "keep": self.keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": r}


MIXER_CONFIGS = {"latent_attention": LatentAttentionConfig, "gla": GLAConfig}


@dataclass(frozen=True)
class ZukotarLayer:
    type: str
    mixer: Any
    mlp: MoEConfig | None


@dataclass(frozen=True)
class ZukotarConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1      # layers loop_start .. loop_stop-1 run this many times in a row
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ZukotarConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_CONFIGS:
                raise ConfigError(f"{where}: 'type' must be one of {sorted(MIXER_CONFIGS)}, got "
                                  f"{L.get('type') if isinstance(L, dict) else L!r}")
            mixer = MIXER_CONFIGS[L["type"]].from_dict(_obj(L, "mixer", where), where + ".mixer")
            mlp = L.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"{where}: 'mlp' must be an object or null")
            layers.append(ZukotarLayer(L["type"], mixer, None if mlp is None else MoEConfig.from_dict(mlp, where + ".mlp")))
        loop = _obj(raw, "loop", "config.json", optional=True)
        start = stop = 0
        times = 1
        if loop is not None:
            start, stop = require_int(loop, "start", minimum=0), require_int(loop, "stop", minimum=0)
            times = require_int(loop, "times", minimum=1)
            if not start < stop <= len(layers):
                raise ConfigError(f"loop: start {start} < stop {stop} <= {len(layers)} layers does not hold")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (eos,)
        return cls(require_int(raw, "vocab"), require_int(raw, "width"),
                   require_float(_obj(raw, "embedding", "config.json"), "scale"),
                   require_float(_obj(raw, "norm", "config.json"), "eps"), tuple(layers), start, stop, times,
                   tuple(int(e) for e in eos))

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def layer_runs(self) -> list[tuple[int, int | None]]:
        """[(layer, pass number if the run begins a pass of the loop, else None)] in running order."""
        n = len(self.layers)
        if not self.has_loop:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, None) for i in range(self.loop_stop, n)]

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": "Zukotar", "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers]}
        if self.has_loop:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
