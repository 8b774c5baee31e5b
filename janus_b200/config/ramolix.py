"""Typed configuration of the Ramolix decoder, read from its config.json.

Keys: `architecture` ("Ramolix"), `vocab`, `width`, `norm.eps`, `embedding.scale` (the embedding is multiplied by
it), `residual_mult` (what a sublayer adds to the residual stream is multiplied by it), and `layers`: a list whose
entries give `type` ("attention", "latent_attention" or "mamba2"), the mixer's sizes and constants under `mixer`,
and the feed-forward under `mlp` (null: none; `kind` "dense" with `ff`).

attention mixer: `heads`, `kv_heads`, `dim`, `vdim` (the values are the projected keys: equal to `dim`), `scale`,
optional `mask` (`size`: the sliding window), optional `rot` (`dims`, `base`, optional `scaling` with `factor`,
`low`, `high`, `original`).
latent_attention mixer: `heads`, `dim`, `vdim`, `kv_rank`, `scale`, optional `kv_from` (the index of the earlier
layer whose cached latents this layer attends over; it then has no latent projection of its own).
mamba2 mixer: `heads`, `vdim`, `state`, `groups`, `conv` (taps), `norm_groups`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader

ARCHITECTURE = "Ramolix"
MAX_POSITIONS = 131072      # the design names no longest sequence; rotation tables are made for as many positions as an engine allows, at most this


def _object(data: Any, where: str) -> Dict[str, Any]:
    if not isinstance(data, dict):
        raise ConfigError(f"key '{where}' must be an object, got {data!r}")
    return data


@dataclass(frozen=True)
class BandRotaryConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None     # factor, low, high, original

    def to_dict(self):
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return d


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: int = 0                    # mask.size; 0: every earlier key is seen
    rot: Optional[BandRotaryConfig] = None

    def to_dict(self):
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.dim}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    kv_from: Optional[int] = None

    def to_dict(self):
        d: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "scale": self.scale,
                             "vdim": self.vdim}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self):
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class GeluMlpConfig:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class RamolixLayer:
    type: str                                   # "attention", "latent_attention" or "mamba2"
    mixer: Any
    mlp: Optional[GeluMlpConfig]

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


def _read_attention(raw: Dict[str, Any], where: str) -> WindowAttentionConfig:
    r = KeyReader(raw)
    heads, kv_heads, dim = r.integer("heads"), r.integer("kv_heads"), r.integer("dim")
    if heads % kv_heads:
        raise ConfigError(f"key '{where}.heads' ({heads}) must be divisible by 'kv_heads' ({kv_heads})")
    vdim = r.integer("vdim", dim)
    if vdim != dim:
        raise ConfigError(f"key '{where}.vdim' ({vdim}) must equal 'dim' ({dim}): the values are the projected keys")
    window = 0
    if raw.get("mask") is not None:
        window = KeyReader(_object(raw["mask"], where + ".mask")).integer("size")
    rot = None
    if raw.get("rot") is not None:
        rr = _object(raw["rot"], where + ".rot")
        k = KeyReader(rr)
        dims = k.integer("dims")
        if dims % 2 or dims > dim:
            raise ConfigError(f"key '{where}.rot.dims' must be even and at most 'dim' ({dim}), got {dims}")
        scaling = None
        if rr.get("scaling") is not None:
            s = KeyReader(_object(rr["scaling"], where + ".rot.scaling"))
            scaling = (s.number("factor"), s.number("low"), s.number("high"), s.number("original"))
        rot = BandRotaryConfig(dims, k.number("base"), scaling)
    return WindowAttentionConfig(heads, kv_heads, dim, r.number("scale"), window=window, rot=rot)


def _read_latent(raw: Dict[str, Any], where: str) -> LatentAttentionConfig:
    r = KeyReader(raw)
    return LatentAttentionConfig(r.integer("heads"), r.integer("dim"), r.integer("vdim"), r.integer("kv_rank"),
                                 r.number("scale"), kv_from=r.integer("kv_from", None, minimum=0))


def _read_mamba2(raw: Dict[str, Any], where: str) -> Mamba2Config:
    r = KeyReader(raw)
    heads, groups = r.integer("heads"), r.integer("groups")
    if heads % groups:
        raise ConfigError(f"key '{where}.heads' ({heads}) must be divisible by 'groups' ({groups})")
    vdim, norm_groups = r.integer("vdim"), r.integer("norm_groups")
    if (heads * vdim) % norm_groups:
        raise ConfigError(f"key '{where}.norm_groups' ({norm_groups}) must divide heads * vdim ({heads * vdim})")
    return Mamba2Config(heads, vdim, r.integer("state"), groups, r.integer("conv"), norm_groups)


_READERS = {"attention": _read_attention, "latent_attention": _read_latent, "mamba2": _read_mamba2}


@dataclass(frozen=True)
class RamolixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[RamolixLayer, ...]

    ARCHITECTURE = ARCHITECTURE

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RamolixConfig":
        r = KeyReader(d)
        norm = KeyReader(_object(d.get("norm"), "norm"))
        embedding = KeyReader(_object(d.get("embedding"), "embedding"))
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"key 'layers' must be a non-empty list, got {type(raw_layers).__name__}")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            raw = _object(raw, where)
            kind = raw.get("type")
            if kind not in _READERS:
                raise ConfigError(f"key '{where}.type': unsupported value {kind!r} (supported: "
                                  f"{', '.join(repr(k) for k in sorted(_READERS))})")
            mixer = _READERS[kind](_object(raw.get("mixer"), where + ".mixer"), where + ".mixer")
            mlp = None
            if raw.get("mlp") is not None:
                m = _object(raw["mlp"], where + ".mlp")
                if m.get("kind") != "dense":
                    raise ConfigError(f"key '{where}.mlp.kind': unsupported value {m.get('kind')!r} (supported: 'dense')")
                mlp = GeluMlpConfig(KeyReader(m).integer("ff"))
            layers.append(RamolixLayer(kind, mixer, mlp))
        for i, layer in enumerate(layers):
            j = layer.mixer.kv_from if layer.type == "latent_attention" else None
            if j is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if j >= i or layers[j].type != "latent_attention" or layers[j].mixer.kv_from is not None:
                raise ConfigError(f"key '{where}' must name an earlier latent_attention layer with a latent of its own, "
                                  f"got {j}")
            if layers[j].mixer.kv_rank != layer.mixer.kv_rank:
                raise ConfigError(f"key '{where}': layer {j} has kv_rank {layers[j].mixer.kv_rank}, this layer "
                                  f"{layer.mixer.kv_rank}")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"), eps=norm.number("eps"),
                   embedding_scale=embedding.number("scale"), residual_mult=r.number("residual_mult", 1.0),
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": ARCHITECTURE, "embedding": {"scale": self.embedding_scale},
                "layers": [layer.to_dict() for layer in self.layers], "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
