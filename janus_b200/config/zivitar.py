"""Typed configuration of the Zivitar decoder, read from its config.json.

Keys: `architecture` ("Zivitar"), `vocab`, `width`, `norm.eps`, optional `streams` (copies of the residual
stream, hyper-connections), optional `logit_scale` and `logit_softcap`, and `layers`: a list whose entries give
`type` ("lightning" or "attention"), the mixer's sizes and constants under `mixer`, the feed-forward under `mlp`
(null: none; `kind` "dense" with `ff` and `limit`), and optionally `weights_of`: the index of the layer whose
tensors this layer uses (with a cache or state of its own).

lightning mixer: `heads`, `dim`, `vdim`, `decay` (one per head).
attention mixer: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `diff`, optional `conv` (taps of the short
convolution), optional `mask` (`size`, `keep_first`), optional `rot` (`dims`, `base`, optional `scaling` with
`factor`, `original`, `fast`, `slow`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader

ARCHITECTURE = "Zivitar"
MAX_POSITIONS = 131072      # the design names no longest sequence; rotation tables are made for as many positions as an engine allows, at most this


def _object(data: Any, where: str) -> Dict[str, Any]:
    if not isinstance(data, dict):
        raise ConfigError(f"key '{where}' must be an object, got {data!r}")
    return data


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None     # factor, original, fast, slow

    def to_dict(self):
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self):
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    conv: int = 0                      # taps; 0: no convolution
    window: int = 0                    # mask.size; 0: every earlier key is seen
    keep_first: int = 0
    rot: Optional[RotaryConfig] = None

    def to_dict(self):
        d: Dict[str, Any] = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                             "scale": self.scale, "vdim": self.vdim}
        if self.conv:
            d["conv"] = self.conv
        if self.window:
            d["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense", "limit": self.limit}


@dataclass(frozen=True)
class ZivitarLayer:
    type: str                                   # "lightning" or "attention"
    mixer: Any                                  # LightningConfig or AttentionConfig
    mlp: Optional[DenseMlpConfig]
    weights_of: Optional[int] = None

    def to_dict(self):
        d = {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


def _read_lightning(raw: Dict[str, Any], where: str) -> LightningConfig:
    r = KeyReader(raw)
    heads = r.integer("heads")
    decay = raw.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(
            isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"key '{where}.decay' must list one number per head ({heads}), got {decay!r}")
    return LightningConfig(heads, r.integer("dim"), r.integer("vdim"), tuple(float(x) for x in decay))


def _read_attention(raw: Dict[str, Any], where: str) -> AttentionConfig:
    r = KeyReader(raw)
    heads, kv_heads = r.integer("heads"), r.integer("kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"key '{where}.heads' ({heads}) must be divisible by 'kv_heads' ({kv_heads})")
    dim = r.integer("dim")
    window = keep_first = 0
    if raw.get("mask") is not None:
        m = KeyReader(_object(raw["mask"], where + ".mask"))
        window, keep_first = m.integer("size"), m.integer("keep_first", 0, minimum=0)
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
            scaling = (s.number("factor"), s.number("original"), s.number("fast"), s.number("slow"))
        rot = RotaryConfig(dims, k.number("base"), scaling)
    diff = r.number("diff", positive=False)
    return AttentionConfig(heads, kv_heads, dim, r.integer("vdim"), r.number("scale"), diff,
                           conv=r.integer("conv", 0, minimum=0), window=window, keep_first=keep_first, rot=rot)


@dataclass(frozen=True)
class ZivitarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[ZivitarLayer, ...]
    streams: Optional[int] = None               # None: one residual stream, plain residual sums
    logit_scale: Optional[float] = None
    logit_softcap: Optional[float] = None

    ARCHITECTURE = ARCHITECTURE

    @property
    def max_positions(self) -> int:
        return MAX_POSITIONS

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def stop_token_ids(self) -> Tuple[int, ...]:
        return ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZivitarConfig":
        r = KeyReader(d)
        norm = KeyReader(_object(d.get("norm"), "norm"))
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"key 'layers' must be a non-empty list, got {type(raw_layers).__name__}")
        layers = []
        for i, raw in enumerate(raw_layers):
            where = f"layers[{i}]"
            raw = _object(raw, where)
            kind = raw.get("type")
            mixer_raw = _object(raw.get("mixer"), where + ".mixer")
            if kind == "lightning":
                mixer = _read_lightning(mixer_raw, where + ".mixer")
            elif kind == "attention":
                mixer = _read_attention(mixer_raw, where + ".mixer")
            else:
                raise ConfigError(f"key '{where}.type': unsupported value {kind!r} (supported: 'lightning', 'attention')")
            mlp = None
            if raw.get("mlp") is not None:
                m = _object(raw["mlp"], where + ".mlp")
                if m.get("kind") != "dense":
                    raise ConfigError(f"key '{where}.mlp.kind': unsupported value {m.get('kind')!r} (supported: 'dense')")
                mk = KeyReader(m)
                mlp = DenseMlpConfig(mk.integer("ff"), mk.number("limit"))
            weights_of = raw.get("weights_of")
            if weights_of is not None:
                if isinstance(weights_of, bool) or not isinstance(weights_of, int) or not 0 <= weights_of < len(raw_layers) \
                        or weights_of == i:
                    raise ConfigError(f"key '{where}.weights_of' must name another layer, got {weights_of!r}")
            layers.append(ZivitarLayer(kind, mixer, mlp, weights_of))
        cfg = cls(vocab=r.integer("vocab"), width=r.integer("width"), eps=norm.number("eps"), layers=tuple(layers),
                  streams=r.integer("streams", None), logit_scale=r.number("logit_scale", None),
                  logit_softcap=r.number("logit_softcap", None))
        for i, layer in enumerate(cfg.layers):
            seen = {i}
            j = i
            while cfg.layers[j].weights_of is not None:
                j = cfg.layers[j].weights_of
                if j in seen:
                    raise ConfigError(f"key 'layers[{i}].weights_of' leads in a circle")
                seen.add(j)
            if j != i and (cfg.layers[j].type != layer.type or cfg.layers[j].mixer != layer.mixer
                           or cfg.layers[j].mlp != layer.mlp):
                raise ConfigError(f"layers[{i}] uses the tensors of layer {j} but differs from it in its sizes")
        if cfg.streams is not None and cfg.streams > 8:
            raise ConfigError(f"key 'streams' must be at most 8, got {cfg.streams}")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "layers": [layer.to_dict() for layer in self.layers],
                             "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        for key in ("streams", "logit_scale", "logit_softcap"):
            if getattr(self, key) is not None:
                d[key] = getattr(self, key)
        return d
