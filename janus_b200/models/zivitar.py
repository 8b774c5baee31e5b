"""The Zivitar decoder as data: a `ModelSpec` made from a `ZivitarConfig`.

Layers are lightning mixers (linear attention with decay, `parts.lightning`) or differential attention
(`parts.diff_attention`), each followed by a clamped gated feed-forward (or none), pre-norm, with the residual
kept in `streams` copies joined by hyper-connections (`parts.connection`) when the configuration has the key.
A layer that names `weights_of` is the same `LayerSpec` run at a second place of the schedule: same tensors, a
cache or state of its own.  Logits are scaled and soft-capped.  Tensor names: `embed`, `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `l<i>.hc1.*`, `l<i>.hc2.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from typing import Dict, List

from ..config.registry import register_architecture
from ..config.zivitar import ZivitarConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer_spec(config: ZivitarConfig, i: int) -> PartSpec:
    layer, p = config.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "lightning":
        return PartSpec("lightning_attention",
                        dict(hidden_size=config.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim, decay=tuple(m.decay),
                             eps=config.eps),
                        weights={n: p + n for n in ("q", "k", "v", "g", "o", "norm")})
    position = None
    if m.rot is not None:
        scaling = None if m.rot.scaling is None else dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
        position = PartSpec("ramped_rotary", dict(dims=m.rot.dims, theta=m.rot.base, max_positions=config.max_positions,
                                                  scaling=scaling))
    weights = {n: p + n for n in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}
    if m.conv:
        weights.update(q_conv=p + "q.conv", k_conv=p + "k.conv", v_conv=p + "v.conv")
    return PartSpec("differential_attention",
                    dict(hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                         scale=m.scale, diff=m.diff, eps=config.eps, conv_taps=m.conv, window=m.window,
                         keep_first=m.keep_first, position=position, rotary_dims=0 if m.rot is None else m.rot.dims),
                    weights=weights)


def zivitar_spec(config: ZivitarConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    index_of: Dict[int, int] = {}           # configuration layer with tensors of its own -> index among the LayerSpecs
    for i, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        p = f"l{i}."
        norm = lambda name: PartSpec("rms_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma=p + name))  # noqa: E731
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec("clamped_glu", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff,
                                                        limit=layer.mlp.limit),
                                    weights=dict(gate=p + "mlp.gate", up=p + "mlp.up", down=p + "mlp.down"))
        extra = ()
        if config.streams is not None:
            def connection(q: int) -> PartSpec:
                return PartSpec("hyper_connection", dict(streams=config.streams, width=config.width),
                                weights=dict(into=p + f"hc{q}.in", out=p + f"hc{q}.out", mix=p + f"hc{q}.mix"))
            extra = (("mixer_connection", "connection", connection(1)),)
            if feed_forward is not None:
                extra += (("feed_forward_connection", "connection", connection(2)),)
        index_of[i] = len(layers)
        layers.append(LayerSpec(mixer=_mixer_spec(config, i), feed_forward=feed_forward, mixer_norm=norm("norm1"),
                                feed_forward_norm=norm("norm2") if feed_forward is not None else None,
                                arrangement="pre_norm" if config.streams is None else "hyper_pre_norm", extra=extra))
    transforms = ()
    if config.logit_scale is not None or config.logit_softcap is not None:
        transforms = (PartSpec("scale_soft_cap", dict(scale=1.0 if config.logit_scale is None else config.logit_scale,
                                                      cap=config.logit_softcap)),)
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index_of[config.owner(i)]) for i in range(len(config.layers))),
        final_norm=PartSpec("rms_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma="final.norm")),
        embedding_weight="embed", head_weight="head", max_positions=config.max_positions,
        logit_transforms=transforms, residual_streams=config.streams or 1, pad_head_width=True)


def build_zivitar(config: ZivitarConfig, dtype, device):
    from ..engine.model import DecoderModel
    return DecoderModel(zivitar_spec(config), dtype, device)


def zivitar_weight_specs(config: ZivitarConfig):
    from ..engine.model import model_weight_specs
    return model_weight_specs(zivitar_spec(config))


register_architecture(ZivitarConfig.ARCHITECTURE, ZivitarConfig, build_zivitar, zivitar_weight_specs)
