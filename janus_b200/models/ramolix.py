"""The Ramolix decoder as data: a `ModelSpec` made from a `RamolixConfig`.

Layers are sliding-window attention whose values are its projected keys (`parts.shared_kv_attention`), latent
attention (`parts.latent_attention`; a layer with `kv_from` is a place of the schedule that reads the latents an
earlier place cached) or the selective state-space mixer (`parts.mamba2`), each followed by a GELU-gated
feed-forward (or none).  The norms sit on the sublayers' outputs and what joins the residual stream is multiplied
by a constant (arrangement `output_norm`); the embedding is scaled; the head is the embedding table itself.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.
"""
from __future__ import annotations

from typing import Dict, List

from ..config.ramolix import RamolixConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer_spec(config: RamolixConfig, i: int) -> PartSpec:
    layer, p = config.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "mamba2":
        return PartSpec("mamba2",
                        dict(hidden_size=config.width, num_heads=m.heads, vdim=m.vdim, state=m.state, groups=m.groups,
                             conv_taps=m.conv, norm_groups=m.norm_groups, eps=config.eps),
                        weights=dict(in_proj=p + "in", conv=p + "conv", conv_bias=p + "conv.b", dt_bias=p + "dt_bias",
                                     A_log=p + "A_log", D=p + "D", norm=p + "norm", o=p + "o"))
    if layer.type == "latent_attention":
        own = m.kv_from is None
        weights = dict(q=p + "q", uk=p + "uk", uv=p + "uv", o=p + "o")
        if own:
            weights.update(dkv=p + "dkv", dkv_norm=p + "dkv.norm")
        return PartSpec("latent_attention",
                        dict(hidden_size=config.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim, rank=m.kv_rank,
                             scale=m.scale, eps=config.eps, own_latent=own), weights=weights)
    position = None
    if m.rot is not None:
        scaling = None if m.rot.scaling is None else dict(zip(("factor", "low", "high", "original"), m.rot.scaling))
        position = PartSpec("band_rotary", dict(dims=m.rot.dims, theta=m.rot.base, max_positions=config.max_positions,
                                                scaling=scaling))
    return PartSpec("shared_kv_attention",
                    dict(hidden_size=config.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, scale=m.scale,
                         eps=config.eps, window=m.window, position=position,
                         rotary_dims=0 if m.rot is None else m.rot.dims, bias=True),
                    weights=dict(q=p + "q", k=p + "k", q_bias=p + "q.b", k_bias=p + "k.b", q_norm=p + "q.norm",
                                 k_norm=p + "k.norm", o=p + "o"))


def ramolix_spec(config: RamolixConfig) -> ModelSpec:
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        norm = lambda name: PartSpec("rms_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma=p + name))  # noqa: E731
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec("gelu_glu", dict(hidden_size=config.width, intermediate_size=layer.mlp.ff),
                                    weights=dict(gate=p + "mlp.gate", up=p + "mlp.up", down=p + "mlp.down"))
        layers.append(LayerSpec(mixer=_mixer_spec(config, i), feed_forward=feed_forward, mixer_norm=norm("norm1"),
                                feed_forward_norm=norm("norm2") if feed_forward is not None else None,
                                arrangement="output_norm",
                                arrangement_params=(("residual_mult", config.residual_mult),)))
        kv_from = layer.mixer.kv_from if layer.type == "latent_attention" else None
        schedule.append(ScheduleEntry(i, reads_cache_of=kv_from))      # layers and places have the same numbers
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rms_norm", dict(width=config.width, eps=config.eps), weights=dict(gamma="final.norm")),
        embedding_weight="embed", head_weight=None, max_positions=config.max_positions,
        embedding_transforms=(PartSpec("scale_soft_cap", dict(scale=config.embedding_scale)),),
        pad_head_width=True)


def build_ramolix(config: RamolixConfig, dtype, device):
    from ..engine.model import DecoderModel
    return DecoderModel(ramolix_spec(config), dtype, device)


def ramolix_weight_specs(config: RamolixConfig):
    from ..engine.model import model_weight_specs
    return model_weight_specs(ramolix_spec(config))


register_architecture(RamolixConfig.ARCHITECTURE, RamolixConfig, build_ramolix, ramolix_weight_specs)
