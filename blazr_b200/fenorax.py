"""Fenorax: a decoder-only design of state-space and chunked-attention layers over several residual streams.

This module only reads the design's config.json and maps it onto the generic specs of blazr_b200/layered.py; the mechanisms
themselves (and their kernels) are shared with any other layer-list design:

    config key                      -> spec
    vocab, width, streams           -> LayeredConfig.vocab / width / streams
    norm.eps, norm.groups           -> eps, norm_groups (every norm of the model, the unit norms of q / k included)
    canon.taps                      -> canon_taps (convolution in front of every sublayer)
    embedding.scale                 -> embed_scale
    layers[i].type = "mamba2"       -> SsmSpec(heads, vdim, state, groups, norm_groups, conv)
    layers[i].type = "attention"    -> AttentionSpec(heads, kv_heads, dim, vdim, scale, chunk = mask.size), no rotation,
                                       unit-RMS q and k, one sigmoid gate per head
    layers[i].mlp = null | {kind: "dense", ff, limit} -> DenseFfSpec(ff, limit, alpha = 1.702, up_shift = 1)

Tensor names: embed, final.norm, l<i>.norm<q>, l<i>.canon<q>, l<i>.hc<q>.{in,out,mix}, l<i>.mix.*, l<i>.mlp.{gate,up,down}.
The output projection is the embedding table itself (without the embedding scale).
"""
from __future__ import annotations

from .layered import AttentionSpec, DenseFfSpec, LayeredConfig, LayerSpec, SsmSpec

ARCHITECTURE = "Fenorax"
GATE_ALPHA = 1.702   # fixed by the design: gate * sigmoid(1.702 * gate) * (up + 1)
UP_SHIFT = 1.0


class ConfigError(ValueError):
    pass


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config: {where} lacks '{key}'")
    return d[key]


def parse_config(cfg: dict) -> LayeredConfig:
    out = LayeredConfig(name=ARCHITECTURE, vocab=int(_need(cfg, "vocab", "top level")), width=int(_need(cfg, "width", "top level")),
                        streams=int(cfg.get("streams", 1)), norm_groups=int(_need(_need(cfg, "norm", "top level"), "groups", "norm")),
                        eps=float(_need(cfg["norm"], "eps", "norm")), canon_taps=int(_need(_need(cfg, "canon", "top level"), "taps", "canon")),
                        embed_scale=float(_need(_need(cfg, "embedding", "top level"), "scale", "embedding")))
    if out.width % out.norm_groups:
        raise ConfigError("config: width is not divisible by norm.groups")
    for i, lay in enumerate(_need(cfg, "layers", "top level")):
        where = f"layers[{i}]"
        kind, m = _need(lay, "type", where), _need(lay, "mixer", where)
        if kind == "mamba2":
            mixer = SsmSpec(heads=int(_need(m, "heads", where)), vdim=int(_need(m, "vdim", where)), state=int(_need(m, "state", where)),
                            groups=int(_need(m, "groups", where)), norm_groups=int(_need(m, "norm_groups", where)), conv=int(_need(m, "conv", where)))
            if mixer.heads % mixer.groups or (mixer.heads * mixer.vdim) % mixer.norm_groups:
                raise ConfigError(f"config: {where}: heads / groups / norm_groups do not divide")
            spec_kind = "ssm"
        elif kind == "attention":
            mask = m.get("mask") or {}
            mixer = AttentionSpec(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=int(_need(m, "dim", where)),
                                  vdim=int(_need(m, "vdim", where)), scale=float(_need(m, "scale", where)), chunk=int(mask.get("size", 0)), window=0,
                                  qk_unit_norm=True, gated=True)
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"config: {where}: heads is not a multiple of kv_heads")
            spec_kind = "attention"
        else:
            raise ConfigError(f"config: {where}: unknown layer type '{kind}'")
        mlp = lay.get("mlp")
        ff = None
        if mlp is not None:
            if _need(mlp, "kind", where + ".mlp") != "dense":
                raise ConfigError(f"config: {where}: unknown feed-forward kind '{mlp['kind']}'")
            ff = DenseFfSpec(ff=int(_need(mlp, "ff", where + ".mlp")), limit=float(_need(mlp, "limit", where + ".mlp")), alpha=GATE_ALPHA, up_shift=UP_SHIFT)
        out.layers.append(LayerSpec(spec_kind, mixer, ff))
    return out
