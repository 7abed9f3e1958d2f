"""Gemosun: a decoder-only design of parallel attention / feed-forward layers over a depth-averaged residual stream.

This module only reads the design's config.json and maps it onto the generic specs of blazr_b200/layered.py (layout "depth"); the
mechanisms and their kernels are shared with any other layer-list design:

    config key                          -> spec
    vocab, width                        -> LayeredConfig.vocab / width (one residual stream, own output projection "head")
    norm.eps                            -> eps of every layer norm (weight, no bias)
    layers[i].type = "attention"        -> AttentionSpec(heads, kv_heads, dim, vdim, scale; window = mask.size, pool = mask.pool,
                                           values_from_keys, one sigmoid gate per head, no unit norm)
    layers[i].mixer.rot                 -> RotarySpec(dims, base, yarn = scaling.(factor, original, fast, slow))
    layers[i].mlp = null                -> no feed-forward branch
    layers[i].mlp.kind = "dense"        -> DenseFfSpec(ff, act = "gelu_tanh")
    layers[i].mlp.kind = "moe"          -> MoeFfSpec(router.experts, router.top, expert.ff, router.groups.(count, keep), act = "relu2",
                                           shared.ff with a sigmoid token gate)

What the design fixes is in code: both branches of a layer read the same input through two layer norms; the values are the keys as
projected; the gate of the dense feed-forward is the tanh form of gelu, the experts use a squared relu; router scores are sigmoids
and a group's score is the sum of its two best.

Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.dwa, l<i>.mix.{q,k,g,o}, l<i>.mlp.{gate,up,down},
l<i>.mlp.router, l<i>.mlp.e<j>.{up,down}, l<i>.mlp.shared.{up,down,sg}.
"""
from __future__ import annotations

from .layered import AttentionSpec, DenseFfSpec, LayeredConfig, LayerSpec, MoeFfSpec, RotarySpec

ARCHITECTURE = "Gemosun"
DENSE_ACT = "gelu_tanh"
EXPERT_ACT = "relu2"


class ConfigError(ValueError):
    pass


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config: {where} lacks '{key}'")
    return d[key]


def _rotary(rot, where: str):
    if rot is None:
        return None
    sc = rot.get("scaling")
    yarn = None
    if sc is not None:
        yarn = (float(_need(sc, "factor", where + ".rot.scaling")), float(_need(sc, "original", where + ".rot.scaling")),
                float(_need(sc, "fast", where + ".rot.scaling")), float(_need(sc, "slow", where + ".rot.scaling")))
        if yarn[0] <= 0 or yarn[2] <= 0 or yarn[3] <= 0:
            raise ConfigError(f"config: {where}: rotary scaling constants must be positive")
    spec = RotarySpec(dims=int(_need(rot, "dims", where + ".rot")), base=float(_need(rot, "base", where + ".rot")), yarn=yarn)
    if spec.dims < 2 or spec.dims % 2:
        raise ConfigError(f"config: {where}: rot.dims must be even")
    return spec


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        return DenseFfSpec(ff=int(_need(mlp, "ff", where)), act=DENSE_ACT)
    if kind == "moe":
        r = _need(mlp, "router", where)
        g = r.get("groups")
        shared = mlp.get("shared")
        spec = MoeFfSpec(experts=int(_need(r, "experts", where + ".router")), top=int(_need(r, "top", where + ".router")),
                         ff=int(_need(_need(mlp, "expert", where), "ff", where + ".expert")),
                         groups=int(_need(g, "count", where + ".router.groups")) if g else 1, keep=int(_need(g, "keep", where + ".router.groups")) if g else 1,
                         act=EXPERT_ACT, shared_ff=int(_need(shared, "ff", where + ".shared")) if shared else 0, shared_gate=True)
        if not 1 <= spec.top <= spec.experts:
            raise ConfigError(f"config: {where}: router.top must lie between 1 and router.experts")
        if spec.groups > 1 and (spec.experts % spec.groups or not 1 <= spec.keep <= spec.groups or spec.keep * (spec.experts // spec.groups) < spec.top):
            raise ConfigError(f"config: {where}: router.groups does not fit experts / top")
        return spec
    raise ConfigError(f"config: {where}: unknown feed-forward kind '{kind}'")


def parse_config(cfg: dict) -> LayeredConfig:
    out = LayeredConfig(name=ARCHITECTURE, vocab=int(_need(cfg, "vocab", "top level")), width=int(_need(cfg, "width", "top level")), streams=1, norm_groups=1,
                        eps=float(_need(_need(cfg, "norm", "top level"), "eps", "norm")), canon_taps=0, embed_scale=1.0, layout="depth", tied_head=False,
                        depth_average=True)
    for i, lay in enumerate(_need(cfg, "layers", "top level")):
        where = f"layers[{i}]"
        kind, m = _need(lay, "type", where), _need(lay, "mixer", where)
        if kind != "attention":
            raise ConfigError(f"config: {where}: unknown layer type '{kind}'")
        mask = m.get("mask") or {}
        mixer = AttentionSpec(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=int(_need(m, "dim", where)),
                              vdim=int(_need(m, "vdim", where)), scale=float(_need(m, "scale", where)), chunk=0, window=int(mask.get("size", 0)),
                              qk_unit_norm=False, gated=True, pool=int(mask.get("pool", 0)), values_from_keys=True, rot=_rotary(m.get("rot"), where))
        if mixer.heads % mixer.kv_heads:
            raise ConfigError(f"config: {where}: heads is not a multiple of kv_heads")
        if mixer.vdim != mixer.dim:
            raise ConfigError(f"config: {where}: the values are the keys, so vdim must equal dim")
        if mixer.pool > 0 and mixer.window < 1:
            raise ConfigError(f"config: {where}: mask.pool needs mask.size")
        if mixer.rot is not None and mixer.rot.dims > mixer.dim:
            raise ConfigError(f"config: {where}: rot.dims exceeds dim")
        out.layers.append(LayerSpec("attention", mixer, _feed_forward(lay.get("mlp"), where + ".mlp")))
    return out
