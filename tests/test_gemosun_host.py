"""Host side of the Gemosun design (no GPU): the configuration reader and its errors, the rotary frequency table against the plain
restatement, the registry, the activation names."""
import copy
import json

import numpy as np
import pytest

import gemosun_oracle as O
from blazr_b200 import gemosun, registry
from blazr_b200.layered import DenseFfSpec, MoeFfSpec, RotarySpec

CFG = {"architecture": "Gemosun", "vocab": 50, "width": 32, "norm": {"eps": 1e-4}, "layers": [
    {"type": "attention", "mixer": {"dim": 8, "vdim": 8, "heads": 4, "kv_heads": 2, "scale": 0.25, "mask": {"size": 9, "pool": 3},
                                    "rot": {"dims": 6, "base": 77.0, "scaling": {"factor": 2.5, "original": 40, "fast": 6.0, "slow": 0.5}}},
     "mlp": {"kind": "dense", "ff": 20}},
    {"type": "attention", "mixer": {"dim": 8, "vdim": 8, "heads": 2, "kv_heads": 2, "scale": 0.5}, "mlp": None},
    {"type": "attention", "mixer": {"dim": 8, "vdim": 8, "heads": 2, "kv_heads": 1, "scale": 0.5, "mask": {"size": 4}, "rot": {"dims": 8, "base": 10.0}},
     "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": 10}}},
    {"type": "attention", "mixer": {"dim": 8, "vdim": 8, "heads": 2, "kv_heads": 1, "scale": 0.5},
     "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 3}}}]}


def test_config_maps_onto_the_generic_specs():
    c = registry.LAYERED["Gemosun"](CFG)
    assert (c.layout, c.tied_head, c.streams, c.canon_taps, c.vocab, c.width, c.eps) == ("depth", False, 1, 0, 50, 32, 1e-4)
    a = c.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.pool, a.chunk) == (4, 2, 8, 8, 0.25, 9, 3, 0)
    assert a.values_from_keys and a.gated and not a.qk_unit_norm
    assert a.rot == RotarySpec(6, 77.0, (2.5, 40.0, 6.0, 0.5))
    assert c.layers[0].ff == DenseFfSpec(ff=20, act="gelu_tanh")
    b = c.layers[1]
    assert b.ff is None and b.mixer.window == 0 and b.mixer.pool == 0 and b.mixer.rot is None
    assert c.layers[2].mixer.rot == RotarySpec(8, 10.0, None) and c.layers[2].mixer.pool == 0
    assert c.layers[2].ff == MoeFfSpec(experts=6, top=2, ff=12, groups=3, keep=2, act="relu2", shared_ff=10, shared_gate=True)
    assert c.layers[3].ff == MoeFfSpec(experts=3, top=3, ff=12, groups=1, keep=1, act="relu2", shared_ff=0, shared_gate=True)


def _broken(edit):
    c = copy.deepcopy(CFG)
    edit(c)
    return c


@pytest.mark.parametrize("edit", [
    lambda c: c.pop("vocab"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="mamba2"),
    lambda c: c["layers"][0]["mixer"].update(vdim=16), lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10),
    lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), lambda c: c["layers"][0]["mlp"].update(kind="glu"),
    lambda c: c["layers"][2]["mlp"]["router"].update(top=7), lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(count=4),
    lambda c: c["layers"][2]["mlp"]["router"]["groups"].update(keep=0), lambda c: c["layers"][2]["mlp"]["router"].update(top=5),
    lambda c: c["layers"][2]["mlp"].pop("expert")])
def test_config_errors_are_named(edit):
    with pytest.raises(gemosun.ConfigError):
        gemosun.parse_config(_broken(edit))


@pytest.mark.parametrize("rot", [{"dims": 6, "base": 77.0, "scaling": {"factor": 2.5, "original": 40, "fast": 6.0, "slow": 0.5}},
                                 {"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}},
                                 {"dims": 4, "base": 3.0, "scaling": {"factor": 2.0, "original": 8, "fast": 100.0, "slow": 50.0}},
                                 {"dims": 16, "base": 500.0}])
def test_rotary_table_follows_the_restatement(rot):
    sc = rot.get("scaling")
    spec = RotarySpec(rot["dims"], rot["base"], (sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None)
    freq, amp = spec.table()
    f, a = O.rotary_frequencies(rot)
    assert freq.dtype == np.float32 and np.allclose(freq, np.asarray(f), rtol=1e-7, atol=0) and abs(amp - a) < 1e-12
    if sc:
        assert np.all(freq <= np.asarray([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=np.float32) * (1 + 1e-6))


def test_registry_picks_the_design_by_its_config(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert registry.architecture_of(str(tmp_path)) == "Gemosun"
    assert set(registry.LAYERED) >= {"Fenorax", "Gemosun"}


def test_oracle_router_groups():
    import torch
    s = torch.tensor([0.9, 0.1, 0.5, 0.6, 0.8, 0.7], dtype=torch.float64)
    # groups of two: sums 1.0, 1.1, 1.5 -> the best one group is the last
    assert O.route(s, 2, 3, 1)[0] == [4, 5]
    assert O.route(s, 2, 3, 2)[0] == [4, 5] and O.route(s, 3, 3, 2)[0] == [4, 5, 3]
    assert O.route(s, 2)[0] == [0, 4]
    w = O.route(s, 2)[1]
    assert abs(w.sum().item() - 1) < 1e-12 and abs(w[0].item() - 0.9 / 1.7) < 1e-12
