"""Host-side parts of the layer-list serving path (no GPU): safetensors reader, design config parser, page / slot pools,
flat step builder, and the engine's scheduler over a stand-in model."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import seq_oracle as O
from blazr_b200 import fenorax, registry
from blazr_b200.batch import StepEntry, build_step
from blazr_b200.cache import CacheFull, CacheManager, PagePool, SlotPool
from blazr_b200.engine import Engine, SamplingParams
from blazr_b200.layered import AttentionSpec, DenseFfSpec, SsmSpec
from blazr_b200.safetensors_loader import Safetensors, SafetensorsError, load_checkpoint


def small_cfg(**over):
    att = {"type": "attention", "mixer": {"dim": 16, "vdim": 8, "heads": 4, "kv_heads": 2, "scale": 0.3, "mask": {"size": 24}},
           "mlp": {"kind": "dense", "ff": 40, "limit": 1.5}}
    ssm = {"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "norm_groups": 4, "conv": 3}, "mlp": None}
    cfg = {"architecture": "Fenorax", "vocab": 61, "width": 48, "streams": 2, "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 2},
           "embedding": {"scale": 2.5}, "layers": [att, ssm]}
    cfg.update(over)
    return cfg


def test_safetensors_roundtrip(tmp_path):
    cfg = small_cfg()
    P = O.random_model(cfg, seed=3)
    O.write_checkpoint(str(tmp_path), cfg, P)
    cfg2, st = load_checkpoint(str(tmp_path))
    assert cfg2 == cfg and set(st.names()) == set(P)
    for k, v in P.items():
        t = st.tensor(k)
        assert t.dtype == torch.bfloat16 and list(t.shape) == list(v.shape) and torch.equal(t.float(), v)
    st.close()
    assert registry.architecture_of(str(tmp_path)) == "Fenorax"


def test_safetensors_rejects_bad_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x00")
    with pytest.raises(SafetensorsError):
        Safetensors(str(p))
    head = json.dumps({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        Safetensors(str(p))
    head = json.dumps({"a": {"dtype": "I32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(head)) + head + struct.pack("<ii", 7, -2))
    s = Safetensors(str(p))
    assert s.tensor("a").tolist() == [7, -2]
    s.close()


def test_config_parser_maps_every_key():
    cfg = small_cfg()
    lc = fenorax.parse_config(cfg)
    assert (lc.vocab, lc.width, lc.streams, lc.norm_groups, lc.canon_taps) == (61, 48, 2, 3, 2)
    assert lc.eps == 1e-5 and lc.embed_scale == 2.5
    a, s = lc.layers
    assert a.kind == "attention" and isinstance(a.mixer, AttentionSpec) and isinstance(a.ff, DenseFfSpec)
    assert (a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim, a.mixer.chunk, a.mixer.window) == (4, 2, 16, 8, 24, 0)
    assert a.mixer.scale == 0.3 and a.mixer.gated and a.mixer.qk_unit_norm
    assert (a.ff.ff, a.ff.limit, a.ff.alpha, a.ff.up_shift) == (40, 1.5, 1.702, 1.0)
    assert s.kind == "ssm" and isinstance(s.mixer, SsmSpec) and s.ff is None
    assert (s.mixer.heads, s.mixer.vdim, s.mixer.state, s.mixer.groups, s.mixer.norm_groups, s.mixer.conv) == (4, 8, 16, 2, 4, 3)


@pytest.mark.parametrize("breakit", ["type", "kv", "mlp", "missing"])
def test_config_parser_errors(breakit):
    cfg = small_cfg()
    if breakit == "type":
        cfg["layers"][0]["type"] = "other"
    elif breakit == "kv":
        cfg["layers"][0]["mixer"]["kv_heads"] = 3
    elif breakit == "mlp":
        cfg["layers"][0]["mlp"]["kind"] = "sparse"
    else:
        del cfg["canon"]
    with pytest.raises(fenorax.ConfigError):
        fenorax.parse_config(cfg)


def test_unknown_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nonesuch"}))
    with pytest.raises(registry.UnknownArchitecture):
        registry.load_model(str(tmp_path), "cpu")


def test_pools_reuse_last_freed_first():
    p = PagePool(4, 16)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.free_blocks == 1
    p.free([1])
    assert p.alloc(2) == [1, 3]
    with pytest.raises(CacheFull):
        p.alloc(1)
    s = SlotPool(2)
    x, y = s.alloc(), s.alloc()
    with pytest.raises(CacheFull):
        s.alloc()
    s.free(x)
    assert s.alloc() == x and y != x


def test_cache_manager_grows_and_releases():
    cm = CacheManager(max_tokens=64, max_seqs=2, block_size=16)
    a = cm.admit("a")
    cm.reserve(a, 17)
    assert len(a.blocks) == 2
    a.n_tokens = 17
    assert cm.pages_needed(a, 15) == 0 and cm.pages_needed(a, 16) == 1
    b = cm.admit("b")
    assert not cm.can_admit()
    with pytest.raises(ValueError):
        cm.admit("a")
    cm.reserve(b, 1)
    held = set(a.blocks) | set(b.blocks)
    assert len(held) == 3
    free_before = cm.pages.free_blocks
    cm.release("a")
    assert cm.pages.free_blocks == free_before + 2 and cm.can_admit()
    c = cm.admit("c")
    assert c.slot == a.slot
    cm.reserve(c, 1)
    assert c.blocks[0] in held          # a freed page comes back first


def test_build_step_layout():
    e = [StepEntry(tokens=[5, 6, 7], pos0=30, slot=2, block_table=[9, 4, 1], want=[0, 2]), StepEntry(tokens=[8], pos0=0, slot=0, block_table=[3], want=[0])]
    sa = build_step(e, block_size=16)
    assert sa.T == 4 and sa.B == 2 and not sa.decode_only
    assert sa.tok_ids.tolist() == [5, 6, 7, 8] and sa.tok_ent.tolist() == [0, 0, 0, 1] and sa.tok_pos.tolist() == [30, 31, 32, 0]
    assert sa.ent_start.tolist() == [0, 3, 4] and sa.ent_slot.tolist() == [2, 0] and sa.ent_pos0.tolist() == [30, 0]
    assert sa.block_table.tolist() == [[9, 4, 1], [3, 0, 0]] and sa.want_rows.tolist() == [0, 2, 3]
    with pytest.raises(ValueError):
        build_step([StepEntry(tokens=[1], pos0=16, slot=0, block_table=[3])], 16)
    with pytest.raises(ValueError):
        build_step([StepEntry(tokens=[1], pos0=0, slot=0, block_table=[3], want=[1])], 16)
    assert build_step([StepEntry(tokens=[1], pos0=5, slot=1, block_table=[2])], 16).decode_only


class _FakeModel:
    """stands in for LayeredModel: records the steps, answers with logits whose arg-max is (last token + 1) % vocab"""
    vocab = 50

    def __init__(self):
        self.dev = torch.device("cpu")
        self.steps = []

    def allocate(self, num_blocks, block_size, max_seqs, max_seq_tokens):
        self.alloc = (num_blocks, block_size, max_seqs, max_seq_tokens)

    def forward(self, sa, sample=False):
        self.steps.append(sa)
        nxt = (sa.tok_ids[sa.want_rows] + 1) % self.vocab
        self.last_ids = torch.from_numpy(nxt.astype(np.int32))
        return torch.nn.functional.one_hot(torch.from_numpy(nxt.astype(np.int64)), self.vocab).float()


def test_scheduler_mixes_decode_and_prompt_portions(monkeypatch):
    monkeypatch.setattr("blazr_b200.seqops.error_flags", lambda: 0)
    m = _FakeModel()
    eng = Engine(m, max_tokens=256, max_seqs=2, block_size=16, max_step_tokens=24, prefill_chunk=20)
    outs = eng.generate([[1, 2, 3], list(range(10, 45)), [7]], SamplingParams(max_new_tokens=4))
    assert outs == [[4, 5, 6, 7], [45, 46, 47, 48], [8, 9, 10, 11]]
    # step 0: the short prompt whole + the first 20 tokens of the long one (budget 24, chunk 20)
    s0 = m.steps[0]
    assert s0.B == 2 and s0.ent_start.tolist() == [0, 3, 23] and s0.want_rows.tolist() == [2]
    # step 1: request 0 decodes beside the rest of the long prompt; the third request waits for a slot
    s1 = m.steps[1]
    assert s1.ent_start.tolist() == [0, 1, 16] and s1.ent_pos0.tolist() == [3, 20] and s1.want_rows.tolist() == [0, 15]
    assert all(s.B <= 2 and s.T <= 24 for s in m.steps)
    late = [i for i, s in enumerate(m.steps) if 7 in s.tok_ids[s.ent_start[:-1][s.ent_pos0 == 0]].tolist()]
    assert late and late[0] >= 4                                      # admitted once a slot was free
    assert eng.cache.pages.free_blocks == eng.cache.pages.num_blocks and eng.cache.slots.free_slots == 2


def test_scheduler_waits_for_pages_and_reports_a_pool_too_small(monkeypatch):
    monkeypatch.setattr("blazr_b200.seqops.error_flags", lambda: 0)
    m = _FakeModel()
    eng = Engine(m, max_tokens=32, max_seqs=2, block_size=16)       # 2 + 2 pages
    outs = eng.generate([list(range(30)), list(range(20, 50))], SamplingParams(max_new_tokens=3))
    assert outs == [[30, 31, 32], [0, 1, 2]]
    eng2 = Engine(_FakeModel(), max_tokens=16, max_seqs=1, block_size=16)    # 2 pages: a 40-token prompt can never fit
    eng2.add_request("x", list(range(40)))
    with pytest.raises(CacheFull):
        while eng2.has_work():
            eng2.step()


def test_run_entries_admits_advances_and_releases():
    m = _FakeModel()
    eng = Engine(m, max_tokens=64, max_seqs=2, block_size=16)
    out = eng.run_entries([{"id": "a", "tokens": [1, 2, 3], "want": [2]}, {"id": "b", "tokens": [9], "want": []}], [])
    assert out.shape == (1, 50) and out[0].argmax() == 4
    assert eng.run_entries([{"id": "b", "tokens": [4, 5], "want": []}], ["a"]) is None
    assert m.steps[1].ent_pos0.tolist() == [1] and "a" not in eng.cache.live and eng.cache.live["b"].n_tokens == 3
    with pytest.raises(ValueError):
        eng.run_entries([{"id": "b", "tokens": [1], "want": []}, {"id": "b", "tokens": [2], "want": []}], [])


def test_sequence_library_exports_what_its_header_declares():
    import re

    from blazr_b200 import seqops
    here = os.path.dirname(os.path.abspath(__file__))
    txt = re.sub(r"/\*.*?\*/", "", open(os.path.join(here, "..", "include", "b200seq.h")).read(), flags=re.S)
    syms = sorted(set(re.findall(r"\b(b200seq_[a-z0-9_]+)\s*\(", txt)))
    L = seqops.lib()
    for s in syms:
        assert hasattr(L, s), f"{s} declared in b200seq.h but not exported"
    assert sorted(seqops.EXPORTS) == syms
