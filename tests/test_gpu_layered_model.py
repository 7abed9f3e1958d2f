"""Fenorax models end to end through the registry, the engine and its cache: small configurations with random weights, compared
with the plain float64 restatement (tests/seq_oracle.py) of whole sequences.  Sizes are chosen unlike each other on purpose
(value size != key size, fewer key heads than query heads, one / several streams and norm groups, odd vocabularies)."""
import copy

import numpy as np
import pytest
import torch

import seq_oracle as O

pytestmark = pytest.mark.gpu


def att(dim=16, vdim=8, heads=4, kv=2, scale=0.3, size=24, ff=40, limit=1.5):
    return {"type": "attention", "mixer": {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv, "scale": scale, "mask": {"size": size}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def ssm(heads=4, vdim=8, state=16, groups=2, norm_groups=4, conv=3, ff=None, limit=1.0):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(layers, vocab=61, width=48, streams=2, groups=3, taps=2, scale=2.5, eps=1e-5):
    return {"architecture": "Fenorax", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps, "groups": groups},
            "canon": {"taps": taps}, "embedding": {"scale": scale}, "layers": layers}


CONFIGS = {
    "mixed": config([att(), ssm(), att(size=7, ff=None), ssm(ff=24)]),
    "one_stream": config([ssm(heads=2, vdim=20, state=8, groups=1, norm_groups=1, conv=2), att(dim=8, vdim=24, heads=2, kv=2, size=5)],
                         vocab=33, width=40, streams=1, groups=1, taps=1),
    "wide": config([att(dim=32, vdim=16, heads=6, kv=1, size=16, scale=0.11, ff=72, limit=0.8), ssm(heads=6, vdim=16, state=24, groups=3, norm_groups=2, conv=4)],
                   vocab=130, width=96, streams=4, groups=4, taps=4, scale=0.7, eps=1e-3),
}


class Case:
    def __init__(self, name, tmp, dtype):
        from blazr_b200 import registry
        self.cfg = copy.deepcopy(CONFIGS[name])
        self.P = O.random_model(self.cfg, seed=11)
        O.write_checkpoint(str(tmp), self.cfg, self.P)
        self.model = registry.load_model(str(tmp), "cuda:0", dtype)
        self._ref = {}

    def engine(self, **kw):
        from blazr_b200.engine import Engine
        return Engine(self.model, **kw)

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = O.forward(self.cfg, self.P, list(tokens))
        return self._ref[key]


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    made = {}

    def get(name, dtype="float32"):
        if (name, dtype) not in made:
            made[(name, dtype)] = Case(name, tmp_path_factory.mktemp(f"{name}_{dtype}"), dtype)
        return made[(name, dtype)]
    return get


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def err(got, ref):
    d = torch.as_tensor(got).double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt().max() / ref.double().std()).item()


TOL32, TOL16 = 5e-5, 1e-1


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_layers(cases, name):
    c = cases(name)
    t = toks(53, c.cfg["vocab"], 1)
    eng = c.engine(max_tokens=64, max_seqs=2)
    got = eng.run_entries([{"id": "a", "tokens": t, "want": list(range(53))}], ["a"])
    assert err(got, c.ref(t)) < TOL32
    # residual stream after every layer
    from blazr_b200.batch import StepEntry, build_step
    seq = eng.cache.admit("b")
    eng.cache.reserve(seq, len(t))
    dbg = []
    c.model.forward(build_step([StepEntry(t, 0, seq.slot, seq.blocks, [0])], eng.cache.block_size), debug_layers=dbg)
    sums = []
    O.forward(c.cfg, c.P, t, layer_sums=sums)
    for g, r in zip(dbg, sums):
        assert (g.double() - r).abs().max().item() < 2e-5 * r.abs().max().item()


def test_bfloat16_mode_stays_close(cases):
    c = cases("mixed", "bfloat16")
    t = toks(90, c.cfg["vocab"], 2)
    eng = c.engine(max_tokens=96, max_seqs=1)
    got = eng.run_entries([{"id": "a", "tokens": t[:60], "want": list(range(60))}], [])
    assert err(got, c.ref(t)[:60]) < TOL16
    for i in range(60, 90):
        got = eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])
        assert err(got, c.ref(t)[i:i + 1]) < TOL16


@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_then_token_by_token(cases, name):
    """long decoding: the decoded tokens cross several chunk edges and page borders"""
    c = cases(name)
    t = toks(100, c.cfg["vocab"], 3)
    ref = c.ref(t)
    eng = c.engine(max_tokens=112, max_seqs=1)
    got = [eng.run_entries([{"id": "a", "tokens": t[:9], "want": [0, 8]}], [])]
    assert err(got[0], ref[[0, 8]]) < TOL32
    for i in range(9, 100):
        got = eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])
        assert err(got, ref[i:i + 1]) < TOL32, f"decoded position {i}"
    assert eng.cache.live["a"].n_tokens == 100


def test_decode_from_the_very_first_token(cases):
    c = cases("mixed")
    t = toks(12, c.cfg["vocab"], 4)
    ref = c.ref(t)
    eng = c.engine(max_tokens=16, max_seqs=1)
    for i in range(12):
        got = eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])
        assert err(got, ref[i:i + 1]) < TOL32, f"position {i}"


@pytest.mark.parametrize("name,sizes", [("mixed", [2, 3, 2, 17, 1, 24, 2, 2, 30, 5]), ("wide", [15, 2, 16, 1, 1, 33, 2, 18]), ("one_stream", [1, 2, 4, 5, 6, 50, 20])])
def test_portions_of_changing_size(cases, name, sizes):
    c = cases(name)
    n = sum(sizes)
    t = toks(n, c.cfg["vocab"], 5)
    ref = c.ref(t)
    eng = c.engine(max_tokens=-(-n // 16) * 16, max_seqs=1)
    lo = 0
    for s in sizes:
        got = eng.run_entries([{"id": "a", "tokens": t[lo:lo + s], "want": list(range(s))}], [])
        assert err(got, ref[lo:lo + s]) < TOL32, f"portion at {lo} of {s}"
        lo += s


def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(cases):
    """four slots, a pool far smaller than the sum of all requests: finished requests hand their pages and slot to new ones while
    others are in the middle of their prompt or decoding"""
    c = cases("mixed")
    V = c.cfg["vocab"]
    seqs = {n: toks(L, V, 20 + i) for i, (n, L) in enumerate([("a", 70), ("b", 9), ("c", 31), ("d", 2), ("e", 48), ("f", 17), ("g", 1), ("h", 26)])}
    eng = c.engine(max_tokens=176, max_seqs=4)
    plan = [[("a", 30), ("b", 2), ("c", 1)], [("c", 5), ("a", 1), ("b", 7), ("d", 2)], [("a", 25), ("e", 3), ("c", 25)], [("e", 45), ("a", 1), ("f", 2)],
            [("a", 13), ("f", 15), ("g", 1), ("h", 2)], [("h", 1)], [("h", 23)]]
    fed = {n: 0 for n in seqs}
    used_slots, used_pages = {}, {}
    for step in plan:
        entries, end = [], []
        for n, k in step:
            entries.append({"id": n, "tokens": seqs[n][fed[n]:fed[n] + k], "want": list(range(k))})
            if fed[n] + k == len(seqs[n]):
                end.append(n)
        assert len(eng.cache.live) + sum(1 for n, _ in step if n not in eng.cache.live) <= 4
        got = eng.run_entries(entries, [])
        for n, _ in step:                                # what each request holds, before the step's finished ones give it back
            used_slots[n] = eng.cache.live[n].slot
            used_pages[n] = list(eng.cache.live[n].blocks)
        for n in end:
            eng.release(n)
        o = 0
        for n, k in step:
            assert err(got[o:o + k], c.ref(seqs[n])[fed[n]:fed[n] + k]) < TOL32, f"{n} at {fed[n]}"
            o += k
            fed[n] += k
    assert all(fed[n] == len(s) for n, s in seqs.items())
    assert len(set(used_slots.values())) <= 4 < len(used_slots)
    all_pages = [p for v in used_pages.values() for p in v]
    assert len(all_pages) > len(set(all_pages))                      # pages went through several owners
    assert eng.cache.pages.free_blocks == eng.cache.pages.num_blocks and eng.cache.slots.free_slots == 4


def test_alone_and_in_a_batch_agree(cases):
    c = cases("wide")
    V = c.cfg["vocab"]
    a, b = toks(40, V, 30), toks(21, V, 31)
    alone = c.engine(max_tokens=48, max_seqs=1)
    ra = alone.run_entries([{"id": "a", "tokens": a, "want": [39]}], ["a"])
    both = c.engine(max_tokens=96, max_seqs=2)
    both.run_entries([{"id": "b", "tokens": b[:20], "want": []}], [])
    rb = both.run_entries([{"id": "b", "tokens": b[20:], "want": [0]}, {"id": "a", "tokens": a, "want": [39]}], [])
    assert err(rb[1:2], torch.from_numpy(ra)) < 1e-5
    assert err(rb[0:1], c.ref(b)[20:21]) < TOL32


def test_chunk_edge_seen_through_the_whole_model(cases):
    """tokens decoded alone around the end of the first chunk; the same weights with a chunk one position longer give logits that
    differ by far more than the tolerance there, so a mask that is one off cannot pass"""
    c = cases("mixed")
    t = toks(60, c.cfg["vocab"], 6)
    ref = c.ref(t)
    size = c.cfg["layers"][0]["mixer"]["mask"]["size"]           # chunk of the first layer
    eng = c.engine(max_tokens=64, max_seqs=1)
    got = eng.run_entries([{"id": "a", "tokens": t[:size - 1], "want": []}], [])
    rows = []
    for i in range(size - 1, size + 2):                           # last of the first chunk, first two of the next, each decoded alone
        rows.append(eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])[0])
    assert err(np.stack(rows), ref[size - 1:size + 2]) < TOL32
    # what a mask one position off would give differs by far more than the tolerance
    wrong = copy.deepcopy(c.cfg)
    wrong["layers"][0]["mixer"]["mask"]["size"] = size + 1
    off = O.forward(wrong, c.P, t)
    assert err(off[size:size + 1], ref[size:size + 1]) > 100 * TOL32


def test_greedy_generation_through_the_scheduler(cases):
    from blazr_b200.engine import SamplingParams
    c = cases("mixed")
    V = c.cfg["vocab"]
    prompts = [toks(n, V, 40 + i) for i, n in enumerate([5, 33, 1, 12, 20, 3])]
    eng = c.engine(max_tokens=224, max_seqs=3, max_step_tokens=40, prefill_chunk=16)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k in range(6):
            lg = O.forward(c.cfg, c.P, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]).item() < 1e-3 * lg.std().item():      # a near tie may fall either way in 32-bit: follow the engine
                seq.append(o[k])
                continue
            assert int(lg.argmax()) == o[k], f"token {k} of prompt of {len(p)}"
            seq.append(o[k])
    assert eng.cache.pages.free_blocks == eng.cache.pages.num_blocks


def test_sampling_with_temperature_is_seeded_and_in_range(cases):
    from blazr_b200.engine import SamplingParams
    c = cases("mixed")
    p = toks(7, c.cfg["vocab"], 50)
    sp = SamplingParams(temperature=0.8, top_k=10, top_p=0.9, seed=5, max_new_tokens=8)
    a = c.engine(max_tokens=32, max_seqs=1).generate([p], sp)[0]
    b = c.engine(max_tokens=32, max_seqs=1).generate([p], sp)[0]
    assert a == b and len(a) == 8 and all(0 <= x < c.cfg["vocab"] for x in a)


def test_trace_replay_command(cases, tmp_path):
    """bin/trace_run as a user starts it: steps on standard input, logits files and 'done' lines out"""
    import json
    import os
    import subprocess
    import sys
    c = cases("one_stream")
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, c.cfg, c.P)
    t = toks(30, c.cfg["vocab"], 7)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": t[:20], "want": [19]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": t[20:29], "want": []}, {"id": "y", "tokens": t[:3], "want": [2]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": t[29:], "want": [0]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = c.ref(t)
    V = c.cfg["vocab"]
    g0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(1, V)
    g1 = np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(1, V)
    g2 = np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(1, V)
    assert err(g0, ref[19:20]) < TOL32 and err(g1, ref[2:3]) < TOL32 and err(g2, ref[29:30]) < TOL32


CONFIGS["long"] = config([ssm(heads=3, vdim=24, state=40, groups=1, norm_groups=3, conv=4), att(dim=24, vdim=40, heads=6, kv=2, size=150, scale=0.2, ff=56),
                          ssm(heads=2, vdim=16, state=130, groups=2, norm_groups=1, conv=2, ff=32)], vocab=77, width=64, streams=3, groups=2, taps=3)


def test_long_portions_next_to_single_tokens(cases):
    """portions of hundreds of tokens (the recurrence runs as parallel segments, attention as query tiles over many key tiles) in the
    same steps as single tokens of another request; then both decode side by side"""
    c = cases("long")
    a, b = toks(520, c.cfg["vocab"], 20), toks(160, c.cfg["vocab"], 21)
    ra, rb = c.ref(a), c.ref(b)
    eng = c.engine(max_tokens=720, max_seqs=2)
    got = eng.run_entries([{"id": "b", "tokens": b[:3], "want": [2]}], [])
    assert err(got, rb[2:3]) < TOL32
    got = eng.run_entries([{"id": "a", "tokens": a[:300], "want": [0, 127, 128, 149, 150, 299]}, {"id": "b", "tokens": [b[3]], "want": [0]}], [])
    assert err(got, torch.cat([ra[[0, 127, 128, 149, 150, 299]], rb[3:4]])) < TOL32
    got = eng.run_entries([{"id": "b", "tokens": b[4:135], "want": [0, 130]}, {"id": "a", "tokens": a[300:470], "want": [0, 1, 169]}], [])
    assert err(got, torch.cat([rb[[4, 134]], ra[[300, 301, 469]]])) < TOL32
    for i in range(25):
        got = eng.run_entries([{"id": "a", "tokens": [a[470 + i]], "want": [0]}, {"id": "b", "tokens": [b[135 + i]], "want": [0]}], [])
        assert err(got, torch.cat([ra[470 + i:471 + i], rb[135 + i:136 + i]])) < TOL32, f"decoded token {i}"
    got = eng.run_entries([{"id": "a", "tokens": a[495:520], "want": [24]}], ["a", "b"])
    assert err(got, ra[519:520]) < TOL32
    from blazr_b200 import seqops
    assert seqops.error_flags() == 0
