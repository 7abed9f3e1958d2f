"""libb200seq operators, each alone, against the plain float64 restatement in tests/seq_oracle.py.

Every sequence operator is run over a flat mixed batch (several entries, portions that continue earlier ones, scattered pages and
slots) and must give, for each sequence, what the whole sequence gives in one piece."""
import numpy as np
import pytest
import torch

import seq_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    from blazr_b200 import seqops
    seqops.lib()
    return seqops


def dev_step(ops, entries, block_size):
    """entries: [(n_tokens, pos0, slot, block_table)] -> (StepDesc, keep-alive tensors)"""
    from blazr_b200.batch import StepEntry, build_step
    sa = build_step([StepEntry([0] * n, p0, slot, bt) for n, p0, slot, bt in entries], block_size)
    t = {k: torch.from_numpy(np.ascontiguousarray(getattr(sa, k))).to(DEV) for k in ("tok_ent", "tok_pos", "ent_start", "ent_slot", "ent_pos0", "block_table")}
    d = ops.StepDesc(t["tok_ent"].data_ptr(), t["tok_pos"].data_ptr(), t["ent_start"].data_ptr(), t["ent_slot"].data_ptr(), t["ent_pos0"].data_ptr(),
                     t["block_table"].data_ptr(), sa.T, sa.B, sa.block_table.shape[1], block_size)
    return d, t


def close(got, ref, tol):
    ref = ref.double()
    err = (got.double().cpu() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("M,N,K", [(1, 37, 40), (3, 64, 96), (7, 130, 200), (9, 61, 33), (70, 130, 72), (200, 257, 136)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_linear_paths(ops, M, N, K, xdt):
    x = rnd(M, K, seed=1).to(xdt)
    w = rnd(N, K, seed=2, scale=K ** -0.5).bfloat16()
    ref = x.double() @ w.double().T
    for path in (ops.PATH_ROWS, ops.PATH_TILED, ops.PATH_AUTO):
        y = torch.full((M, N + 3), 7.0, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), y[:, :N], path)
        close(y[:, :N], ref, 5e-6)
        assert bool((y[:, N:] == 7.0).all())


@pytest.mark.parametrize("M,N,K", [(32, 128, 64), (70, 130, 72), (200, 257, 136), (129, 61, 8), (300, 448, 520), (1000, 96, 200)])
def test_linear_tensor_core_path(ops, M, N, K):
    x = rnd(M, K + 8, seed=11).bfloat16()[:, :K]                 # rows with a stride that is not K
    w = rnd(N, K, seed=12, scale=K ** -0.5).bfloat16()
    ref = x.double() @ w.double().T
    y = torch.full((M, N + 1), 7.0, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), y[:, :N], ops.PATH_TC)
    close(y[:, :N], ref, 5e-6)
    assert bool((y[:, N:] == 7.0).all()) and ops.error_flags() == 0
    auto = torch.empty(M, N, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), auto)                        # the automatic choice takes this path from 32 rows
    assert torch.equal(auto, y[:, :N])
    one = torch.empty(32, N, device=DEV)                          # a row's result does not depend on the rows beside it
    ops.linear(x[M - 32:].to(DEV), w.to(DEV), one, ops.PATH_TC)
    assert torch.equal(one, y[M - 32:, :N])


@pytest.mark.parametrize("M,F,K,limit", [(33, 40, 48, 1.5), (260, 129, 200, 0.6), (128, 64, 64, 7.0)])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_gate_up_projection_fused_with_its_activation(ops, M, F, K, limit, odt):
    x = rnd(M, K, seed=13, scale=2.0).bfloat16()
    wg, wu = rnd(F, K, seed=14, scale=K ** -0.5).bfloat16(), rnd(F, K, seed=15, scale=K ** -0.5).bfloat16()
    g = torch.clamp(x.double() @ wg.double().T, max=limit)
    u = torch.clamp(x.double() @ wu.double().T, -limit, limit)
    ref = g * torch.sigmoid(1.702 * g) * (u + 1)
    w_il = torch.stack([wg, wu], 1).reshape(2 * F, K).contiguous()
    out = torch.full((M, F + 2), 3.0, device=DEV, dtype=odt)
    ops.linear_gated(x.to(DEV), w_il.to(DEV), limit, 1.702, 1.0, out[:, :F])
    close(out[:, :F].float(), ref, 1e-5 if odt == torch.float32 else 1e-2)
    assert bool((out[:, F:] == 3.0).all()) and ops.error_flags() == 0
    # the unfused pair of kernels on the same interleaved weight gives the same numbers
    gu = torch.empty(M, 2 * F, device=DEV)
    ops.linear(x.to(DEV), w_il.to(DEV), gu, ops.PATH_TC)
    two = torch.empty(M, F, device=DEV, dtype=odt)
    ops.gated_act(gu, limit, 1.702, 1.0, two, interleaved=True)
    assert torch.equal(two, out[:, :F])


def test_linear_row_does_not_depend_on_the_batch(ops):
    x = rnd(40, 96, seed=3)
    w = rnd(50, 96, seed=4).bfloat16().to(DEV)
    for path in (ops.PATH_ROWS, ops.PATH_TILED):
        full = torch.empty(40, 50, device=DEV)
        ops.linear(x.to(DEV), w, full, path)
        one = torch.empty(1, 50, device=DEV)
        ops.linear(x[17:18].contiguous().to(DEV), w, one, path)
        assert torch.equal(one[0], full[17])


@pytest.mark.parametrize("S,W,groups", [(1, 40, 1), (3, 48, 2), (4, 30, 5), (8, 1200, 3), (8, 4096, 4), (6, 2304, 2)])
def test_stream_mix_and_group_norm(ops, S, W, groups):
    T, eps = 5, 1e-3
    X, y = rnd(T, S, W, seed=5), rnd(T, W, seed=6)
    outv, mix, inw, nw = rnd(S, seed=7), rnd(S, S, seed=8), rnd(S, seed=9), rnd(W, seed=10)
    Xn = torch.einsum("st,nsw->ntw", mix.double(), X.double()) + outv.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("s,nsw->nw", inw.double(), Xn)
    ref = O.group_rms(u, groups, eps, nw.double())
    Xd = X.to(DEV).clone()
    out = torch.empty(T, W, device=DEV)
    ops.hc_norm(Xd, y.to(DEV), torch.cat([outv, mix.reshape(-1)]).to(DEV), inw.to(DEV), nw.to(DEV), groups, eps, out)
    close(Xd, Xn, 1e-6)
    close(out, ref, 1e-5)
    # collapse only (no pending update), selected rows, bfloat16 output
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, W, device=DEV, dtype=torch.bfloat16)
    ops.hc_norm(Xd, None, None, inw.to(DEV), nw.to(DEV), groups, eps, out2, rows=rows)
    close(out2.float(), ref[[3, 0]], 1e-2)
    g = torch.empty(T, W, device=DEV)
    ops.group_rmsnorm(u.float().to(DEV), nw.to(DEV), groups, eps, g)
    close(g, ref, 1e-5)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("mode", ["residual", "silu"])
def test_causal_conv_carries_its_tail(ops, taps, mode):
    C, slots = 70, 5
    lens = {"a": 23, "b": 9, "c": 1, "d": 12}
    xs = {k: rnd(n, C, seed=20 + i) for i, (k, n) in enumerate(lens.items())}
    w, b = rnd(C, taps, seed=30), rnd(C, seed=31)
    ref = {}
    for k, x in xs.items():
        c = O.causal_conv(x.double(), w.double(), b.double() if mode == "silu" else None)
        ref[k] = O.silu(c) if mode == "silu" else x.double() + c
    state = torch.full((slots, max(taps - 1, 1), C), 99.0, device=DEV)      # stale: a fresh sequence must not read it
    slot = {"a": 3, "b": 0, "c": 4, "d": 1}
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    # portions down to one token, shorter than the carried tail; entries of other sequences in between
    plan = [[("a", 1), ("b", 2)], [("a", 2), ("c", 1), ("b", 1)], [("b", 6), ("a", 17)], [("a", 1), ("d", 12)], [("a", 2)]]
    for step in plan:
        ents = [(n, fed[k], slot[k], [0]) for k, n in step]
        d, keep = dev_step(ops, ents, 4096)
        x = torch.cat([xs[k][fed[k]:fed[k] + n] for k, n in step]).to(DEV)
        out = torch.empty_like(x)
        ops.causal_conv(x, w.to(DEV), b.to(DEV) if mode == "silu" else None, state, d, ops.CONV_SILU if mode == "silu" else ops.CONV_RESIDUAL, out)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n].cpu())
            o += n
            fed[k] += n
    for k in lens:
        assert fed[k] == lens[k]
        close(torch.cat(got[k]), ref[k], 1e-5)


@pytest.mark.parametrize("F,limit", [(33, 0.7), (128, 2.0)])
def test_gated_activation(ops, F, limit):
    gu = rnd(6, 2 * F, seed=40, scale=2.0)
    g = torch.clamp(gu[:, :F].double(), max=limit)
    u = torch.clamp(gu[:, F:].double(), -limit, limit)
    ref = g * torch.sigmoid(1.702 * g) * (u + 1)
    out = torch.empty(6, F, device=DEV)
    ops.gated_act(gu.to(DEV), limit, 1.702, 1.0, out)
    close(out, ref, 1e-6)
    assert (gu[:, :F] > limit).any() and (gu[:, F:] < -limit).any() and (gu[:, :F] < -limit).any()   # every branch of the clamps is hit


def test_argmax_first_maximum(ops):
    lg = rnd(4, 1000, seed=41)
    lg[1, 77] = lg[1, 901] = 50.0
    lg[2, 999] = 60.0
    ids = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.argmax(lg.to(DEV), ids)
    assert ids.tolist() == [int(lg[0].argmax()), 77, 999, int(lg[3].argmax())]


def run_attention(ops, q, k, v, gate, scale, chunk, window, eps, plan, block_size, n_pages, act=torch.float32, seed=0, split=True):
    """feeds sequences (dict name -> (q, k, v, gate) of whole sequences) through prep + attend as the plan says; pages are taken
    from a shuffled list; returns name -> [T, H*V]"""
    names = list(q)
    H, D = q[names[0]].shape[1:]
    G, V = v[names[0]].shape[1:]
    kpool = torch.full((n_pages, block_size, G, D), 1e4, device=DEV)
    vpool = torch.full((n_pages, block_size, G, V), 1e4, device=DEV)
    free = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    pages = {n: [] for n in names}
    fed = {n: 0 for n in names}
    got = {n: [] for n in names}
    for step in plan:
        ents = []
        for n, cnt in step:
            while len(pages[n]) * block_size < fed[n] + cnt:
                pages[n].append(free.pop())
            ents.append((cnt, fed[n], 0, pages[n]))
        d, keep = dev_step(ops, ents, block_size)
        rows = [torch.cat([q[n][fed[n]:fed[n] + c].reshape(c, -1), k[n][fed[n]:fed[n] + c].reshape(c, -1), v[n][fed[n]:fed[n] + c].reshape(c, -1)]
                          + ([gate[n][fed[n]:fed[n] + c]] if gate is not None else []), 1) for n, c in step]
        qkvg = torch.cat(rows).contiguous().to(DEV)
        out = torch.empty(qkvg.shape[0], H * V, device=DEV, dtype=act)
        ops.attn_prep(qkvg, d, kpool, vpool, H, G, D, V, eps)
        scratch = None
        if split:    # steps of few tokens deal the key tiles to several blocks and merge: the work area starts as NaN
            keys = max(len(p) for p in pages.values()) * block_size
            need = ops.attn_scratch_floats(qkvg.shape[0], len(step), H, G, V, min(keys, chunk or keys, window or keys))
            scratch = torch.full((max(need, 1),), float("nan"), device=DEV)
        ops.attn(qkvg, d, kpool, vpool, H, G, D, V, scale, chunk, window, gate is not None, out, scratch)
        o = 0
        for n, c in step:
            got[n].append(out[o:o + c].float().cpu())
            o += c
            fed[n] += c
        for n, c in step:            # a finished sequence gives its pages back at once: the next one gets them
            if fed[n] == q[n].shape[0]:
                free.extend(pages[n])
                pages[n] = []
    assert ops.error_flags() == 0
    return {n: torch.cat(got[n]) for n in names}


def attention_case(T, H, G, D, V, seed):
    return rnd(T, H, D, seed=seed), rnd(T, G, D, seed=seed + 1), rnd(T, G, V, seed=seed + 2), rnd(T, H, seed=seed + 3)


@pytest.mark.parametrize("H,G,D,V,chunk,window,bs", [(4, 2, 16, 8, 24, 0, 16), (3, 3, 20, 40, 7, 0, 4), (2, 1, 64, 64, 0, 0, 16), (4, 4, 8, 8, 0, 10, 8),
                                                     (6, 2, 12, 33, 16, 5, 16)])
def test_attention_mixed_batch_matches_whole_sequences(ops, H, G, D, V, chunk, window, bs):
    eps, scale = 1e-4, 0.37
    lens = {"a": 75, "b": 30, "c": 3}
    data = {n: attention_case(T, H, G, D, V, 50 + 10 * i) for i, (n, T) in enumerate(lens.items())}
    q, k, v, gate = ({n: d[j] for n, d in data.items()} for j in range(4))
    ref = {}
    for n in lens:
        qn = O.group_rms(q[n].double(), 1, eps)
        kn = O.group_rms(k[n].double(), 1, eps)
        ref[n] = O.masked_attention(qn, kn, v[n].double(), scale, chunk, window, torch.sigmoid(gate[n].double())).reshape(lens[n], -1)
    plan = [[("a", 40), ("b", 2)], [("b", 1), ("a", 1), ("c", 3)], [("a", 2), ("b", 27)], [("a", 32)]]
    got = run_attention(ops, q, k, v, gate, scale, chunk, window, eps, plan, bs, n_pages=-(-75 // bs) + -(-30 // bs) + 2)
    for n in lens:
        close(got[n], ref[n], 2e-5)


@pytest.mark.parametrize("decode", [False, True])
def test_attention_chunk_edges_show(ops, decode):
    """one key carries a value that stands out and a direction every later query points at: the output shows at once whether the key
    was visible, so a chunk edge that is one position off cannot hide among many small weights"""
    H = G = 1
    D, V, chunk, bs, T = 16, 8, 20, 16, 70
    hot = 39                                           # last position of the chunk [20, 40)
    q = torch.zeros(T, H, D)
    k = rnd(T, G, D, seed=60, scale=0.05)
    v = rnd(T, G, V, seed=61, scale=0.1)
    q[:, 0, 0] = 1.0
    k[hot] = 0
    k[hot, 0, 0] = 1.0
    v[hot] = 100.0
    plan = [[("a", 35)]] + [[("a", 1)]] * 35 if decode else [[("a", 38)], [("a", 2)], [("a", 30)]]
    got = run_attention(ops, {"a": q}, {"a": k}, {"a": v}, None, 40.0, chunk, 0, -1.0, plan, bs, n_pages=6)["a"]
    ref = O.masked_attention(q.double(), k.double(), v.double(), 40.0, chunk, 0).reshape(T, -1)
    close(got, ref, 2e-5)
    assert got[hot].min() > 99 and got[hot - 1].abs().max() < 5      # the key sees itself; earlier positions of its chunk do not
    assert got[hot + 1].abs().max() < 5                                # first position of the next chunk: just outside


def test_attention_far_key_among_hundreds_and_window_edges(ops):
    H, G, D, V, bs, T, window = 2, 1, 32, 16, 16, 400, 128
    q, k, v, _ = attention_case(T, H, G, D, V, 70)
    k = k * 0.05
    far = 16                                           # first slot of a page
    q[:, :, :] = 0
    q[:, :, 3] = 1.0
    k[far] = 0
    k[far, 0, 3] = 1.0
    v[far] = -50.0
    for win in (0, window):
        plan = [[("a", 300)], [("a", 2)]] + [[("a", 1)]] * 98
        got = run_attention(ops, {"a": q}, {"a": k}, {"a": v}, None, 30.0, 0, win, -1.0, plan, bs, n_pages=26)["a"]
        ref = O.masked_attention(q.double(), k.double(), v.double(), 30.0, 0, win).reshape(T, -1)
        close(got, ref, 2e-5)
        if win:
            assert got[far + win - 1].max() < -49 and got[far + win].abs().max() < 5    # last query that sees it, first that does not
        else:
            assert got[T - 1].max() < -49                                                # 383 positions back, through 24 pages


@pytest.mark.parametrize("H,G,N,V", [(4, 2, 16, 8), (3, 1, 32, 40), (2, 2, 5, 64), (6, 3, 64, 32), (1, 1, 128, 7)])
def test_state_space_scan_carries_state_between_portions(ops, H, G, N, V):
    lens = {"a": 37, "b": 11, "c": 2}
    inner = H * V
    ld = 2 * inner + 2 * G * N + H
    slot = {"a": 2, "b": 0, "c": 2}                 # c takes a's slot after a finished: stale state must not leak
    data, ref = {}, {}
    A_log, Dp, dtb = rnd(H, seed=80, scale=0.5), rnd(H, seed=81), rnd(H, seed=82)
    for i, (n, T) in enumerate(lens.items()):
        proj = rnd(T, ld, seed=83 + i)
        xbc = rnd(T, inner + 2 * G * N, seed=90 + i)
        data[n] = (proj, xbc)
        y = O.ssm_recurrence(xbc[:, :inner].double().reshape(T, H, V), xbc[:, inner:inner + G * N].double().reshape(T, G, N),
                             xbc[:, inner + G * N:].double().reshape(T, G, N), proj[:, ld - H:].double(), dtb.double(), A_log.double(), Dp.double())
        ref[n] = y.reshape(T, inner) * O.silu(proj[:, :inner].double())
    state = torch.full((3, H, N, V), 1e3, device=DEV)
    plan = [[("a", 20), ("b", 1)], [("b", 2), ("a", 1)], [("a", 16), ("b", 8)], [("c", 2)]]
    fed = {n: 0 for n in lens}
    got = {n: [] for n in lens}
    for step in plan:
        d, keep = dev_step(ops, [(c, fed[n], slot[n], [0]) for n, c in step], 4096)
        proj = torch.cat([data[n][0][fed[n]:fed[n] + c] for n, c in step]).to(DEV)
        xbc = torch.cat([data[n][1][fed[n]:fed[n] + c] for n, c in step]).to(DEV)
        out = torch.empty(proj.shape[0], inner, device=DEV)
        ops.ssm_scan(proj, 0, ld - H, xbc, A_log.to(DEV), Dp.to(DEV), dtb.to(DEV), state, d, H, V, N, G, out)
        o = 0
        for n, c in step:
            got[n].append(out[o:o + c].cpu())
            o += c
            fed[n] += c
    for n in lens:
        close(torch.cat(got[n]), ref[n], 2e-5)


def test_state_space_long_memory_shows(ops):
    """decay close to one and a single early input: every later output still carries it, so a state that is dropped or reset between
    steps shows"""
    H = G = 1
    N, V, T = 8, 4, 120
    inner, ld = H * V, 2 * H * V + 2 * N + H
    proj = torch.zeros(T, ld)
    proj[:, :inner] = 3.0                               # gate input
    proj[:, ld - 1] = -2.0                              # small step
    xbc = torch.zeros(T, inner + 2 * N)
    xbc[0, :inner] = 50.0
    xbc[0, inner:inner + N] = 1.0
    xbc[:, inner + N:] = 1.0
    A_log, Dp, dtb = torch.tensor([-6.0]), torch.zeros(1), torch.zeros(1)
    y = O.ssm_recurrence(xbc[:, :inner].double().reshape(T, 1, V), xbc[:, inner:inner + N].double().reshape(T, 1, N),
                         xbc[:, inner + N:].double().reshape(T, 1, N), proj[:, ld - 1:].double(), dtb.double(), A_log.double(), Dp.double())
    ref = y.reshape(T, inner) * O.silu(proj[:, :inner].double())
    state = torch.zeros((1, H, N, V), device=DEV)
    outs, fed = [], 0
    for c in [1, 2, 50] + [1] * 67:
        d, keep = dev_step(ops, [(c, fed, 0, [0])], 4096)
        out = torch.empty(c, inner, device=DEV)
        ops.ssm_scan(proj[fed:fed + c].to(DEV), 0, ld - 1, xbc[fed:fed + c].to(DEV), A_log.to(DEV), Dp.to(DEV), dtb.to(DEV), state, d, H, V, N, G, out)
        outs.append(out.cpu())
        fed += c
    got = torch.cat(outs)
    close(got, ref, 2e-5)
    assert got[-1].min() > 0.5 * got[0].max() > 0


@pytest.mark.parametrize("H,G,N,V", [(2, 1, 16, 24), (3, 3, 40, 33), (2, 2, 128, 64), (1, 1, 200, 9)])
def test_state_space_scan_segments_in_parallel(ops, H, G, N, V):
    """steps of many tokens cut every portion into segments that run side by side; the result is that of one walk in order, also for
    a portion that continues an earlier one, ends inside a segment, or shares the step with single tokens of other sequences"""
    lens = {"a": 700, "b": 150, "c": 131}
    inner = H * V
    ld = 2 * inner + 2 * G * N + H
    slot = {"a": 1, "b": 0, "c": 2}
    data, ref = {}, {}
    A_log, Dp, dtb = rnd(H, seed=180, scale=0.5) - 2.0, rnd(H, seed=181), rnd(H, seed=182)
    for i, (n, T) in enumerate(lens.items()):
        proj = rnd(T, ld, seed=183 + i)
        xbc = rnd(T, inner + 2 * G * N, seed=190 + i)
        data[n] = (proj, xbc)
        y = O.ssm_recurrence(xbc[:, :inner].double().reshape(T, H, V), xbc[:, inner:inner + G * N].double().reshape(T, G, N),
                             xbc[:, inner + G * N:].double().reshape(T, G, N), proj[:, ld - H:].double(), dtb.double(), A_log.double(), Dp.double())
        ref[n] = y.reshape(T, inner) * O.silu(proj[:, :inner].double())
    state = torch.full((3, H, N, V), 1e3, device=DEV)
    plan = [[("a", 300), ("b", 1)], [("b", 1), ("a", 129), ("c", 130)], [("a", 271), ("b", 148), ("c", 1)]]
    fed = {n: 0 for n in lens}
    got = {n: [] for n in lens}
    for step in plan:
        d, keep = dev_step(ops, [(c, fed[n], slot[n], [0]) for n, c in step], 4096)
        T = sum(c for _, c in step)
        proj = torch.cat([data[n][0][fed[n]:fed[n] + c] for n, c in step]).to(DEV)
        xbc = torch.cat([data[n][1][fed[n]:fed[n] + c] for n, c in step]).to(DEV)
        need = ops.ssm_scratch_floats(T, len(step), H, V, N)
        assert need > 0
        scratch = torch.full((need,), float("nan"), device=DEV)
        out = torch.empty(T, inner, device=DEV)
        ops.ssm_scan(proj, 0, ld - H, xbc, A_log.to(DEV), Dp.to(DEV), dtb.to(DEV), state, d, H, V, N, G, out, scratch)
        o = 0
        for n, c in step:
            got[n].append(out[o:o + c].cpu())
            o += c
            fed[n] += c
    for n in lens:
        close(torch.cat(got[n]), ref[n], 3e-5)


@pytest.mark.parametrize("H,G,D,V", [(8, 2, 32, 32), (5, 5, 18, 70), (6, 1, 128, 130)])
def test_attention_key_splits_agree_with_one_block(ops, H, G, D, V):
    """a long prompt in one step, then single tokens: with and without the work area (keys split among blocks or not)"""
    T = 450
    q, k, v, gate = attention_case(T, H, G, D, V, seed=300)
    ref = O.masked_attention(O.group_rms(q.double(), 1, 1e-6), O.group_rms(k.double(), 1, 1e-6), v.double(), 0.3, 200, 0, torch.sigmoid(gate.double())).reshape(T, -1)
    plan = [[("a", 380)]] + [[("a", 1)] for _ in range(70)]
    for split in (True, False):
        got = run_attention(ops, {"a": q}, {"a": k}, {"a": v}, {"a": gate}, 0.3, 200, 0, 1e-6, plan, 16, 40, split=split)["a"]
        close(got, ref, 2e-5)


@pytest.mark.parametrize("S,W,groups,taps", [(1, 40, 1, 1), (3, 48, 2, 3), (2, 33, 3, 4), (4, 1024, 2, 2), (6, 4224, 2, 4), (2, 64, 1, 6), (8, 8200, 5, 3)])
def test_stream_mix_norm_and_convolution_in_one_kernel(ops, S, W, groups, taps):
    """steps of one token per entry: stream update, collapse, norm and the carried convolution in one launch, against the separate
    operators' restatement over whole sequences; a sequence's first token must not read what its slot held before"""
    steps, eps = 9, 1e-4
    seqs = {"a": 0, "b": 3, "c": 1}                       # name -> slot
    X = {n: rnd(steps, S, W, seed=400 + i) for i, n in enumerate(seqs)}
    y = {n: rnd(steps, W, seed=410 + i) for i, n in enumerate(seqs)}
    outv, mix, inw, nw, cw = rnd(S, seed=420), rnd(S, S, seed=421), rnd(S, seed=422), rnd(W, seed=423), rnd(W, taps, seed=424)
    ref = {}
    for n in seqs:
        Xn = torch.einsum("st,nsw->ntw", mix.double(), X[n].double()) + outv.double()[None, :, None] * y[n].double()[:, None, :]
        h = O.group_rms(torch.einsum("s,nsw->nw", inw.double(), Xn), groups, eps, nw.double())
        ref[n] = h + O.causal_conv(h, cw.double())
    state = torch.full((4, max(taps - 1, 1), W), 77.0, device=DEV)
    post = torch.cat([outv, mix.reshape(-1)]).to(DEV)
    for t in range(steps):
        names = [n for n in seqs if not (n == "c" and t < 4)]       # c joins late, in a's and b's company
        pos = {n: t - (4 if n == "c" else 0) for n in names}
        d, keep = dev_step(ops, [(1, pos[n], seqs[n], [0]) for n in names], 4096)
        Xd = torch.stack([X[n][pos[n]] for n in names]).to(DEV).contiguous()
        yd = torch.stack([y[n][pos[n]] for n in names]).to(DEV).contiguous()
        out = torch.empty(len(names), W, device=DEV)
        ops.hc_norm_conv(Xd, yd, post, inw.to(DEV), nw.to(DEV), groups, eps, cw.to(DEV), state, d, out)
        for i, n in enumerate(names):
            close(out[i], ref[n][pos[n]], 2e-5)


@pytest.mark.parametrize("M,F,K", [(1, 37, 40), (4, 64, 96), (8, 130, 200)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_gate_up_projection_with_few_rows(ops, M, F, K, xdt):
    limit = 0.9
    x, wg, wu = rnd(M, K, seed=500).to(xdt), rnd(F, K, seed=501, scale=K ** -0.5).bfloat16(), rnd(F, K, seed=502, scale=K ** -0.5).bfloat16()
    g = torch.clamp(x.double() @ wg.double().T, max=limit)
    u = torch.clamp(x.double() @ wu.double().T, -limit, limit)
    ref = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    w_il = torch.stack([wg, wu], 1).reshape(2 * F, K).contiguous()
    out = torch.empty(M, F, device=DEV)
    ops.linear_gated(x.to(DEV), w_il.to(DEV), limit, 1.702, 1.0, out)
    close(out, ref, 1e-5)
