"""The operators the Gemosun design added to libb200seq, each alone, against the plain float64 restatement in
tests/gemosun_oracle.py: activation epilogues, the depth-averaged residual with its layer norms, rotary positions, values taken
from the keys, the sliding window with pooled blocks over scattered and reused pages, the expert router, expert projections in
both forms, the combine step."""
import numpy as np
import pytest
import torch

import gemosun_oracle as O

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


# ---- activations ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K,xdt", [(1, 38, 40, torch.float32), (5, 64, 96, torch.bfloat16), (8, 130, 200, torch.float32), (33, 40, 48, torch.bfloat16),
                                       (260, 130, 200, torch.bfloat16)])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_projection_with_gelu_gate_and_with_squared_relu(ops, M, N, K, xdt, odt):
    """few rows: the weight-streaming kernel; many rows: the tensor-core epilogues; both against product + activation"""
    x = rnd(M, K, seed=1, scale=1.5).to(xdt)
    w = rnd(N, K, seed=2, scale=K ** -0.5).bfloat16()
    z = x.double() @ w.double().T
    tol = 5e-6 if odt == torch.float32 else 6e-3
    out = torch.full((M, N // 2 + 2), 7.0, device=DEV, dtype=odt)
    ops.linear_act(x.to(DEV), w.to(DEV), ops.ACT_GELU_TANH, out[:, :N // 2])
    close(out[:, :N // 2], O.gelu_tanh(z[:, 0::2]) * z[:, 1::2], tol)
    assert bool((out[:, N // 2:] == 7.0).all())
    out = torch.full((M, N + 1), 7.0, device=DEV, dtype=odt)
    ops.linear_act(x.to(DEV), w.to(DEV), ops.ACT_RELU2, out[:, :N])
    close(out[:, :N], O.relu_squared(z), tol)
    assert bool((out[:, N:] == 7.0).all()) and ops.error_flags() == 0
    # the activation alone, on a product that is in memory
    zf = z.float().to(DEV)
    o2 = torch.empty(M, N // 2, device=DEV, dtype=odt)
    ops.act(zf, ops.ACT_GELU_TANH, o2)
    close(o2, O.gelu_tanh(zf.cpu().double()[:, 0::2]) * zf.cpu().double()[:, 1::2], tol)
    o3 = torch.empty(M, N, device=DEV, dtype=odt)
    ops.act(zf, ops.ACT_RELU2, o3)
    close(o3, O.relu_squared(zf.cpu().double()), tol)


# ---- depth-averaged residual + layer norms ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,W,n_prev", [(5, 48, 0), (9, 44, 1), (3, 130, 4), (40, 1024, 7), (2, 33, 2)])
def test_depth_average_and_two_layer_norms(ops, T, W, n_prev):
    eps = 1e-3
    cap = T + 3
    hist = rnd(n_prev + 1, cap, W, seed=3).to(DEV)
    x, y1, y2 = rnd(T, W, seed=4) + 0.7, rnd(T, W, seed=5), rnd(T, W, seed=6)
    dwa = rnd(n_prev + 1, seed=7, scale=0.5)
    w1, w2 = 1 + rnd(W, seed=8, scale=0.2), rnd(W, seed=9)
    new = x.double() + (y1.double() + y2.double())
    avg = sum(dwa[j].double() * hist[j, :T].cpu().double() for j in range(n_prev)) + dwa[n_prev].double() * new
    hist_out = torch.zeros(T, W, device=DEV)
    x_out = torch.zeros(T, W, device=DEV)
    o1, o2 = torch.empty(T, W, device=DEV), torch.empty(T, W, device=DEV, dtype=torch.float32)
    ops.depth_norm(x.to(DEV), o1, w1.to(DEV), eps, out2=o2, w2=w2.to(DEV), y1=y1.to(DEV), y2=y2.to(DEV), hist=hist, n_prev=n_prev, dwa=dwa.to(DEV),
                   hist_out=hist_out, x_out=x_out)
    close(hist_out, new, 1e-6)
    close(x_out, avg, 2e-6)
    close(o1, O.layer_norm(avg, w1.double(), eps), 1e-5)
    close(o2, O.layer_norm(avg, w2.double(), eps), 1e-5)
    # one branch, no averaging, bfloat16 output, only some rows
    rows = torch.tensor([T - 1, 0], dtype=torch.int32)
    ob = torch.empty(2, W, device=DEV, dtype=torch.bfloat16)
    ops.depth_norm(x.to(DEV), ob, w1.to(DEV), eps, y1=y1.to(DEV), x_out=x_out, rows=rows.to(DEV))
    close(ob.float(), O.layer_norm((x.double() + y1.double())[rows.long()], w1.double(), eps), 6e-3)
    # the norm alone (first layer)
    ops.depth_norm(x.to(DEV), o1, w1.to(DEV), eps)
    close(o1, O.layer_norm(x.double(), w1.double(), eps), 1e-5)


# ---- attention ------------------------------------------------------------------------------------------------------------------------
def run_attention(ops, q, k, gate, scale, window, pool, rot, plan, block_size, n_pages, act=torch.float32, seed=0, values_from_keys=True, v=None):
    """feeds sequences (dict name -> [T, heads, D] of whole sequences, before rotation) through prep + attend as the plan says; pages
    come from a shuffled list and go back when a sequence ends; pools start with large values; returns name -> [T, H * V]"""
    names = list(q)
    H, D = q[names[0]].shape[1:]
    G = k[names[0]].shape[1]
    V = D if values_from_keys else v[names[0]].shape[2]
    per_page = -(-block_size // pool) if pool else 1
    kpool = torch.full((n_pages, block_size, G, D), 1e4, device=DEV)
    vpool = torch.full((n_pages, block_size, G, V), 1e4, device=DEV)
    kpp = torch.full((n_pages, per_page, G, D), 1e4, device=DEV)
    vpp = torch.full((n_pages, per_page, G, V), 1e4, device=DEV)
    freq = None
    amp = 1.0
    if rot:
        f, amp = O.rotary_frequencies(rot)
        freq = torch.tensor(f, dtype=torch.float32, device=DEV)
    desc = ops.attn_desc(H, G, D, V, scale, values_from_keys=values_from_keys, gated=gate is not None, window=window, pool=pool, rot_freq=freq, rot_scale=amp)
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
        rows = [torch.cat([q[n][fed[n]:fed[n] + c].reshape(c, -1), k[n][fed[n]:fed[n] + c].reshape(c, -1)]
                          + ([] if values_from_keys else [v[n][fed[n]:fed[n] + c].reshape(c, -1)])
                          + ([gate[n][fed[n]:fed[n] + c]] if gate is not None else []), 1) for n, c in step]
        proj = torch.cat(rows).contiguous().to(DEV)
        assert proj.shape[1] == desc.width
        out = torch.empty(proj.shape[0], H * V, device=DEV, dtype=act)
        ops.attn_prep_ex(proj, d, desc, kpool, vpool, kpp, vpp)
        ctx = max(len(p) for p in pages.values()) * block_size
        need = ops.attn_scratch_floats(proj.shape[0], len(step), H, G, V, min(ctx, window or ctx) + (ctx // pool if pool else 0))
        scratch = torch.full((max(need, 1),), float("nan"), device=DEV)
        ops.attn_ex(proj, d, desc, kpool, vpool, out, scratch, kpp, vpp)
        o = 0
        for n, c in step:
            got[n].append(out[o:o + c].float().cpu())
            o += c
            fed[n] += c
        for n, c in step:
            if fed[n] == q[n].shape[0]:
                free.extend(pages[n])
                pages[n] = []
    assert ops.error_flags() == 0
    return {n: torch.cat(got[n]) for n in names}


def reference_attention(q, k, gate, scale, window, pool, rot, v=None):
    qd, kd = q.double(), k.double()
    vd = kd.clone() if v is None else v.double()
    o = O.window_pool_attention(O.rotate(qd, rot), O.rotate(kd, rot), vd, scale, window, pool, gate.double() if gate is not None else None)
    return o.reshape(q.shape[0], -1)


ROT = {"dims": 8, "base": 50.0, "scaling": {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0}}


@pytest.mark.parametrize("H,G,D,window,pool,bs,rot", [(4, 2, 16, 24, 4, 16, ROT), (3, 3, 10, 7, 3, 4, {"dims": 10, "base": 9.0}), (2, 1, 64, 16, 16, 16, None),
                                                      (4, 4, 8, 1, 1, 8, {"dims": 2, "base": 3.0}), (6, 2, 12, 10, 40, 16, ROT), (2, 2, 20, 9, 0, 16, ROT),
                                                      (2, 1, 16, 0, 0, 16, ROT)])
def test_window_with_pooled_blocks_in_a_mixed_batch(ops, H, G, D, window, pool, bs, rot):
    """unequal sequences fed in portions beside single tokens, through scattered pages that a finished sequence hands on"""
    scale = 0.37
    lens = {"a": 90, "b": 30, "c": 3, "d": 41}
    q = {n: rnd(T, H, D, seed=50 + 10 * i) for i, (n, T) in enumerate(lens.items())}
    k = {n: rnd(T, G, D, seed=51 + 10 * i) for i, (n, T) in enumerate(lens.items())}
    gate = {n: rnd(T, H, seed=52 + 10 * i) for i, (n, T) in enumerate(lens.items())}
    plan = [[("a", 40), ("b", 2)], [("b", 1), ("a", 1), ("c", 3)], [("a", 2), ("b", 27)], [("a", 32), ("d", 7)], [("d", 2), ("a", 1)], [("a", 14), ("d", 32)]]
    got = run_attention(ops, q, k, gate, scale, window, pool, rot, plan, bs, n_pages=-(-90 // bs) + -(-30 // bs) + 4)
    for n in lens:
        close(got[n], reference_attention(q[n], k[n], gate[n], scale, window, pool, rot), 2e-5)


def test_own_value_projection_and_unequal_value_size(ops):
    """the same kernels with a value projection of another size than the keys (no rotation, no pooling of the other design's kind)"""
    H, G, D, V, window, pool = 4, 2, 12, 20, 6, 2
    T = 50
    q, k, v = rnd(T, H, D, seed=1), rnd(T, G, D, seed=2), rnd(T, G, V, seed=3)
    got = run_attention(ops, {"a": q}, {"a": k}, None, 0.3, window, pool, None, [[("a", 33)], [("a", 2)]] + [[("a", 1)]] * 15, 8, 8, values_from_keys=False, v={"a": v})["a"]
    close(got, reference_attention(q, k, None, 0.3, window, pool, None, v=v), 2e-5)


@pytest.mark.parametrize("decode", [False, True])
def test_window_and_pool_edges_show(ops, decode):
    """the first key of one block points where every query points and (being also the value) stands out in the output, which then
    shows at once whether the key is seen itself (inside the window), not at all (it has left the window but its block does not yet
    lie wholly before the window), or through the block's mean"""
    H = G = 1
    D, window, pool, bs, T = 16, 12, 8, 16, 80
    hot = 3 * pool                                     # position 24, first of the block 24 .. 31
    q = torch.zeros(T, H, D)
    q[:, 0, 0] = 1.0
    k = rnd(T, G, D, seed=60, scale=0.02)
    k[hot] = 0
    k[hot, 0, 0] = 1.0
    k[hot, 0, 1] = 50.0                                # shows in the output (the values are the keys)
    plan = [[("a", 20)]] + [[("a", 1)]] * 60 if decode else [[("a", 30)], [("a", 2)], [("a", 11)], [("a", 37)]]
    got = run_attention(ops, {"a": q}, {"a": k}, None, 40.0, window, pool, None, plan, bs, n_pages=6)["a"]
    close(got, reference_attention(q, k, None, 40.0, window, pool, None), 2e-5)
    assert abs(got[hot - 1, 1]) < 2 and got[hot, 1] > 49              # causal
    assert got[hot + window - 1, 1] > 49                               # position 35: the last one with key 24 in its window
    assert abs(got[hot + window, 1]) < 2                               # position 36: just outside, and the block is not pooled yet
    first_pooled = hot + pool - 1 + window                             # 43: the block's last position is now `window` back
    assert abs(got[first_pooled - 1, 1]) < 2                           # pool_out
    assert 3 < got[first_pooled, 1] < 50.0 / pool + 0.5                # pool_in: the mean of eight values, one of them 50
    assert 3 < got[T - 1, 1] < 50.0 / pool + 0.5


def test_pooled_block_far_back_among_hundreds(ops):
    """one block far back carries keys the queries point at: its mean key must win the soft-max over hundreds of other pooled blocks and
    the window, through many pages, in a long portion and in single tokens"""
    H, G, D, window, pool, bs, T = 2, 1, 32, 64, 4, 16, 900
    q = torch.zeros(T, H, D)
    q[:, :, 3] = 1.0
    k = rnd(T, G, D, seed=70, scale=0.05)
    far = 5                                            # positions 20 .. 23, in the second page
    k[far * pool:(far + 1) * pool] = 0
    k[far * pool:(far + 1) * pool, 0, 3] = 1.0
    k[far * pool:(far + 1) * pool, 0, 4] = -30.0
    plan = [[("a", 700)], [("a", 2)], [("a", 150)]] + [[("a", 1)]] * 48
    got = run_attention(ops, {"a": q}, {"a": k}, None, 30.0, window, pool, None, plan, bs, n_pages=58)["a"]
    ref = reference_attention(q, k, None, 30.0, window, pool, None)
    close(got, ref, 2e-5)
    assert got[T - 1, 4] < -29 and got[699, 4] < -29 and got[701, 4] < -29


# ---- mixture of experts ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,E,top,groups,keep", [(7, 8, 2, 4, 2), (40, 16, 5, 2, 1), (3, 6, 3, 3, 2), (5, 5, 1, 5, 3), (9, 12, 5, 1, 1), (2, 64, 8, 8, 4), (4, 3, 3, 1, 1)])
def test_router_choice_and_weights(ops, T, E, top, groups, keep):
    z = rnd(T, E + 2, seed=80, scale=2.0)
    ids = torch.full((T * top,), -1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T * top, device=DEV)
    cnt = torch.full((E,), 99, dtype=torch.int32, device=DEV)
    ops.moe_route(z.to(DEV)[:, :E], E, groups, keep, top, ids, wts, cnt)
    ids, wts = ids.cpu().view(T, top), wts.cpu().view(T, top)
    for t in range(T):
        chosen, w = O.route(torch.sigmoid(z[t, :E].double()), top, groups, keep)
        assert ids[t].tolist() == chosen
        close(wts[t], w, 1e-6)
    assert cnt.cpu().tolist() == [int((ids == e).sum()) for e in range(E)]


@pytest.mark.parametrize("T,E,extra,top,groups,keep,K,xdt", [(1, 8, 1, 2, 4, 2, 40, torch.float32), (8, 16, 0, 5, 2, 1, 96, torch.bfloat16), (3, 6, 2, 3, 3, 2, 33, torch.float32),
                                                             (4, 12, 1, 4, 1, 1, 200, torch.bfloat16)])
def test_router_projection_and_choice_in_one_kernel(ops, T, E, extra, top, groups, keep, K, xdt):
    """single-token steps: the stacked router weight (experts' rows + rows riding behind them) projected and the choice made at once"""
    x = rnd(T, K, seed=90).to(xdt)
    w = rnd(E + extra, K, seed=91, scale=3.0 * K ** -0.5).bfloat16()
    z = torch.full((T, E + extra + 1), 7.0, device=DEV)
    ids = torch.full((T * top,), -1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T * top, device=DEV)
    ops.moe_router(x.to(DEV), w.to(DEV), E, groups, keep, top, z[:, :E + extra], ids, wts)
    zr = x.double() @ w.double().T
    close(z[:, :E + extra], zr, 5e-6)
    assert bool((z[:, E + extra:] == 7.0).all())
    for t in range(T):
        chosen, wt = O.route(torch.sigmoid(zr[t, :E]), top, groups, keep)
        assert ids.cpu().view(T, top)[t].tolist() == chosen
        close(wts.cpu().view(T, top)[t], wt, 2e-6)


@pytest.mark.parametrize("T,E,top,N,K,xdt", [(3, 4, 2, 24, 40, torch.float32), (70, 8, 3, 50, 36, torch.float32), (5, 6, 1, 33, 64, torch.bfloat16),
                                             (130, 5, 2, 72, 96, torch.bfloat16), (600, 9, 3, 200, 136, torch.bfloat16)])
def test_expert_projections_per_pair_and_over_sorted_tiles(ops, T, E, top, N, K, xdt):
    """up (gathers the token's row, squared relu) and down (plain) in both forms give what each pair's expert gives alone; the combine
    step weighs them in choice order and adds the gated shared branch"""
    g = torch.Generator().manual_seed(5)
    x = rnd(T, K, seed=81).to(xdt)
    w_up, w_down = rnd(E, N, K, seed=82, scale=K ** -0.5).bfloat16(), rnd(E, K, N, seed=83, scale=N ** -0.5).bfloat16()
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    pairs = T * top
    idf = ids.reshape(-1)
    mid_ref = torch.stack([O.relu_squared(x[p // top].double() @ w_up[idf[p]].double().T) for p in range(pairs)])
    shared, gz = rnd(T, K, seed=84), rnd(T, 3, seed=85)
    for form in ("rows", "tiles"):
        ids_d, wts_d = idf.to(DEV), wts.reshape(-1).to(DEV)
        order = offs = slot = None
        if form == "tiles":
            cnt = torch.bincount(idf.long(), minlength=E).to(torch.int32).to(DEV)
            order, offs, slot = torch.empty(pairs, dtype=torch.int32, device=DEV), torch.empty(E + 1, dtype=torch.int32, device=DEV), torch.empty(pairs, dtype=torch.int32, device=DEV)
            ops.moe_sort(ids_d, pairs, E, cnt, offs, order, slot)
            oc = order.cpu().long()
            assert sorted(oc.tolist()) == list(range(pairs)) and bool((idf[oc][1:] >= idf[oc][:-1]).all())        # by expert ...
            assert all(oc[i] < oc[i + 1] for i in range(pairs - 1) if idf[oc[i]] == idf[oc[i + 1]])                # ... and stable
            assert offs.cpu().tolist() == [0] + torch.cumsum(torch.bincount(idf.long(), minlength=E), 0).tolist()
            assert bool((slot.cpu().long()[oc] == torch.arange(pairs)).all())
        mid = torch.full((pairs, N), 7.0, device=DEV, dtype=xdt)
        ops.moe_linear(x.to(DEV), top, w_up.to(DEV), ids_d, order, offs, pairs, ops.ACT_RELU2, mid)
        perm = order.cpu().long() if order is not None else torch.arange(pairs)
        close(mid.float(), mid_ref[perm], 5e-6 if xdt == torch.float32 else 6e-3)
        if form == "tiles" and xdt == torch.bfloat16 and pairs >= 32:
            # the tokens' rows gathered into sorted order first: the same projection on tensor-core tiles, one group of rows per expert
            xs = torch.full((pairs, K), 7.0, device=DEV, dtype=xdt)
            ops.moe_gather(x.to(DEV), top, order, pairs, xs)
            assert torch.equal(xs.cpu(), x[perm // top])
            mid_tc = torch.full((pairs + 1, N), 7.0, device=DEV, dtype=xdt)
            ops.moe_linear(xs, 0, w_up.to(DEV), ids_d, order, offs, pairs, ops.ACT_RELU2, mid_tc[:pairs])
            close(mid_tc[:pairs].float(), mid_ref[perm], 6e-3)
            assert bool((mid_tc[pairs:] == 7.0).all()) and ops.error_flags() == 0
        ys = torch.full((pairs, K), 7.0, device=DEV)
        ops.moe_linear(mid, 0, w_down.to(DEV), ids_d, order, offs, pairs, ops.ACT_NONE, ys)
        ys_ref = torch.stack([mid.float().cpu().double()[r] @ w_down[idf[perm[r]]].double().T for r in range(pairs)])
        close(ys, ys_ref, 5e-6)
        y = torch.empty(T, K, device=DEV)
        ops.moe_combine(ys, wts_d, slot, T, top, shared.to(DEV), gz.to(DEV)[:, 1], y)
        inv = torch.empty(pairs, dtype=torch.long)
        inv[perm] = torch.arange(pairs)
        y_ref = (wts.double()[:, :, None] * ys_ref[inv].view(T, top, K)).sum(1) + torch.sigmoid(gz[:, 1].double())[:, None] * shared.double()
        close(y, y_ref, 5e-6)
        ops.moe_combine(ys, wts_d, slot, T, top, None, None, y)
        close(y, (wts.double()[:, :, None] * ys_ref[inv].view(T, top, K)).sum(1), 5e-6)
