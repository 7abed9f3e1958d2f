"""Layer-list models: a model is a list of layers, each one token mixer (attention over the paged KV pool, or a state-space
recurrence with per-slot state) plus an optional feed-forward, wrapped in the pieces a design switches on: several residual
streams with learned mixing, grouped RMS norms, a short carried-state convolution in front of every sublayer.  The mechanisms
are parameterised (window / chunk size, score scale, unit-norm epsilon, gate, state size, clamp limit, ...) so that another
design can list them in another combination; blazr_b200/fenorax.py maps one design's config.json onto these specs.

One step function serves prefill, decode and mixed steps: `LayeredModel.forward(step)` takes a flat batch of tokens (prompt
portions beside single decoded tokens, blazr_b200/batch.py: build_step) and runs every layer once over all of them.  All math
runs in libb200seq kernels (blazr_b200/seqops.py); PyTorch holds the buffers.  What must be 32-bit is 32-bit in both modes:
the residual streams, norms, scores and soft-max, recurrent state, step sizes and decays, the KV pool.  `dtype` only selects
the activation type fed to the linear layers (bfloat16: tensor-core tiles; float32: exact fma tiles).

The decode-only step of a fixed batch size is captured into a CUDA graph (reference src/engine/cuda_graphs.rs:101-130).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from . import seqops
from .batch import StepArrays


# ---- specs -----------------------------------------------------------------------------------------------------------------
@dataclass
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int                 # per-head query / key size
    vdim: int                # per-head value size
    scale: float
    chunk: int = 0           # > 0: a query sees only keys of its own chunk of this many positions (counted from position 0)
    window: int = 0          # > 0: a query sees only the last `window` positions
    qk_unit_norm: bool = True
    gated: bool = True       # one sigmoid gate per head on the output


@dataclass
class SsmSpec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int                # taps of the convolution over x | B | C


@dataclass
class DenseFfSpec:
    ff: int
    limit: float
    alpha: float = 1.702     # gate activation g * sigmoid(alpha * g)
    up_shift: float = 1.0    # (up + up_shift)


@dataclass
class LayerSpec:
    kind: str                # "attention" | "ssm"
    mixer: object
    ff: Optional[DenseFfSpec]


@dataclass
class LayeredConfig:
    name: str
    vocab: int
    width: int
    streams: int
    norm_groups: int
    eps: float
    canon_taps: int          # taps of the convolution in front of every sublayer
    embed_scale: float
    layers: List[LayerSpec] = field(default_factory=list)


class _Workspace:
    """device buffers of one step capacity (addresses stay put: a step of fixed shape can be graph-captured)"""

    def __init__(self, model: "LayeredModel", cap: int):
        cfg, dev = model.cfg, model.dev
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=model.act_dtype, device=dev)
        self.cap = cap
        W = cfg.width
        self.X = torch.empty((cap, cfg.streams, W), **f32)
        self.h = torch.empty((cap, W), **f32)
        self.a = torch.empty((cap, W), **act)
        self.y = torch.empty((cap, W), **f32)
        self.proj = torch.empty((cap, model.max_proj), **f32)
        self.xbc = torch.empty((cap, max(1, model.max_xbc)), **f32)
        self.inner_f = torch.empty((cap, max(1, model.max_inner)), **f32)
        self.inner_a = torch.empty((cap, max(1, model.max_inner)), **act)
        self.fin = torch.empty((cap, W), **act)
        self.logits = torch.empty((cap, cfg.vocab), **f32)
        self.scratch = torch.empty(max(1, model.scratch_floats(cap)), **f32)      # work area: segmented state-space scan, key-split attention
        self.next_ids = torch.empty((cap,), dtype=torch.int32, device=dev)
        # int32 step arrays in one buffer: ids | ent | pos | want | start | slot | pos0 | block_table
        B, mb = model.max_seqs, model.max_blocks
        self.off = {}
        o = 0
        for k, n in (("ids", cap), ("ent", cap), ("pos", cap), ("want", cap), ("start", B + 1), ("slot", B), ("pos0", B), ("bt", B * mb)):
            self.off[k] = (o, n)
            o += -(-n // 4) * 4
        self.meta = torch.zeros(o, dtype=torch.int32, device=dev)
        self.copied = None
        self.meta_host = torch.zeros(o, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(o, dtype=torch.int32)

    def view(self, k: str) -> torch.Tensor:
        o, n = self.off[k]
        return self.meta[o:o + n]


class LayeredModel:
    """weights + per-layer cache / state + the step function"""

    def __init__(self, cfg: LayeredConfig, tensors, device, dtype: str = "bfloat16"):
        """tensors: name -> torch CPU tensor (callable or mapping with the checkpoint's names)"""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.act_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        get = tensors if callable(tensors) else tensors.__getitem__
        dev = self.dev
        S, W = cfg.streams, cfg.width
        if S > 8 or cfg.canon_taps > 8:
            raise ValueError("at most 8 residual streams and 8 convolution taps")

        def lin(*names):   # linear weights stay bfloat16; several projections of one input are stacked along N (one launch)
            parts = []
            for n in names:
                t = get(n)
                if t.dtype != torch.bfloat16:
                    if dtype == "float32" and t.dtype in (torch.float32, torch.float64) and not torch.equal(t.bfloat16().to(t.dtype), t):
                        raise ValueError(f"{n}: float32 mode needs weights that are exact in bfloat16")
                    t = t.to(torch.bfloat16)
                parts.append(t)
            return torch.cat(parts, 0).contiguous().to(dev)

        def vec(name):
            return get(name).to(torch.float32).contiguous().to(dev)

        def hc(pre):    # (in [S], post = out [S] | mix [S, S])
            return vec(pre + "in"), torch.cat([get(pre + "out").float().reshape(-1), get(pre + "mix").float().reshape(-1)]).contiguous().to(dev)

        self.embed = lin("embed")
        self.final_norm = vec("final.norm")
        if tuple(self.embed.shape) != (cfg.vocab, W) or self.final_norm.numel() != W:
            raise ValueError("embedding / final norm shapes do not fit the configuration")
        self.ones_in = torch.ones(S, dtype=torch.float32, device=dev)
        self.layers: List[Dict[str, object]] = []
        self.max_proj = self.max_xbc = self.max_inner = 1
        self.weight_bytes = self.embed.numel() * 2
        for i, ls in enumerate(cfg.layers):
            L: Dict[str, object] = {"spec": ls}
            p = f"l{i}."
            L["norm1"], L["canon1"] = vec(p + "norm1"), vec(p + "canon1")
            L["hc1_in"], L["hc1_post"] = hc(p + "hc1.")
            m = ls.mixer
            if ls.kind == "attention":
                names = [p + "mix.q", p + "mix.k", p + "mix.v"] + ([p + "mix.g"] if m.gated else [])
                L["w_in"] = lin(*names)
                L["w_o"] = lin(p + "mix.o")
                n_in = m.heads * m.dim + m.kv_heads * (m.dim + m.vdim) + (m.heads if m.gated else 0)
                if tuple(L["w_in"].shape) != (n_in, W) or tuple(L["w_o"].shape) != (W, m.heads * m.vdim):
                    raise ValueError(f"layer {i}: attention tensor shapes do not fit the configuration")
                self.max_inner = max(self.max_inner, m.heads * m.vdim)
            elif ls.kind == "ssm":
                L["w_in"] = lin(p + "mix.in")
                L["w_o"] = lin(p + "mix.o")
                L["conv_w"], L["conv_b"] = vec(p + "mix.conv"), vec(p + "mix.conv.b")
                L["dt_bias"], L["A_log"], L["D"], L["mnorm"] = vec(p + "mix.dt_bias"), vec(p + "mix.A_log"), vec(p + "mix.D"), vec(p + "mix.norm")
                inner, gn = m.heads * m.vdim, m.groups * m.state
                if tuple(L["w_in"].shape) != (2 * inner + 2 * gn + m.heads, W) or tuple(L["conv_w"].shape) != (inner + 2 * gn, m.conv):
                    raise ValueError(f"layer {i}: state-space tensor shapes do not fit the configuration")
                self.max_inner = max(self.max_inner, inner)
                self.max_xbc = max(self.max_xbc, inner + 2 * gn)
            else:
                raise ValueError(f"layer {i}: unknown mixer kind {ls.kind}")
            self.max_proj = max(self.max_proj, L["w_in"].shape[0])
            self.weight_bytes += (L["w_in"].numel() + L["w_o"].numel()) * 2
            if ls.ff is not None:
                L["norm2"], L["canon2"] = vec(p + "norm2"), vec(p + "canon2")
                L["hc2_in"], L["hc2_post"] = hc(p + "hc2.")
                gu = lin(p + "mlp.gate", p + "mlp.up")          # stored with alternating rows (gate j, up j): the pair meets in one warp
                L["w_gu"] = gu.view(2, ls.ff.ff, W).transpose(0, 1).reshape(2 * ls.ff.ff, W).contiguous()
                L["w_down"] = lin(p + "mlp.down")
                if tuple(gu.shape) != (2 * ls.ff.ff, W) or tuple(L["w_down"].shape) != (W, ls.ff.ff):
                    raise ValueError(f"layer {i}: feed-forward tensor shapes do not fit the configuration")
                self.max_proj = max(self.max_proj, 2 * ls.ff.ff)
                self.max_inner = max(self.max_inner, ls.ff.ff)
                self.weight_bytes += (L["w_gu"].numel() + L["w_down"].numel()) * 2
            self.layers.append(L)
        self.max_seqs = self.max_blocks = self.block_size = 0
        self._ws: Dict[int, _Workspace] = {}
        self._graphs: Dict[int, object] = {}
        self.use_graphs = True

    # ---- cache and state -------------------------------------------------------------------------------------------------------
    def allocate(self, num_blocks: int, block_size: int, max_seqs: int, max_seq_tokens: int) -> None:
        """KV pools for `num_blocks` pages, state for `max_seqs` slots; block tables hold up to max_seq_tokens positions"""
        dev, cfg = self.dev, self.cfg
        f32 = dict(dtype=torch.float32, device=dev)
        self.block_size, self.max_seqs = block_size, max_seqs
        self.max_blocks = max(1, -(-max_seq_tokens // block_size))
        hist = cfg.canon_taps - 1
        for L in self.layers:
            ls = L["spec"]
            m = ls.mixer
            L["canon1_state"] = torch.zeros((max_seqs, max(hist, 1), cfg.width), **f32)
            if ls.ff is not None:
                L["canon2_state"] = torch.zeros((max_seqs, max(hist, 1), cfg.width), **f32)
            if ls.kind == "attention":
                L["kpool"] = torch.zeros((max(1, num_blocks), block_size, m.kv_heads, m.dim), **f32)
                L["vpool"] = torch.zeros((max(1, num_blocks), block_size, m.kv_heads, m.vdim), **f32)
            else:
                L["conv_state"] = torch.zeros((max_seqs, max(m.conv - 1, 1), m.heads * m.vdim + 2 * m.groups * m.state), **f32)
                L["ssm_state"] = torch.zeros((max_seqs, m.heads, m.state, m.vdim), **f32)
        self._ws.clear()
        self._graphs.clear()

    def scratch_floats(self, cap: int) -> int:
        """floats of the largest work area any layer wants for a step of up to `cap` tokens"""
        need = 0
        seen = set()
        for L in self.layers:
            m = L["spec"].mixer
            if L["spec"].kind == "ssm":
                need = max(need, seqops.ssm_scratch_floats(cap, self.max_seqs, m.heads, m.vdim, m.state))
            else:
                keys = self.max_blocks * self.block_size
                keys = min(keys, m.chunk) if m.chunk > 0 else keys
                keys = min(keys, m.window) if m.window > 0 else keys
                key = (m.heads, m.kv_heads, m.vdim, keys)
                if key not in seen:     # the split count falls as the step grows: the largest need is at some T <= cap
                    seen.add(key)
                    need = max([need] + [seqops.attn_scratch_floats(T, 1, m.heads, m.kv_heads, m.vdim, keys) for T in range(1, cap + 1)])
        return need

    def cache_bytes(self) -> int:
        keys = ("canon1_state", "canon2_state", "kpool", "vpool", "conv_state", "ssm_state")
        return sum(L[k].numel() * 4 for L in self.layers for k in keys if k in L)

    def _workspace(self, T: int) -> _Workspace:
        cap = 8
        while cap < T:
            cap *= 2
        ws = self._ws.get(cap)
        if ws is None:
            ws = self._ws[cap] = _Workspace(self, cap)
        return ws

    # ---- the step ----------------------------------------------------------------------------------------------------------------
    def _upload(self, ws: _Workspace, sa: StepArrays) -> None:
        if sa.B > self.max_seqs or sa.block_table.shape[1] > self.max_blocks:
            raise ValueError("step exceeds the engine's request or block-table capacity")
        h = ws.meta_host
        if ws.copied is not None:
            ws.copied.synchronize()    # the previous step's copy out of the pinned buffer must be over before it is rewritten
        hn = h.numpy()
        for k, arr in (("ids", sa.tok_ids), ("ent", sa.tok_ent), ("pos", sa.tok_pos), ("want", sa.want_rows), ("start", sa.ent_start), ("slot", sa.ent_slot),
                       ("pos0", sa.ent_pos0)):
            o, _ = ws.off[k]
            hn[o:o + arr.shape[0]] = arr
        o, _ = ws.off["bt"]
        bt = np.zeros((sa.B, self.max_blocks), dtype=np.int32)
        bt[:, :sa.block_table.shape[1]] = sa.block_table
        hn[o:o + bt.size] = bt.reshape(-1)
        ws.meta.copy_(h, non_blocking=True)
        if self.dev.type == "cuda":
            ws.copied = torch.cuda.Event()
            ws.copied.record(torch.cuda.current_stream(self.dev))

    def _desc(self, ws: _Workspace, T: int, B: int) -> seqops.StepDesc:
        ptr = lambda k: ws.view(k).data_ptr()
        return seqops.StepDesc(ptr("ent"), ptr("pos"), ptr("start"), ptr("slot"), ptr("pos0"), ptr("bt"), T, B, self.max_blocks, self.block_size)

    def forward(self, sa: StepArrays, sample: bool = False, debug_layers: Optional[list] = None) -> torch.Tensor:
        """runs one step; returns f32 logits [R, vocab] of the wanted rows (a view of a buffer the next step overwrites);
        sample: also leaves the greedy token of every wanted row in `self.last_ids` (int32 [R], device)"""
        if not self.block_size:
            raise RuntimeError("allocate() the cache first")
        T, B, R = sa.T, sa.B, int(sa.want_rows.shape[0])
        ws = self._workspace(T)
        self._upload(ws, sa)
        graphable = self.use_graphs and debug_layers is None and sa.decode_only and R == T and self.dev.type == "cuda" \
            and bool((sa.want_rows == np.arange(T)).all())
        if graphable:
            key = (T, bool(sample))
            g = self._graphs.get(key)
            if g is None:
                self._run(ws, T, B, R, sample, None)        # warm-up outside capture (module loading, attribute calls)
                torch.cuda.synchronize(self.dev)
                # the warm-up run advanced the carried state: capture must not run it twice -> capture on a side stream, then the
                # captured launches are NOT executed; state was advanced exactly once by the warm-up.
                g = torch.cuda.CUDAGraph()
                s = torch.cuda.Stream(self.dev)
                s.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(s):
                    with torch.cuda.graph(g, stream=s):
                        self._run(ws, T, B, R, sample, None)
                torch.cuda.current_stream(self.dev).wait_stream(s)
                self._graphs[key] = g
            else:
                g.replay()
        else:
            self._run(ws, T, B, R, sample, debug_layers)
        self.last_ids = ws.next_ids[:R]
        return ws.logits[:R]

    def _run(self, ws: _Workspace, T: int, B: int, R: int, sample: bool, debug_layers: Optional[list]) -> None:
        cfg = self.cfg
        ops = seqops
        st = self._desc(ws, T, B)
        X, h, a, y = ws.X[:T], ws.h[:T], ws.a[:T], ws.y[:T]
        ops.embed_streams(self.embed, ws.view("ids"), cfg.embed_scale, X)
        y_prev = post_prev = None
        for L in self.layers:
            ls: LayerSpec = L["spec"]
            for q in ((1, 2) if ls.ff is not None else (1,)):
                if T == B:      # one token per entry: the convolution's history is all in the carried state -> one kernel
                    ops.hc_norm_conv(X, y_prev, post_prev, L[f"hc{q}_in"], L[f"norm{q}"], cfg.norm_groups, cfg.eps, L[f"canon{q}"], L[f"canon{q}_state"], st, a)
                else:
                    ops.hc_norm(X, y_prev, post_prev, L[f"hc{q}_in"], L[f"norm{q}"], cfg.norm_groups, cfg.eps, h)
                    ops.causal_conv(h, L[f"canon{q}"], None, L[f"canon{q}_state"], st, ops.CONV_RESIDUAL, a)
                if q == 2:
                    self._dense_ff(L, ls.ff, ws, T, a, y)
                elif ls.kind == "attention":
                    self._attention(L, ls.mixer, ws, st, T, a, y)
                else:
                    self._ssm(L, ls.mixer, ws, st, T, a, y)
                y_prev, post_prev = y, L[f"hc{q}_post"]
            if debug_layers is not None:   # the streams' sum after this layer (the pending stream update applied on a copy)
                S = cfg.streams
                outv, mix = post_prev[:S], post_prev[S:].reshape(S, S)
                Xn = torch.einsum("st,nsw->ntw", mix, X) + outv[None, :, None] * y[:, None, :]
                debug_layers.append(Xn.sum(1).cpu())
        if R:
            ops.hc_norm(X, y_prev, post_prev, self.ones_in, self.final_norm, cfg.norm_groups, cfg.eps, ws.fin[:R], rows=ws.view("want")[:R])
            ops.linear(ws.fin[:R], self.embed, ws.logits[:R])
            if sample:
                ops.argmax(ws.logits[:R], ws.next_ids[:R])

    def _attention(self, L, m: AttentionSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        n_in = L["w_in"].shape[0]
        qkvg = ws.proj[:T, :n_in]
        seqops.linear(a, L["w_in"], qkvg)
        seqops.attn_prep(qkvg, st, L["kpool"], L["vpool"], m.heads, m.kv_heads, m.dim, m.vdim, self.cfg.eps if m.qk_unit_norm else -1.0)
        o = ws.inner_a.view(-1)[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        seqops.attn(qkvg, st, L["kpool"], L["vpool"], m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.chunk, m.window, m.gated, o, ws.scratch)
        seqops.linear(o, L["w_o"], y)

    def _ssm(self, L, m: SsmSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        inner, gn = m.heads * m.vdim, m.groups * m.state
        n_in = 2 * inner + 2 * gn + m.heads
        proj = ws.proj[:T, :n_in]
        seqops.linear(a, L["w_in"], proj)
        xbc = ws.xbc.view(-1)[:T * (inner + 2 * gn)].view(T, inner + 2 * gn)
        seqops.causal_conv(proj[:, inner:2 * inner + 2 * gn], L["conv_w"], L["conv_b"], L["conv_state"], st, seqops.CONV_SILU, xbc)
        yg = ws.inner_f.view(-1)[:T * inner].view(T, inner)
        seqops.ssm_scan(proj, 0, 2 * inner + 2 * gn, xbc, L["A_log"], L["D"], L["dt_bias"], L["ssm_state"], st, m.heads, m.vdim, m.state, m.groups, yg, ws.scratch)
        yn = ws.inner_a.view(-1)[:T * inner].view(T, inner)
        seqops.group_rmsnorm(yg, L["mnorm"], m.norm_groups, self.cfg.eps, yn)
        seqops.linear(yn, L["w_o"], y)

    def _dense_ff(self, L, f: DenseFfSpec, ws: _Workspace, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        act = ws.inner_a.view(-1)[:T * f.ff].view(T, f.ff)
        if T <= 8 or (T >= seqops.TC_MIN_ROWS and seqops.tc_usable(a, a.shape[1])):     # projection and activation in one kernel
            seqops.linear_gated(a, L["w_gu"], f.limit, f.alpha, f.up_shift, act)
        else:
            gu = ws.proj[:T, :2 * f.ff]
            seqops.linear(a, L["w_gu"], gu)
            seqops.gated_act(gu, f.limit, f.alpha, f.up_shift, act, interleaved=True)
        seqops.linear(act, L["w_down"], y)
