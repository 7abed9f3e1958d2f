"""Plain, slow restatement of the Gemosun layer types in torch (CPU, float64): one function per mechanism, position by position
where the mechanism is a mask.  Test infrastructure only: nothing here is imported by the package, and nothing of the package is
imported here.

Notation: T tokens of ONE sequence, W model width, weights as a dict name -> tensor with the checkpoint's names.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w over the last dimension; no bias"""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def rotary_frequencies(rot: dict):
    """(frequency of every pair [dims / 2], factor on cos and sin)"""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        where = lambda turns: dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq[i] = freq[i] / sc["factor"] * ramp + freq[i] * (1.0 - ramp)
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return freq, amp


def rotate(x: torch.Tensor, rot: Optional[dict], first_pos: int = 0) -> torch.Tensor:
    """x [T, heads, D]: the pairs (2i, 2i + 1) below rot.dims turn by position * frequency_i; the rest passes"""
    if not rot:
        return x
    freq, amp = rotary_frequencies(rot)
    out = x.clone()
    for t in range(x.shape[0]):
        for i, f in enumerate(freq):
            a = (first_pos + t) * f
            c, s = math.cos(a) * amp, math.sin(a) * amp
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


def window_pool_attention(q, k, v, scale: float, window: int = 0, pool: int = 0, gate=None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] of one sequence (k, v as the cache holds them).  Position i sees the positions j with
    0 <= i - j < window (window 0: all j <= i) and, when pool > 0, one mean key / mean value for every block b of `pool` positions
    with b * pool + pool - 1 <= i - window; one soft-max over both; gate [T, H]: logits of a sigmoid on each head's output"""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        first = max(0, i - window + 1) if window > 0 else 0
        blocks = []
        if pool > 0:
            b = 0
            while b * pool + pool - 1 <= i - window:
                blocks.append(b)
                b += 1
        for h in range(H):
            g = h // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [k[j, g] for j in range(first, i + 1)]
            vals = [v[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [v[j, g] for j in range(first, i + 1)]
            s = torch.stack([(q[i, h] * kk).sum() for kk in keys]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = (p[:, None] * torch.stack(vals)).sum(0)
    if gate is not None:
        out = out * torch.sigmoid(gate)[:, :, None]
    return out


def attention_mixer(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ P[pre + "q"].T).reshape(T, H, D)
    k = (h @ P[pre + "k"].T).reshape(T, G, D)
    v = k.clone()                                   # the values are the keys as projected
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    mask = m.get("mask") or {}
    o = window_pool_attention(q, k, v, m["scale"], mask.get("size", 0), mask.get("pool", 0), gate=h @ P[pre + "g"].T)
    return o.reshape(T, -1) @ P[pre + "o"].T


def dense_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    return (gelu_tanh(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def route(scores: torch.Tensor, top: int, groups: int = 1, keep: int = 1):
    """scores [E] of one token -> (chosen experts in falling order of score, their weights)"""
    E = scores.shape[0]
    allowed = list(range(E))
    if groups > 1:
        size = E // groups
        gsc = []
        for g in range(groups):
            part = sorted(scores[g * size:(g + 1) * size].tolist(), reverse=True)
            gsc.append(sum(part[:2]))
        best = sorted(range(groups), key=lambda g: (-gsc[g], g))[:keep]
        allowed = [e for e in range(E) if e // size in best]
    chosen = sorted(allowed, key=lambda e: (-scores[e].item(), e))[:top]
    w = torch.stack([scores[e] for e in chosen])
    return chosen, w / (w.sum() + 1e-20)


def moe_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ P[pre + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(s[t], r["top"], gr["count"], gr["keep"])
        for e, we in zip(chosen, w):
            out[t] += we * (relu_squared(h[t] @ P[pre + f"e{e}.up"].T) @ P[pre + f"e{e}.down"].T)
    if mlp.get("shared"):
        sh = relu_squared(h @ P[pre + "shared.up"].T) @ P[pre + "shared.down"].T
        out = out + sh * torch.sigmoid(h @ P[pre + "shared.sg"].T)
    return out


def forward(cfg: dict, P: Dict[str, torch.Tensor], tokens: List[int], layer_out: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of one sequence; layer_out receives the residual stream after every layer (after the depth average)"""
    P = {k: v.double() for k, v in P.items()}
    eps = cfg["norm"]["eps"]
    x = P["embed"][torch.tensor(tokens)]
    results = [x]
    for i, lay in enumerate(cfg["layers"]):
        pre = f"l{i}."
        y = attention_mixer(layer_norm(x, P[pre + "norm1"], eps), P, pre + "mix.", lay["mixer"])
        if lay["mlp"] is not None:
            hin = layer_norm(x, P[pre + "norm2"], eps)
            y = y + (dense_ff(hin, P, pre + "mlp.") if lay["mlp"]["kind"] == "dense" else moe_ff(hin, P, pre + "mlp.", lay["mlp"]))
        results.append(x + y)
        x = sum(P[pre + "dwa"][j] * results[j] for j in range(i + 2))
        if layer_out is not None:
            layer_out.append(x.clone())
    return layer_norm(x, P["final.norm"], eps) @ P["head"].T


def random_model(cfg: dict, seed: int = 0, router_scale: float = 2.5) -> Dict[str, torch.Tensor]:
    """random bfloat16-representable weights with the checkpoint's names and shapes.  Router rows are large so that the scores lie
    far apart (a choice never rests on a close call); depth weights put most of the mass on the newest result."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).bfloat16().float()
    P = {"embed": r(cfg["vocab"], W, sc=1.0), "head": r(cfg["vocab"], W, sc=W ** -0.5), "final.norm": 1 + r(W, sc=0.1)}
    for i, lay in enumerate(cfg["layers"]):
        m = lay["mixer"]
        pre = f"l{i}."
        P[pre + "norm1"] = 1 + r(W, sc=0.1)
        P[pre + "mix.q"] = r(m["heads"] * m["dim"], W, sc=2.0 * W ** -0.5)
        P[pre + "mix.k"] = r(m["kv_heads"] * m["dim"], W, sc=2.0 * W ** -0.5)
        P[pre + "mix.g"] = r(m["heads"], W, sc=W ** -0.5)
        P[pre + "mix.o"] = r(W, m["heads"] * m["vdim"], sc=(m["heads"] * m["vdim"]) ** -0.5)
        mlp = lay["mlp"]
        if mlp is not None:
            P[pre + "norm2"] = 1 + r(W, sc=0.1)
            if mlp["kind"] == "dense":
                P[pre + "mlp.gate"], P[pre + "mlp.up"] = r(mlp["ff"], W, sc=W ** -0.5), r(mlp["ff"], W, sc=W ** -0.5)
                P[pre + "mlp.down"] = r(W, mlp["ff"], sc=mlp["ff"] ** -0.5)
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                P[pre + "mlp.router"] = r(E, W, sc=router_scale * W ** -0.5)
                for e in range(E):
                    P[pre + f"mlp.e{e}.up"] = r(ff, W, sc=W ** -0.5)
                    P[pre + f"mlp.e{e}.down"] = r(W, ff, sc=ff ** -0.5)
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    P[pre + "mlp.shared.up"], P[pre + "mlp.shared.down"] = r(sf, W, sc=W ** -0.5), r(W, sf, sc=sf ** -0.5)
                    P[pre + "mlp.shared.sg"] = r(1, W, sc=W ** -0.5)
        d = r(i + 2, sc=0.15)
        d[i + 1] += 1.0
        P[pre + "dwa"] = d
    return {k: v.bfloat16().float() for k, v in P.items()}      # the checkpoint holds bfloat16: what is not representable is rounded here


def write_checkpoint(folder: str, cfg: dict, P: Dict[str, torch.Tensor]) -> None:
    """config.json + model.safetensors (bfloat16), written with the file format's own rules"""
    import json
    import os
    import struct

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    head, blobs, off = {}, [], 0
    for k, v in P.items():
        b = v.bfloat16().contiguous().view(torch.uint8).numpy().tobytes()
        head[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
