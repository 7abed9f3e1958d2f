"""Plain, slow restatement of the Fenorax layer types in torch (CPU, float64 by default): one function per mechanism,
token by token where the mechanism is a recurrence.  Test infrastructure only: nothing here is imported by the package,
and nothing of the package is imported here.

Notation: T tokens of ONE sequence, W model width, weights as a dict name -> tensor with the checkpoint's names.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def group_rms(x: torch.Tensor, groups: int, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [..., D] split into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times w"""
    shp = x.shape
    p = x.reshape(*shp[:-1], groups, shp[-1] // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    y = p.reshape(shp)
    return y * w if w is not None else y


def causal_conv(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j) (+ bias), zeros before the start"""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    if bias is not None:
        out = out + bias
    return out


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def ssm_recurrence(x, B, Cm, dt_raw, dt_bias, A_log, D, S0=None, return_state=False):
    """x [T, H, V], B and Cm [T, G, N], dt_raw [T, H]: S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T;  y_t = S_t^T C_t + D x_t"""
    T, H, V = x.shape
    G, N = B.shape[1], B.shape[2]
    dt = softplus(dt_raw + dt_bias)
    A = torch.exp(A_log)
    S = torch.zeros(H, N, V, dtype=x.dtype) if S0 is None else S0.clone()
    y = torch.zeros(T, H, V, dtype=x.dtype)
    per = H // G
    for t in range(T):
        for hh in range(H):
            g = hh // per
            S[hh] = torch.exp(-A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ Cm[t, g] + D[hh] * x[t, hh]
    return (y, S) if return_state else y


def masked_attention(q, k, v, scale, chunk=0, window=0, gate=None):
    """q [T, H, D], k [T, G, D], v [T, G, V]; query i sees key j <= i of its own chunk (chunk > 0) and with i - j < window (window > 0)"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    per = H // G
    for i in range(T):
        lo = (i // chunk) * chunk if chunk > 0 else 0
        if window > 0:
            lo = max(lo, i - window + 1)
        for hh in range(H):
            g = hh // per
            p = torch.softmax((k[lo:i + 1, g] @ q[i, hh]) * scale, 0)
            out[i, hh] = (p[:, None] * v[lo:i + 1, g]).sum(0)
            if gate is not None:
                out[i, hh] = out[i, hh] * gate[i, hh]
    return out


def mamba2(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    """state-space mixer; m: heads, vdim, state, groups, norm_groups, conv"""
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ P[pre + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P[pre + "conv"], P[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    y = ssm_recurrence(x, B, Cm, dt, P[pre + "dt_bias"], P[pre + "A_log"], P[pre + "D"])
    y = y.reshape(T, inner) * silu(z)
    y = group_rms(y, m["norm_groups"], eps, P[pre + "norm"])
    return y @ P[pre + "o"].T


def chunk_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, m: dict, eps: float) -> torch.Tensor:
    """softmax attention without rotation, unit-RMS q and k, keys of the query's own chunk only, one sigmoid gate per head"""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    cs = m["mask"]["size"]
    q = group_rms((h @ P[pre + "q"].T).reshape(T, H, D), 1, eps)
    k = group_rms((h @ P[pre + "k"].T).reshape(T, G, D), 1, eps)
    v = (h @ P[pre + "v"].T).reshape(T, G, V)
    gate = torch.sigmoid(h @ P[pre + "g"].T)             # [T, H]
    out = masked_attention(q, k, v, m["scale"], chunk=cs, gate=gate)
    return out.reshape(T, H * V) @ P[pre + "o"].T


def dense_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], pre: str, m: dict) -> torch.Tensor:
    lim = m["limit"]
    g = torch.clamp(h @ P[pre + "gate"].T, max=lim)
    u = torch.clamp(h @ P[pre + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ P[pre + "down"].T


def forward(cfg: dict, P: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layer_sums: Optional[list] = None) -> torch.Tensor:
    """logits [T, vocab] of one whole sequence"""
    P = {k: v.to(dtype) for k, v in P.items()}
    eps, ng = cfg["norm"]["eps"], cfg["norm"]["groups"]
    S = cfg["streams"]
    x0 = P["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    X = [x0.clone() for _ in range(S)]
    for i, lay in enumerate(cfg["layers"]):
        subs = [1] if lay["mlp"] is None else [1, 2]
        for q in subs:
            hc = f"l{i}.hc{q}."
            u = sum(P[hc + "in"][s] * X[s] for s in range(S))
            h = group_rms(u, ng, eps, P[f"l{i}.norm{q}"])
            h = h + causal_conv(h, P[f"l{i}.canon{q}"])
            if q == 1:
                if lay["type"] == "mamba2":
                    y = mamba2(h, P, f"l{i}.mix.", lay["mixer"], eps)
                elif lay["type"] == "attention":
                    y = chunk_attention(h, P, f"l{i}.mix.", lay["mixer"], eps)
                else:
                    raise ValueError(lay["type"])
            else:
                y = dense_ff(h, P, f"l{i}.mlp.", lay["mlp"])
            X = [sum(P[hc + "mix"][s, t] * X[s] for s in range(S)) + P[hc + "out"][t] * y for t in range(S)]
        if layer_sums is not None:
            layer_sums.append(sum(X))
    x = group_rms(sum(X), ng, eps, P["final.norm"])
    return x @ P["embed"].T


def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """random bfloat16-representable weights with the checkpoint's names and shapes"""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).bfloat16().float()
    P = {"embed": r(cfg["vocab"], W, sc=0.5), "final.norm": 1 + r(W, sc=0.1)}
    S, taps = cfg["streams"], cfg["canon"]["taps"]
    for i, lay in enumerate(cfg["layers"]):
        m = lay["mixer"]
        for q in ([1] if lay["mlp"] is None else [1, 2]):
            P[f"l{i}.norm{q}"] = 1 + r(W, sc=0.1)
            P[f"l{i}.canon{q}"] = r(W, taps, sc=0.3)
            P[f"l{i}.hc{q}.in"] = (torch.full((S,), 1.0 / S) + r(S, sc=0.2)).bfloat16().float()
            P[f"l{i}.hc{q}.out"] = (torch.ones(S) + r(S, sc=0.2)).bfloat16().float()
            P[f"l{i}.hc{q}.mix"] = (torch.eye(S) + r(S, S, sc=0.1)).bfloat16().float()
        pre = f"l{i}.mix."
        if lay["type"] == "mamba2":
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            P[pre + "in"] = r(2 * inner + 2 * GN + m["heads"], W, sc=W ** -0.5)
            P[pre + "conv"] = r(inner + 2 * GN, m["conv"], sc=0.5)
            P[pre + "conv.b"] = r(inner + 2 * GN, sc=0.1)
            P[pre + "dt_bias"] = r(m["heads"], sc=1.0)
            P[pre + "A_log"] = r(m["heads"], sc=0.7)
            P[pre + "D"] = r(m["heads"])
            P[pre + "norm"] = 1 + r(inner, sc=0.1)
            P[pre + "o"] = r(W, inner, sc=inner ** -0.5)
        else:
            P[pre + "q"] = r(m["heads"] * m["dim"], W, sc=W ** -0.5)
            P[pre + "k"] = r(m["kv_heads"] * m["dim"], W, sc=W ** -0.5)
            P[pre + "v"] = r(m["kv_heads"] * m["vdim"], W, sc=W ** -0.5)
            P[pre + "g"] = r(m["heads"], W, sc=W ** -0.5)
            P[pre + "o"] = r(W, m["heads"] * m["vdim"], sc=(m["heads"] * m["vdim"]) ** -0.5)
        if lay["mlp"] is not None:
            ff = lay["mlp"]["ff"]
            P[f"l{i}.mlp.gate"] = r(ff, W, sc=W ** -0.5)
            P[f"l{i}.mlp.up"] = r(ff, W, sc=W ** -0.5)
            P[f"l{i}.mlp.down"] = r(W, ff, sc=ff ** -0.5)
    return {k: v.bfloat16().float() for k, v in P.items()}


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
