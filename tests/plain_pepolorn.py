"""A plain, slow implementation of the Pepolorn design, one function per mechanism, in torch on the CPU.

It shares no code with the engine: it takes a configuration (the nested dict of ``config.json``) and a dict of
tensors by name and walks whole sequences token by token where a recurrence is involved.  Everything runs in
the type of the tensors it is given (tests pass float64 or float32).

Notation: W the width, T the tokens of one sequence, positions count from 0.
    rms(v)        = v / sqrt(mean(v^2) + eps)
    block         x += (1 + w1) * rms(mixer(x));  x += (1 + w2) * rms(ff(x))      (the parts read x itself)
    output        logits = E ((1 + wf) * rms(x)),  E the embedding table
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def offset_norm(v, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms(v, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ------------------------------------------------------------------------------------------ rotation --
def rotary_frequencies(rot: Mapping) -> tuple:
    """(frequencies [dims/2] float64, factor on cos and sin) of a rotation with optional YaRN scaling."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(v: torch.Tensor, positions: torch.Tensor, rot: Mapping) -> torch.Tensor:
    """v [T, heads, dim]; the first rot.dims elements of every head turn, pairs (i, i + dims/2)."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * m).to(v.dtype)[:, None, :], (torch.sin(ang) * m).to(v.dtype)[:, None, :]
    a, b = v[..., : dims // 2], v[..., dims // 2: dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------------------ mixers --
def chunked_attention(h, w: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    """Softmax attention inside chunks of mask.size positions; q and k unit-normed per head after the rotation."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = (h @ w[p + ".q"].T).view(T, H, d)
    k = (h @ w[p + ".k"].T).view(T, G, d)
    v = (h @ w[p + ".v"].T).view(T, G, dv)
    q, k = rms(rotate(q, pos, m["rot"]), eps), rms(rotate(k, pos, m["rot"]), eps)
    size = int(m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        j0 = (i // size) * size
        for hh in range(H):
            g = hh // (H // G)
            sc = (k[j0: i + 1, g] @ q[i, hh]) * float(m["scale"])
            pr = torch.softmax(sc, dim=0)
            out[i, hh] = pr @ v[j0: i + 1, g]
    return out.reshape(T, H * dv) @ w[p + ".o"].T


def lightning_attention(h, w, p: str, m: Mapping, eps: float, state: Optional[torch.Tensor] = None):
    """Linear attention with a constant decay per head: S = decay * S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[p + ".q"].T).view(T, H, d)
    k = silu(h @ w[p + ".k"].T).view(T, H, d)
    v = silu(h @ w[p + ".v"].T).view(T, H, dv)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms(o.reshape(T, H * dv), eps) * w[p + ".norm"] * torch.sigmoid(h @ w[p + ".g"].T)
    return y @ w[p + ".o"].T, S


def parallel_mixer(h, w, p: str, m: Mapping, eps: float):
    left = chunked_attention(h, w, p + ".left", m["left"], eps)
    right, _ = lightning_attention(h, w, p + ".right", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mamba2_mixer(h, w, p: str, m: Mapping, eps: float):
    T = h.shape[0]
    H, dv, N, G, taps = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"])
    inner = H * dv
    u = h @ w[p + ".in"].T
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    cw, cb = w[p + ".conv"], w[p + ".conv.b"]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], dim=0)
    conv = cb[None, :].expand(T, -1).clone()
    for j in range(taps):
        conv = conv + padded[j: j + T] * cw[:, j][None, :]
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, dv)
    B = conv[:, inner: inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + ".dt_bias"])
    rate = torch.exp(w[p + ".A_log"])
    S = torch.zeros(H, N, dv, dtype=h.dtype)
    y = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = torch.exp(-rate[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * B[t, g][:, None] * x[t, hh][None, :]
            y[t, hh] = S[hh].T @ C[t, g] + w[p + ".D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + ".norm"]
    return y @ w[p + ".o"].T


# ------------------------------------------------------------------------------------------ feed-forward --
def dense_ff(h, w, p: str):
    return (gelu_tanh(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


def route(h, w, p: str, r: Mapping):
    """(expert ids [T, top], weights [T, top]): sigmoid scores; the choice uses score + correction and is limited
    to the best groups (a group scored by its two largest choice scores); the weights are the plain scores."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {}
    count = int(groups.get("count", 1))
    keep = int(groups.get("keep", count))
    s = torch.sigmoid(h @ w[p + ".router"].T)
    choice = s + w[p + ".correction"]
    T = h.shape[0]
    per = E // count
    gs = choice.view(T, count, per).topk(min(2, per), dim=-1).values.sum(-1)
    open_groups = gs.topk(keep, dim=-1).indices
    mask = torch.zeros(T, count, dtype=torch.bool)
    mask.scatter_(1, open_groups, True)
    masked = torch.where(mask[:, :, None].expand(T, count, per).reshape(T, E), choice,
                         torch.full_like(choice, -float("inf")))
    ids = masked.topk(top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def moe_ff(h, w, p: str, ml: Mapping):
    ids, wts = route(h, w, p, ml["router"])
    out = torch.zeros(h.shape[0], w[p + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            q = f"{p}.e{e}"
            out[t] += a * ((silu(w[q + ".gate"] @ h[t]) * (w[q + ".up"] @ h[t])) @ w[q + ".down"].T)
    return out


# ------------------------------------------------------------------------------------------ model --
def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{L['weights_of']}" if L.get("weights_of") is not None else f"l{i}"
        if L["type"] == "parallel":
            a = parallel_mixer(x, w, p + ".mix", L["mixer"], eps)
        elif L["type"] == "mamba2":
            a = mamba2_mixer(x, w, p + ".mix", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + offset_norm(a, w[p + ".norm1"], eps)
        ml = L.get("mlp")
        if ml is not None:
            f = dense_ff(x, w, p + ".mlp") if ml["kind"] == "dense" else moe_ff(x, w, p + ".mlp", ml)
            x = x + offset_norm(f, w[p + ".norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["embed"].T


# ------------------------------------------------------------------------------------------ random weights --
def random_weights(cfg: Mapping, seed: int) -> Dict[str, torch.Tensor]:
    """Tensors of a model of ``cfg`` (float64, values that bfloat16 holds exactly), by name."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float64) * std + mean).to(torch.bfloat16).double()

    def lin(out, inp, gain=1.0):
        return rnd(out, inp, std=gain / math.sqrt(inp))
    w = {"embed": rnd(int(cfg["vocab"]), W), "final.norm": rnd(W, std=0.1)}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}", L["mixer"]
        w[p + ".norm1"] = rnd(W, std=0.1)
        if L["type"] == "mamba2":
            H, dv, N, G, taps = (int(m[k]) for k in ("heads", "vdim", "state", "groups", "conv"))
            inner, C = H * dv, H * dv + 2 * G * N
            w[p + ".mix.in"] = lin(2 * inner + 2 * G * N + H, W, 1.5)
            w[p + ".mix.conv"] = rnd(C, taps, std=0.5)
            w[p + ".mix.conv.b"] = rnd(C, std=0.2)
            w[p + ".mix.dt_bias"] = rnd(H, std=0.7)
            w[p + ".mix.A_log"] = rnd(H, std=0.6, mean=-0.5)
            w[p + ".mix.D"] = rnd(H, std=0.3, mean=1.0)
            w[p + ".mix.norm"] = rnd(inner, std=0.2, mean=1.0)
            w[p + ".mix.o"] = lin(W, inner)
        else:
            a, b = m["left"], m["right"]
            w[p + ".mix.left.q"] = lin(int(a["heads"]) * int(a["dim"]), W)
            w[p + ".mix.left.k"] = lin(int(a["kv_heads"]) * int(a["dim"]), W)
            w[p + ".mix.left.v"] = lin(int(a["kv_heads"]) * int(a["vdim"]), W)
            w[p + ".mix.left.o"] = lin(W, int(a["heads"]) * int(a["vdim"]))
            kq, kv = int(b["heads"]) * int(b["dim"]), int(b["heads"]) * int(b["vdim"])
            w[p + ".mix.right.q"], w[p + ".mix.right.k"] = lin(kq, W), lin(kq, W)
            w[p + ".mix.right.v"], w[p + ".mix.right.g"] = lin(kv, W), lin(kv, W)
            w[p + ".mix.right.norm"] = rnd(kv, std=0.2, mean=1.0)
            w[p + ".mix.right.o"] = lin(W, kv)
        ml = L.get("mlp")
        if ml is None:
            continue
        w[p + ".norm2"] = rnd(W, std=0.1)
        if ml["kind"] == "dense":
            F = int(ml["ff"])
            w[p + ".mlp.gate"], w[p + ".mlp.up"], w[p + ".mlp.down"] = lin(F, W), lin(F, W), lin(W, F)
        else:
            E, F = int(ml["router"]["experts"]), int(ml["expert"]["ff"])
            w[p + ".mlp.router"] = lin(E, W, 3.0)
            w[p + ".mlp.correction"] = rnd(E, std=0.4, mean=-0.2)
            for e in range(E):
                q = f"{p}.mlp.e{e}"
                w[q + ".gate"], w[q + ".up"], w[q + ".down"] = lin(F, W), lin(F, W), lin(W, F)
    return w
