"""A plain, slow implementation of the Kolorax design, one function per mechanism.

Whole sequences, one token after the other where a mechanism is recurrent, in the
precision of the tensors it is given (the tests use float64).  Nothing here is
shared with the package: it is what the package's kernels are held against.

Notation.  W: model width.  A layer is  x += m * mixer(LN1(x));  x += m * ff(LN2(x)).
Mixers: ``wkv`` (a matrix-valued recurrent state per head with a per-channel,
data-dependent decay) and ``latent_attention`` (keys and values are re-made from a
small cached latent vector plus one rotated key part shared by the heads).
Feed-forward: routed experts, chosen within the best groups, plus a shared expert.
A range of layers may run several times with the same weights; each pass starts
from a mix of the stream and the embedding output.
"""
import math

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_half(x, positions, base, dims=None):
    """x [T, n]; the first r = dims (default n) elements turn, pairs (i, i + r/2), angle = position * base^(-2i/r);
    the rest pass unchanged."""
    if dims is not None and dims < x.shape[-1]:
        return torch.cat([rotate_half(x[..., :dims], positions, base), x[..., dims:]], dim=-1)
    r = x.shape[-1]
    half = r // 2
    f = torch.tensor([base ** (-2.0 * i / r) for i in range(half)], dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * torch.cos(a) - v * torch.sin(a), v * torch.cos(a) + u * torch.sin(a)], dim=-1)


# ------------------------------------------------------------------ wkv mixer --
def wkv_mixer(h, w, p, heads, dim, eps, state=None):
    """h [T, W].  state: None (a sequence's start) or (previous h [W], S [heads, dim, dim]).
    Returns (out [T, W], state)."""
    T, W = h.shape
    prev, S = (torch.zeros(W, dtype=h.dtype), torch.zeros(heads, dim, dim, dtype=h.dtype)) if state is None else state
    S = S.clone()
    out = []
    u = w[f"{p}.u"]
    for t in range(T):
        x = h[t]
        mix = {s: x + (prev - x) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
        r = (w[f"{p}.r"] @ mix["r"]).view(heads, dim)
        k = (w[f"{p}.k"] @ mix["k"]).view(heads, dim)
        v = (w[f"{p}.v"] @ mix["v"]).view(heads, dim)
        g = w[f"{p}.g"] @ mix["g"]
        gate = g * torch.sigmoid(g)
        dec = torch.exp(-torch.exp(w[f"{p}.w2"] @ torch.tanh(w[f"{p}.w1"] @ mix["w"]) + w[f"{p}.w0"])).view(heads, dim)
        o = torch.empty(heads, dim, dtype=h.dtype)
        for hh in range(heads):
            kv = torch.outer(k[hh], v[hh])                      # [key channel, value channel]
            o[hh] = (S[hh] + u[hh][:, None] * kv).T @ r[hh]
            S[hh] = dec[hh][:, None] * S[hh] + kv
        o = rms_unit(o, eps).reshape(-1) * w[f"{p}.norm"] * gate
        out.append(w[f"{p}.o"] @ o)
        prev = x
    return torch.stack(out), (prev, S)


# ------------------------------------------------------- latent attention mixer --
def latent_attention_mixer(h, w, p, positions, *, heads, dim, rot_dim, vdim, kv_rank, scale, base, eps, cached=None,
                           rot_dims=None):
    """h [T, W] at ``positions``.  cached: None or (c [n, kv_rank], k_rot [n, rot_dim]) of earlier tokens.
    Returns (out [T, W], (c, k_rot) of all tokens so far)."""
    T = h.shape[0]
    q = (h @ w[f"{p}.q"].T).view(T, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    q_rot = torch.stack([rotate_half(q_rot[:, hh], positions, base, rot_dims) for hh in range(heads)], dim=1)
    dkv = h @ w[f"{p}.dkv"].T
    c = rms_unit(dkv[:, :kv_rank], eps) * w[f"{p}.dkv.norm"]
    k_rot = rotate_half(dkv[:, kv_rank:], positions, base, rot_dims)
    if cached is not None:
        c = torch.cat([cached[0], c])
        k_rot = torch.cat([cached[1], k_rot])
    n = c.shape[0]
    k_plain = (c @ w[f"{p}.uk"].T).view(n, heads, dim)
    val = (c @ w[f"{p}.uv"].T).view(n, heads, vdim)
    out = torch.empty(T, heads, vdim, dtype=h.dtype)
    for t in range(T):
        vis = n - T + t + 1                                   # keys 0 .. own place
        for hh in range(heads):
            s = (k_plain[:vis, hh] @ q_plain[t, hh] + k_rot[:vis] @ q_rot[t, hh]) * scale
            out[t, hh] = torch.softmax(s, dim=0) @ val[:vis, hh]
    gate = torch.sigmoid(h @ w[f"{p}.g"].T)
    return (out.reshape(T, -1) * gate) @ w[f"{p}.o"].T, (c, k_rot)


# ------------------------------------------------------------- feed-forward --
def expert(x, w, p, limit):
    g = torch.clamp(x @ w[f"{p}.gate"].T, max=limit)
    u = torch.clamp(x @ w[f"{p}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[f"{p}.down"].T


def route(z, top, group_count, group_keep):
    """z [E] router logits.  Returns (chosen experts, weights)."""
    s = torch.softmax(z, dim=0)
    E = s.shape[0]
    per = E // group_count
    gscore = s.view(group_count, per).max(dim=1).values
    keep = torch.topk(gscore, group_keep).indices.tolist()
    allowed = torch.full((E,), float("-inf"), dtype=s.dtype)
    for g in keep:
        allowed[g * per:(g + 1) * per] = s[g * per:(g + 1) * per]
    chosen = torch.topk(allowed, top).indices
    wts = s[chosen] / (s[chosen].sum() + 1e-20)
    return chosen.tolist(), wts


def moe(x, w, p, cfg):
    """x [T, W]; cfg: the layer's 'mlp' entry."""
    r = cfg["router"]
    out = torch.zeros_like(x)
    z = x @ w[f"{p}.router"].T
    for t in range(x.shape[0]):
        chosen, wts = route(z[t], r["top"], r["groups"]["count"], r["groups"]["keep"])
        for e, a in zip(chosen, wts):
            out[t] += a * expert(x[t:t + 1], w, f"{p}.e{e}", cfg["expert"]["limit"])[0]
    if cfg.get("shared") is not None:
        out = out + expert(x, w, f"{p}.shared", cfg["shared"]["limit"])
    return out


# ------------------------------------------------------------------ the model --
def layer_runs(cfg):
    """[(layer, pass number or None at a run that does not open a pass)] in the order they run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    runs += [(i, None) for i in range(loop["stop"], n)]
    return runs


def forward(cfg, w, tokens, *, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer run)."""
    dt = w["embed"].dtype
    eps = cfg["norm"]["eps"]
    m = cfg["residual_mult"]
    T = len(tokens)
    pos = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    x0 = x.clone()
    after = []
    for i, opens in layer_runs(cfg):
        L = cfg["layers"][i]
        p = f"l{i}"
        if opens is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][opens]
        hn = layer_norm(x, w[f"{p}.norm1"], w[f"{p}.norm1.b"], eps)
        mx = L["mixer"]
        if L["type"] == "wkv":
            a, _ = wkv_mixer(hn, w, f"{p}.mix", mx["heads"], mx["dim"], eps)
        elif L["type"] == "latent_attention":
            a, _ = latent_attention_mixer(hn, w, f"{p}.mix", pos, heads=mx["heads"], dim=mx["dim"], rot_dim=mx["rot_dim"],
                                          vdim=mx["vdim"], kv_rank=mx["kv_rank"], scale=mx["scale"],
                                          base=mx["rot"]["base"], eps=eps, rot_dims=mx["rot"].get("dims"))
        else:
            raise ValueError(L["type"])
        x = x + m * a
        if L.get("mlp") is not None:
            hn = layer_norm(x, w[f"{p}.norm2"], w[f"{p}.norm2.b"], eps)
            x = x + m * moe(hn, w, f"{p}.mlp", L["mlp"])
        after.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


# ------------------------------------------------------- small random models --
def tensor_shapes(cfg, decay_rank=8):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "final.norm.b": (W,), "head": (cfg["vocab"], W)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}", L["mixer"]
        out[f"{p}.norm1"] = out[f"{p}.norm1.b"] = (W,)
        if L["type"] == "wkv":
            hd = mx["heads"] * mx["dim"]
            for s in "rkvgw":
                out[f"{p}.mix.mu.{s}"] = (W,)
            for s in "rkvg":
                out[f"{p}.mix.{s}"] = (hd, W)
            rank = mx.get("decay_rank", decay_rank)
            out[f"{p}.mix.w1"], out[f"{p}.mix.w2"], out[f"{p}.mix.w0"] = (rank, W), (hd, rank), (hd,)
            out[f"{p}.mix.u"], out[f"{p}.mix.norm"], out[f"{p}.mix.o"] = (mx["heads"], mx["dim"]), (hd,), (W, hd)
        else:
            H = mx["heads"]
            out[f"{p}.mix.q"] = (H * (mx["dim"] + mx["rot_dim"]), W)
            out[f"{p}.mix.dkv"] = (mx["kv_rank"] + mx["rot_dim"], W)
            out[f"{p}.mix.dkv.norm"] = (mx["kv_rank"],)
            out[f"{p}.mix.uk"] = (H * mx["dim"], mx["kv_rank"])
            out[f"{p}.mix.uv"] = (H * mx["vdim"], mx["kv_rank"])
            out[f"{p}.mix.g"] = (H * mx["vdim"], W)
            out[f"{p}.mix.o"] = (W, H * mx["vdim"])
        ml = L.get("mlp")
        if ml is not None:
            out[f"{p}.norm2"] = out[f"{p}.norm2.b"] = (W,)
            out[f"{p}.mlp.router"] = (ml["router"]["experts"], W)
            names = [(f"e{e}", ml["expert"]["ff"]) for e in range(ml["router"]["experts"])]
            if ml.get("shared") is not None:
                names.append(("shared", ml["shared"]["ff"]))
            for nm, ff in names:
                out[f"{p}.mlp.{nm}.gate"] = out[f"{p}.mlp.{nm}.up"] = (ff, W)
                out[f"{p}.mlp.{nm}.down"] = (W, ff)
    return out


def random_weights(cfg, seed, decay_rank=8, dtype=torch.bfloat16):
    """Seeded weights, rounded once to ``dtype`` and returned in float64.  Matrices are scaled by
    1/sqrt(fan-in) so that activations keep their size; decays spread over (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf not in ("u", "step"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if leaf == "embed":
                t = t * math.sqrt(shape[1])
            if leaf == "router":
                t = t * 3.0
        elif name.endswith(".b"):
            t = torch.randn(shape, generator=g) * 0.1
        elif leaf == "w0":
            t = torch.randn(shape, generator=g) * 1.5 - 1.0
        elif leaf in ("u", "step"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf in "rkvgw" and ".mu." in name:
            t = torch.rand(shape, generator=g)
        else:                                   # norm weights
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        w[name] = t.to(dtype).double()
    return w
