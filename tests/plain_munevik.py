"""A plain, slow implementation of the Munevik design on the CPU: one function per mechanism, written from the design's
equations, sharing nothing with the engine.  Everything runs over a whole sequence at once (no cache, no state carried):
the engine's steps, pages and slots must reproduce it however a sequence is cut.  ``DT`` is float64 so that the oracle's own
rounding is far below every tolerance.

Notation: x [T, d] the stream, h a sub-layer's input, w a dict of tensors by full name, p a name prefix ending in '.'.
"""
import math

import torch

DT = torch.float64


def layer_norm(x, weight, bias, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_pairs(x, positions, base, dims):
    """Pairs (2i, 2i+1) of the last axis turned by positions * base**(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=DT)
    ang = positions.to(DT)[:, None] * base ** (-2.0 * i / dims)
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cos, sin = ang.cos(), ang.sin()
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * cos - odd * sin
    out[..., 1::2] = odd * cos + even * sin
    return out


def latent_kv(h, w, p, m, eps):
    """(latent c [T, rank], rotated shared key part [T, rot_dim]) of a layer that owns a down-projection."""
    T = h.shape[0]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :m["kv_rank"]], w[p + "dkv.norm"], eps)
    kr = rotate_pairs(down[:, m["kv_rank"]:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, p, m, kv):
    """kv = (c, kr) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    q = (h @ w[p + "q"].T).view(T, H, dn + dr)
    q_plain = q[..., :dn]
    q_rot = rotate_pairs(q[..., dn:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    keys = (c @ w[p + "uk"].T).view(T, H, dn)
    vals = (c @ w[p + "uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                               # [T, H]
    out = torch.zeros(T, H, dv, dtype=DT)
    for t in range(T):
        lo = max(0, t - m["mask"]["size"] + 1)
        for hd in range(H):
            score = (keys[lo:t + 1, hd] @ q_plain[t, hd] + kr[lo:t + 1] @ q_rot[t, hd]) * m["scale"]
            out[t, hd] = torch.softmax(score, 0) @ vals[lo:t + 1, hd]
    out = out * gate[..., None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rglru(h, w, p, m, decay=8.0):
    T, W, B, taps = h.shape[0], m["width"], m["blocks"], m["conv"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    xin = h @ w[p + "x"].T + w[p + "x.b"]
    u = torch.zeros(T, W, dtype=DT)
    for t in range(T):
        for k in range(taps):                                            # tap taps-1 is the current token's
            src = t - (taps - 1) + k
            if src >= 0:
                u[t] += w[p + "conv"][:, k] * xin[src]
        u[t] += w[p + "conv.b"]
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    a = torch.exp(-decay * r * torch.nn.functional.softplus(w[p + "lam"]))
    S = torch.zeros(W, dtype=DT)
    out = torch.empty(T, W, dtype=DT)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        out[t] = S * y[t]
    return out @ w[p + "o"].T


def clamped_glu(h, w, p, limit, alpha=1.702, shift=1.0):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + shift)) @ w[p + "down"].T


def swiglu(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(scores, groups, keep, top, group_top=2):
    """Chosen expert ids per token, by plain loops.  scores [T, E]."""
    T, E = scores.shape
    per = E // groups
    chosen = []
    for t in range(T):
        s = scores[t].tolist()
        gscore = [sum(sorted(s[g * per:(g + 1) * per], reverse=True)[:group_top]) for g in range(groups)]
        kept = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // per in kept]
        chosen.append(sorted(allowed, key=lambda e: (-s[e], e))[:top])
    return chosen


def moe(h, w, p, f):
    r = f["router"]
    scores = torch.sigmoid(h @ w[p + "router"].T)
    chosen = route(scores, r["groups"]["count"], r["groups"]["keep"], r["top"])
    out = torch.zeros_like(h)
    for t, experts in enumerate(chosen):
        for e in experts:
            out[t] += scores[t, e] * r["scale"] * swiglu(h[t:t + 1], w, f"{p}e{e}.")[0]
    if f.get("shared") is not None:
        out = out + swiglu(h, w, p + "shared.")
    return out


def forward(cfg, weights, tokens, streams=None):
    """Logits [T, vocab] of one sequence.  ``streams``: a list that receives the stream after every layer."""
    w = {k: (v.to(DT) if v.dtype.is_floating_point else v) for k, v in weights.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.tensor(list(tokens))]
    kv = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kv[i] = latent_kv(x, w, p + "mix.", m, eps)
                src = i
            mixed = latent_attention(x, w, p + "mix.", m, kv[src])
        else:
            mixed = rglru(x, w, p + "mix.", m)
        x = layer_norm(alpha * x + mixed, w[p + "norm1"], w[p + "norm1.b"], eps)
        f = L["mlp"]
        if f is not None:
            ff = clamped_glu(x, w, p + "mlp.", f["limit"]) if f["kind"] == "dense" else moe(x, w, p + "mlp.", f)
            x = layer_norm(alpha * x + ff, w[p + "norm2"], w[p + "norm2.b"], eps)
        if streams is not None:
            streams.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["embed"].T
