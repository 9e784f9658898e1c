"""A plain, slow implementation of the Mizupel design in float64: whole sequences, no cache, no state carried between calls,
one function per mechanism.  It shares no code with the engine; the tests compare the engine with it.

Notation: ``x`` [S, width] is a sequence's residual stream, ``h`` a sub-layer's normed input, ``W[name]`` a tensor of the
model folder (matrices are stored [out, in] and applied as ``h @ W.T``), ``m`` a layer's ``mixer`` object of config.json.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------------------ attention
def short_conv(u, w):
    """u [S, C], w [C, taps]: y[t] = sum_j w[:, j] * u[t - taps + 1 + j], zeros before the sequence."""
    S, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(S):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


def rotary_frequencies(rot):
    dims = rot["dims"]
    freqs = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            wavelength = 2.0 * math.pi / f
            if wavelength > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wavelength >= sc["original"] / sc["high"]:
                s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        freqs.append(f)
    return freqs


def rotate(x, rot, first_position=0):
    """x [S, heads, D]: the first rot.dims values of every head, value i paired with value i + dims/2."""
    if not rot or not rot["dims"]:
        return x
    out = x.clone()
    half = rot["dims"] // 2
    for i, f in enumerate(rotary_frequencies(rot)):
        for t in range(x.shape[0]):
            a = (first_position + t) * f
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * math.cos(a) - v * math.sin(a)
            out[t, :, i + half] = v * math.cos(a) + u * math.sin(a)
    return out


def attention(h, W, p, m):
    S = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads", H), m.get("vdim", D)
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    v = h @ W[p + "v"].T + W[p + "v.b"]
    if m.get("conv") is not None:
        q, k, v = short_conv(q, W[p + "q.conv"]), short_conv(k, W[p + "k.conv"]), short_conv(v, W[p + "v.conv"])
    q = rotate(q.view(S, H, D), m.get("rot"))
    k = rotate(k.view(S, G, D), m.get("rot"))
    v = v.view(S, G, Dv)
    window = m["mask"]["size"] if m.get("mask") else None
    gate = torch.sigmoid(h @ W[p + "g"].T)                            # [S, H]
    out = torch.zeros(S, H, Dv, dtype=F64)
    for head in range(H):
        kv_head = head // (H // G)
        for i in range(S):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, kv_head] @ q[i, head]) * m["scale"]
            if m.get("softcap"):
                s = m["softcap"] * torch.tanh(s / m["softcap"])
            out[i, head] = torch.softmax(s, 0) @ v[lo:i + 1, kv_head]
    return (out * gate[:, :, None]).reshape(S, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ time mixing with a matrix state
def wkv(h, W, p, m, eps):
    S, d = h.shape
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, d, dtype=F64), h[:-1]])
    mix = {s: h + (before - h) * W[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[p + "r"].T).view(S, H, D)
    k = (mix["k"] @ W[p + "k"].T).view(S, H, D)
    v = (mix["v"] @ W[p + "v"].T).view(S, H, D)
    gate = torch.nn.functional.silu(mix["g"] @ W[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(S, H, D)
    u = W[p + "u"].reshape(H, D)
    out = torch.zeros(S, H, D, dtype=F64)
    for head in range(H):
        state = torch.zeros(D, D, dtype=F64)                          # [key channel, value channel]
        for t in range(S):
            kv = torch.outer(k[t, head], v[t, head])
            out[t, head] = (state + u[head][:, None] * kv).T @ r[t, head]
            state = decay[t, head][:, None] * state + kv
    out = rms_norm(out, eps).reshape(S, H * D) * W[p + "norm"] * gate
    return out @ W[p + "o"].T


def mlstm(h, W, p, m, eps):
    S = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[p + "q"].T).view(S, H, D) / math.sqrt(D)
    k = (h @ W[p + "k"].T).view(S, H, D)
    v = (h @ W[p + "v"].T).view(S, H, Dv)
    log_i = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    out = torch.zeros(S, H, Dv, dtype=F64)
    for head in range(H):
        C, n, mx = torch.zeros(D, Dv, dtype=F64), torch.zeros(D, dtype=F64), 0.0
        for t in range(S):
            new_mx = max(log_f[t, head].item() + mx, log_i[t, head].item())
            keep, take = math.exp(log_f[t, head].item() + mx - new_mx), math.exp(log_i[t, head].item() - new_mx)
            C = keep * C + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            mx = new_mx
            out[t, head] = (C.T @ q[t, head]) / (max(abs((n @ q[t, head]).item()), math.exp(-mx)) + 1e-6)
    out = rms_norm(out, eps).reshape(S, H * Dv) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forward, model
def relu2_mlp(h, W, p):
    return torch.relu(h @ W[p + "up"].T) ** 2 @ W[p + "down"].T


def mixer(kind, h, W, p, m, eps):
    if kind == "attention":
        return attention(h, W, p, m)
    return wkv(h, W, p, m, eps) if kind == "wkv" else mlstm(h, W, p, m, eps)


def forward(cfg, W, tokens, stream_after=None):
    """Logits [S, vocab] of one sequence; ``stream_after`` (a list) receives the stream after every layer entry."""
    W = {k: (v.to(F64) if v.dtype.is_floating_point else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        owner = L.get("weights_of")
        p = f"l{i if owner is None else owner}."
        x = x + mixer(L["type"], rms_norm(x, eps) * W[p + "norm1"], W, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            x = x + relu2_mlp(rms_norm(x, eps) * W[p + "norm2"], W, p + "mlp.")
        if stream_after is not None:
            stream_after.append(x.clone())
    logits = (rms_norm(x, eps) * W["final.norm"]) @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
