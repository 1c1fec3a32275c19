"""The Tuganex design written out plainly: float64, token by token, one function per mechanism.

Nothing here is shared with ``pih_b200``: the tests compare the engine with these functions.  A model is a dict
``config`` (the keys of config.json) and a dict ``w`` of float64 tensors by name.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rotate(x, positions, dims, base):
    """Rotate-half over the first ``dims`` columns of the last axis; x [T, ..., d], positions [T]."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def softplus(z):
    return math.log1p(math.exp(z)) if z < 30 else z


def xielu(z, p, q):
    ap, aq = softplus(float(p)), 0.5 + softplus(float(q))
    pos = ap * z * z + 0.5 * z
    neg = aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def silu(z):
    return z * torch.sigmoid(z)


def retention(h, m, w, pre, eps, S0=None, start=0):
    """One sequence: h [T, width] -> ([T, width], final state [heads, dim, vdim])."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    q = (h @ w[pre + "q"].T).reshape(T, H, d)
    k = (h @ w[pre + "k"].T).reshape(T, H, d)
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    q = rotate(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate(k, pos, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    S = torch.zeros(H, d, dv, dtype=F) if S0 is None else S0.clone()
    decay = torch.tensor(m["decay"], dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, S


def attention_keys_values(h, m, w, pre, eps, start=0):
    """Keys after norm and rotation [T, G, 2, dim] and values [T, G, vdim] of one sequence's rows."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    k = (h @ w[pre + "k"].T).reshape(T, G, 2, d)
    k = rotate(rms_unit(k, eps) * w[pre + "k.norm"], pos, m["rot"]["dims"], m["rot"]["base"])
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    return k, v


def differential_lambda(m, w, pre):
    return (math.exp(float((w[pre + "lq1"] * w[pre + "lk1"]).sum())) - math.exp(float((w[pre + "lq2"] * w[pre + "lk2"]).sum()))
            + m["diff"])


def differential_attention(h, m, w, pre, eps, keys, values, start=0):
    """h [T, width]: the rows at positions start..; keys / values: ALL of the sequence's up to the last row."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    q = (h @ w[pre + "q"].T).reshape(T, H, 2, d)
    q = rotate(rms_unit(q, eps) * w[pre + "q.norm"], pos, m["rot"]["dims"], m["rot"]["base"])
    lam = differential_lambda(m, w, pre)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        n = start + t + 1
        for hd in range(H):
            g = hd // (H // G)
            maps = []
            for j in range(2):
                s = (keys[:n, g, j] @ q[t, hd, j]) * m["scale"]
                maps.append(torch.softmax(s, dim=0) @ values[:n, g])
            out[t, hd] = maps[0] - lam * maps[1]
    out = rms_unit(out, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def dense_ff(h, w, pre):
    z = h @ w[pre + "up"].T + w[pre + "up.b"]
    a = xielu(z, w[pre + "act"][0], w[pre + "act"][1])
    return a @ w[pre + "down"].T + w[pre + "down.b"]


def gated_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, f, w, pre):
    """Per row: the chosen experts and their weights, [T, top] each."""
    r = f["router"]
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ w[pre + "router"].T, dim=-1)
    c = s + w[pre + "correction"]
    groups = r.get("groups")
    if groups:
        size = n // groups["count"]
        best = c.reshape(-1, groups["count"], size).max(dim=-1).values
        keep = torch.zeros_like(best, dtype=torch.bool)
        for t in range(best.shape[0]):
            order = sorted(range(groups["count"]), key=lambda g: (-float(best[t, g]), g))
            for g in order[:groups["keep"]]:
                keep[t, g] = True
        c = torch.where(keep.repeat_interleave(size, dim=1), c, torch.full_like(c, -math.inf))
    chosen = torch.zeros(h.shape[0], r["top"], dtype=torch.long)
    for t in range(h.shape[0]):
        order = sorted(range(n), key=lambda e: (-float(c[t, e]), e))
        chosen[t] = torch.tensor(order[:r["top"]])
    return chosen, torch.gather(s, 1, chosen)


def mixture(h, f, w, pre):
    r = f["router"]
    chosen, weights = route(h, f, w, pre)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= r["experts"]:
                out[t] += a * h[t]
            else:
                out[t] += a * gated_ff(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].T) * gated_ff(h, w, pre + "shared.")
    return out


def feed_forward(h, f, w, pre):
    return dense_ff(h, w, pre) if f["kind"] == "dense" else mixture(h, f, w, pre)


def model_layers(config, w, tokens, state=None):
    """One sequence's next ``tokens`` from ``state`` (None: a new sequence).  Returns (the stream after every layer
    [layers, T, width], logits [T, vocab], state)."""
    eps = config["norm"]["eps"]
    if state is None:
        state = {"n": 0, "S": {}, "K": {}, "V": {}}
    start = state["n"]
    x = w["embed"][torch.tensor(tokens)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "retention":
            y, state["S"][i] = retention(x, m, w, pre, eps, state["S"].get(i), start)
        else:
            src = m.get("kv_from")
            if src is None:
                k, v = attention_keys_values(x, m, w, pre, eps, start)
                state["K"][i] = k if i not in state["K"] else torch.cat([state["K"][i], k])
                state["V"][i] = v if i not in state["V"] else torch.cat([state["V"][i], v])
                src = i
            y = differential_attention(x, m, w, pre, eps, state["K"][src], state["V"][src], start)
        x = x + rms_unit(y, eps) * w[f"l{i}.norm1"]
        if layer.get("mlp"):
            x = x + rms_unit(feed_forward(x, layer["mlp"], w, f"l{i}.mlp."), eps) * w[f"l{i}.norm2"]
        streams.append(x)
    state["n"] = start + len(tokens)
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["head"].T
    return torch.stack(streams), logits, state
