"""A plain, slow restatement of the Rigotar design in float64, one function per mechanism.

Nothing here is shared with the product: no kernels, no parts, no cache.  Every function takes whole
sequences (rows are the positions 0..T-1 of ONE sequence) and loops over tokens where the design has a
recurrence.  Weights come as a dict of float64 tensors by their names in the weight file.

Notation: ``x`` [T, width] is the residual stream, ``h`` a mixer's input (the normed stream), linear
weights are [out, in] and applied as ``h @ W.T``.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x divided by sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    """RMS norm whose weight is a single number."""
    return rms_unit(x, eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def short_conv(x, taps_w, bias=None):
    """Causal convolution over time, per channel.  x [T, C]; taps_w [C, taps] with the LAST column
    multiplying the current token; inputs before the start are zero."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    out = torch.zeros(T, C, dtype=x.dtype)
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j][None, :]
    if bias is not None:
        out = out + bias[None, :]
    return out


def gated_delta_mixer(h, w, p, m, eps):
    """The gated delta rule.  ``m``: the mixer's sizes (heads, kv_heads, dim, vdim, conv)."""
    T = h.shape[0]
    H, KH, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, KH, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, KH, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                     # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(h @ w[p + "g"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    per_kv = H // KH
    for hd in range(H):
        S = torch.zeros(D, V, dtype=F64)
        kh = hd // per_kv
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, hd] = S.T @ q[t, kh]
    out = rms_unit(out, eps) * w[p + "norm"][None, None, :] * gate
    return out.reshape(T, H * V) @ w[p + "o"].T


def rglru_mixer(h, w, p, m):
    """Recurrent block with a real-gated linear recurrent unit."""
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"][None, :])
    u = short_conv(h @ w[p + "x"].T + w[p + "x.b"][None, :], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"][None]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"][None]).reshape(T, W)
    log_a = -8.0 * r * softplus(w[p + "lam"])[None, :]
    a = torch.exp(log_a)
    S = torch.zeros(W, dtype=F64)
    out = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


def latent_attention_mixer(h, w, p, m, eps):
    """Attention over a cached low-rank latent, no positions, a sink in the softmax denominator, an output gate."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    c = rms_unit(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"][None, :]
    k = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                      # [T, H]
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd].T) * m["scale"]                                # [T, T]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        top = torch.maximum(s.max(dim=-1).values, w[p + "sink"][hd])
        e = torch.exp(s - top[:, None])
        denom = e.sum(-1) + torch.exp(w[p + "sink"][hd] - top)
        out[:, hd] = (e / denom[:, None]) @ v[:, hd]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T


def moe_ffn(h, w, p, f):
    """Mixture of experts: the ``top`` largest router logits choose, softmax over the chosen logits weighs."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            ep = f"{p}e{e}."
            a = silu(h[t] @ w[ep + "gate"].T) * (h[t] @ w[ep + "up"].T)
            out[t] = out[t] + wt[t, j] * (a @ w[ep + "down"].T)
    return out


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = i
        while "weights_of" in cfg["layers"][src]:
            src = cfg["layers"][src]["weights_of"]
        p = f"l{src}."
        h = scalar_norm(x, w[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "delta":
            x = x + gated_delta_mixer(h, w, p + "mix.", m, eps)
        elif kind == "rglru":
            x = x + rglru_mixer(h, w, p + "mix.", m)
        elif kind == "latent_attention":
            x = x + latent_attention_mixer(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            x = x + moe_ffn(scalar_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T
