"""The Gorulorn decoder, plainly: one function per mechanism, float64 throughout, a whole
sequence at a time, no cache, no batching.  It shares no code with the package; the engine's
tests hold the kernels and the step function to it.

Notation: ``x`` [T, W] activations of one sequence (positions 0..T-1), ``w`` a dict of the
model's tensors by name (float64), ``cfg`` the dict of config.json, ``p`` a tensor-name prefix.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, weight, eps):
    """Mean taken off, divided by the root of the variance (mean of squared deviations) + eps, times a weight."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * weight


def silu(x):
    return x * torch.sigmoid(x)


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------

def short_convolution(u, taps_w):
    """Per channel, over time: y_t = sum_j w[:, j] u_(t - taps + 1 + j); zeros before the first token."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), u], dim=0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y


def rotate(x, positions, dims, base):
    """x [T, heads, d]: element i of the first ``dims`` turns together with element i + dims/2 by position * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(T, size, keep_first=0):
    """[T, T] bool: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_attention(q, k, v, scale, mask, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head a reads key head a // (H / G).  ``sink`` [H]: a number per head
    whose exponential joins the denominator and nothing else."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[a].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[a] - m)
        out[:, a] = (e / den) @ v[:, g]
    return out


def window_attention(h, w, p, m, eps):
    """Grouped-query attention: biased projections, a short convolution on each of them, a norm per head on queries and
    keys, rotation of part of each head, a sliding window that also keeps the first tokens."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G = m.get("kv_heads") or H
    dv = m.get("vdim") or d
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ w[p + n].T
        if p + n + ".b" in w:
            u = u + w[p + n + ".b"]
        if m.get("conv"):
            u = short_convolution(u, w[p + n + ".conv"])
        proj[n] = u
    q, k, v = proj["q"].view(T, H, d), proj["k"].view(T, G, d), proj["v"].view(T, G, dv)
    if p + "q.norm" in w:
        q = rms(q, eps) * w[p + "q.norm"]
        k = rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        pos = torch.arange(T)
        q, k = rotate(q, pos, rot["dims"], rot["base"]), rotate(k, pos, rot["dims"], rot["base"])
    mask = m.get("mask") or {}
    vis = visible(T, int(mask.get("size") or T), int(mask.get("keep_first") or 0))
    o = softmax_attention(q, k, v, float(m["scale"]), vis)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Queries through a normalised latent; keys and values of every head from one normalised latent per token; no
    positions; a sliding window; a sink in the softmax's denominator."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    dv = m.get("vdim") or d
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d)
    c = rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    mask = m.get("mask") or {}
    vis = visible(T, int(mask.get("size") or T))
    o = softmax_attention(q, k, v, float(m["scale"]), vis, sink=w.get(p + "sink"))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def routed_experts(h, w, p, mlp):
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert run on its score times the input, outputs summed."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = torch.sigmoid(h @ w[p + "router"].T)                         # [T, E]
    chosen = torch.topk(s, top, dim=-1).indices
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            z = s[t, e] * h[t]
            pe = f"{p}e{e}."
            y[t] += (silu(z @ w[pe + "gate"].T) * (z @ w[pe + "up"].T)) @ w[pe + "down"].T
    return y


def mixer(h, w, p, layer, eps):
    if layer["type"] == "attention":
        return window_attention(h, w, p, layer["mixer"], eps)
    if layer["type"] == "latent_attention":
        return latent_attention(h, w, p, layer["mixer"], eps)
    raise ValueError(layer["type"])


def layer_forward(x, w, i, layer, eps):
    """Both sublayers between two norms each: x += post(sublayer(pre(x)))."""
    p = f"l{i}."
    y = mixer(layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer, eps)
    x = x + layer_norm(y, w[p + "norm1b"], eps)
    if layer.get("mlp") is not None:
        y = routed_experts(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        x = x + layer_norm(y, w[p + "norm2b"], eps)
    return x


def layer_runs(cfg):
    """The order in which layers run: (layer, pass or None); a looped span runs ``times`` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, w, tokens, keep=None):
    """Logits [T, vocab] of one sequence; ``keep``: a list that receives the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    loop = cfg.get("loop")
    for i, t in layer_runs(cfg):
        if t is not None and i == int(loop["start"]):
            x = x + w["loop.step"][t]
        x = layer_forward(x, w, i, cfg["layers"][i], eps)
        if keep is not None:
            keep.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
