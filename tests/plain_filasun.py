"""The Filasun decoder, plainly: one function per mechanism, token by token where the
mechanism is a recurrence, float64 throughout, no cache, no batching.  It shares no code
with the package; the engine's tests hold the kernels and the step function to it.

Notation: ``x`` [T, W] activations of one sequence (positions 0..T-1), ``w`` a dict of the
model's tensors by name (float64), ``cfg`` the dict of config.json.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


# ---------------------------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------------------------

def windowed_attention(h, w, p, m):
    """Softmax attention over the last ``m['mask']['size']`` positions, grouped key heads, scores
    capped by a tanh, a penalty that grows linearly with the distance, one sigmoid gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                           # [T, H]
    cap, size = float(m["softcap"]), int(m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        lo = max(0, i - size + 1)
        dist = torch.arange(i - lo, -1, -1, dtype=F)                 # i - j for j = lo..i
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ q[i, a]) * float(m["scale"])
            s = cap * torch.tanh(s / cap)
            s = s - 2.0 ** (-8.0 * (a + 1) / H) * dist
            out[i, a] = torch.softmax(s, dim=0) @ v[lo:i + 1, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def decayed_linear_attention(h, w, p, m, eps):
    """A matrix of state per head that fades by a constant factor a token and takes the outer
    product of key and value; read out with the query; heads normalised together, gated, projected."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms(o.reshape(T, H * dv), eps) * w[p + "norm"]
    y = y * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = windowed_attention(h, w, p + "left.", m["left"])
    right = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def selective_state_space(h, w, p, m, eps):
    """Input-dependent step sizes, a scalar decay per head, a short causal convolution before,
    a gate and a norm in groups after."""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    C = xbc.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), xbc], dim=0)
    conv = torch.zeros(T, C, dtype=F)
    for t in range(T):
        conv[t] = (padded[t:t + taps] * w[p + "conv"].T).sum(dim=0) + w[p + "conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, P)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    Cm = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                              # [T, H]
    rate = torch.exp(w[p + "A_log"])
    S = torch.zeros(H, N, P, dtype=F)
    y = torch.zeros(T, H, P, dtype=F)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = torch.exp(-rate[a] * dt[t, a]) * S[a] + dt[t, a] * B[t, g][:, None] * x[t, a][None, :]
            y[t, a] = S[a].T @ Cm[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def clamped_glu(h, w, p, m):
    limit = float(m["limit"])
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def hyper_sublayer(xs, w, p, norm_w, eps, fn):
    """xs [T, s, W]: read one input as a weighted sum of the streams, run the sublayer on its norm,
    mix the streams among themselves and add the output to each with its own factor."""
    u = torch.einsum("s,tsw->tw", w[p + "in"], xs)
    y = fn(rms(u, eps) * norm_w)
    return torch.einsum("sr,tsw->trw", w[p + "mix"], xs) + w[p + "out"][None, :, None] * y[:, None, :]


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------

def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence fed whole; with ``return_layers`` also the sum of the streams after every layer."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] + w["pos"][:T]
    s = int(cfg["streams"])
    xs = x[:, None, :].repeat(1, s, 1)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "parallel":
            mixer = lambda hh: parallel_mixer(hh, w, p + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            mixer = lambda hh: selective_state_space(hh, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        xs = hyper_sublayer(xs, w, p + "hc1.", w[p + "norm1"], eps, mixer)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            xs = hyper_sublayer(xs, w, p + "hc2.", w[p + "norm2"], eps, lambda hh: clamped_glu(hh, w, p + "mlp.", layer["mlp"]))
        after.append(xs.sum(dim=1))
    x = rms(xs.sum(dim=1), eps) * w["final.norm"]
    logits = x @ w["head"].T
    cap = float(cfg["logit_softcap"])
    logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits
