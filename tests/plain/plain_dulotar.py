"""A plain, slow restatement of the Dulotar design in float64, one function per mechanism, for whole
sequences at once (no cache, no state carried between calls, no batching). It reads the design's config
dictionary and a dictionary of tensors by name and shares nothing with the engine.

Notation: T tokens, positions 0 .. T - 1; matrices are stored [out, in] and applied as x @ W.T.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def f64(t):
    return t.to(F)


def silu(z):
    return z * torch.sigmoid(z)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis; var is the mean squared deviation."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * f64(w) + f64(b)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, w):
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    w = f64(w)
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * w[:, j]
    return y


def rotate_interleaved(x, positions, dims, base):
    """x [T, heads, d]: coordinates (2i, 2i + 1), i < dims / 2, turn by position * base^(-2i / dims)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F)
    ang = positions.to(F)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, chunk=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def conv_attention(h, m, w, p):
    """The softmax branch: projections, a short convolution on each, rotation, capped scores, chunks."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        y = h @ f64(w[p + n]).T
        if (p + n + ".conv") in w:
            y = causal_conv(y, w[p + n + ".conv"])
        proj[n] = y
    q, k, v = proj["q"].view(T, H, d), proj["k"].view(T, G, d), proj["v"].view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot") or {}
    q = rotate_interleaved(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_interleaved(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    mask = visible(T, (m.get("mask") or {}).get("size"))
    cap = m.get("softcap")
    out = torch.zeros(T, H, dv, dtype=F)
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, hq] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * dv) @ f64(w[p + "o"]).T


def lightning_attention(h, m, w, p, eps):
    """The linear branch: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; norm over all heads, gate, W_o."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ f64(w[p + "q"]).T).view(T, H, d)
    k = silu(h @ f64(w[p + "k"]).T).view(T, H, d)
    v = silu(h @ f64(w[p + "v"]).T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        lam = float(m["decay"][hh])
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = lam * S + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S.T @ q[t, hh]
    y = unit_rms(o.reshape(T, H * dv), eps) * f64(w[p + "norm"])
    y = y * torch.sigmoid(h @ f64(w[p + "g"]).T)
    return y @ f64(w[p + "o"]).T


def parallel_mixer(h, m, w, p, eps):
    left = conv_attention(h, m["left"], w, p + "left.")
    right = lightning_attention(h, m["right"], w, p + "right.", eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mingru(h, m, w, p):
    """S_t = (1 - z) S_(t-1) + z c, z = sigmoid(W_z h + b), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0)."""
    T = h.shape[0]
    z = torch.sigmoid(h @ f64(w[p + "z"]).T + f64(w[p + "z.b"]))
    u = h @ f64(w[p + "x"]).T + f64(w[p + "x.b"])
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = silu(h @ f64(w[p + "g"]).T)
    S = torch.zeros(z.shape[1], dtype=F)
    out = torch.zeros_like(z)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S * gate[t]
    return out @ f64(w[p + "o"]).T


def wkv(h, m, w, p, eps):
    """Time mixing with a decay per head and key channel; the current token's pair gets a bonus u."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]], dim=0)
    mix = {s: h + (prev - h) * f64(w[p + "mu." + s]) for s in ("r", "k", "v", "g", "w")}
    r = (mix["r"] @ f64(w[p + "r"]).T).view(T, H, d)
    k = (mix["k"] @ f64(w[p + "k"]).T).view(T, H, d)
    v = (mix["v"] @ f64(w[p + "v"]).T).view(T, H, d)
    gate = silu(mix["g"] @ f64(w[p + "g"]).T)
    lw = torch.tanh(mix["w"] @ f64(w[p + "w1"]).T) @ f64(w[p + "w2"]).T + f64(w[p + "w0"])
    decay = torch.exp(-torch.exp(lw)).view(T, H, d)
    u = f64(w[p + "u"])
    o = torch.zeros(T, H, d, dtype=F)
    for hh in range(H):
        S = torch.zeros(d, d, dtype=F)
        for t in range(T):
            kv = torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = (S + u[hh][:, None] * kv).T @ r[t, hh]
            S = decay[t, hh][:, None] * S + kv
    y = unit_rms(o, eps).reshape(T, H * d) * f64(w[p + "norm"]) * gate
    return y @ f64(w[p + "o"]).T


def dense_ffn(h, w, p):
    return torch.relu(h @ f64(w[p + "up"]).T) ** 2 @ f64(w[p + "down"]).T


def run_layers(cfg, w, tokens):
    """The stream after every layer run: list of [T, width]."""
    eps = cfg["norm"]["eps"]
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    taps = (cfg.get("canon") or {}).get("taps", 0)
    after = []
    for i, entry in enumerate(cfg["layers"]):
        src = entry.get("weights_of", i)
        L = f"l{src}."
        h = layer_norm(x, w[L + "norm1"], w[L + "norm1.b"], eps)
        if taps:
            h = h + causal_conv(h, w[L + "canon1"])
        kind, m = entry["type"], entry["mixer"]
        if kind == "parallel":
            y = parallel_mixer(h, m, w, L + "mix.", eps)
        elif kind == "mingru":
            y = mingru(h, m, w, L + "mix.")
        elif kind == "wkv":
            y = wkv(h, m, w, L + "mix.", eps)
        else:
            raise ValueError(kind)
        x = x + y
        if entry.get("mlp") is not None:
            x = x + dense_ffn(layer_norm(x, w[L + "norm2"], w[L + "norm2.b"], eps), w, L + "mlp.")
        after.append(x)
    return after


def forward(cfg, w, tokens):
    """Logits [T, vocab] of one sequence."""
    x = run_layers(cfg, w, tokens)[-1]
    return layer_norm(x, w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"]) @ f64(w["head"]).T
