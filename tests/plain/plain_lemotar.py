"""A plain, slow restatement of the Lemotar design in float64, one function per mechanism, for whole
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


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + f64(w))


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * f64(w)


def pair_frequencies(dims, base, scaling=None):
    """One frequency a pair and the factor on cos and sin. Without `scaling`: base^(-2i / dims) and 1. With it
    (factor, original, fast, slow): frequencies of pairs that turn slowly are divided by the factor, with a
    linear ramp over the pair's number between the two bounds, and cos and sin grow by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0

    def where(turns):
        return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / scaling["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate(x, positions, dims, freqs, magnitude, layout):
    """x [T, ..., d]: the first `dims` coordinates turn; pair i is (2i, 2i + 1) for layout "interleaved" and
    (i, i + dims / 2) for "half". (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * freqs[i]."""
    if not dims:
        return x
    ang = positions.to(F)[:, None] * freqs[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = (torch.cos(ang) * magnitude).reshape(shape), (torch.sin(ang) * magnitude).reshape(shape)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def window_mask(T, size=None):
    """[T, T] True where query i sees key j: 0 <= i - j < size (size None: every earlier key)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size:
        ok &= (i - j) < size
    return ok


def softmax_with_sink(scores, ok, sink):
    """scores [H, T, T]; the denominator holds exp(sink_h) once more (sink [H]); masked keys weigh nothing."""
    s = scores.masked_fill(~ok[None], -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def softcap(s, cap):
    return cap * torch.tanh(s / cap) if cap else s


def rotate_part(x, m):
    """The rotated part of a latent-attention query or key: halves paired, frequencies stretched where the mixer says so."""
    rot = m.get("rot")
    if not rot or not rot["dims"]:
        return x
    freqs, mag = pair_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    return rotate(x, torch.arange(x.shape[0]), rot["dims"], freqs, mag, "half")


def latent_rows(h, m, w, p, eps):
    """What a layer with a latent projection caches: the normed latent [T, kv_rank] and the rotated shared key part."""
    T = h.shape[0]
    R, r = m["kv_rank"], m["rot_dim"]
    z = h @ f64(w[p + "dkv"]).T
    c = norm_plain(z[:, :R], w[p + "dkv.norm"], eps)
    return c, rotate_part(z[:, R:R + r], m)


def latent_attention(h, m, w, p, eps, latent):
    """`latent` = (c, kr) of this layer or of the layer it reads."""
    T = h.shape[0]
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = latent
    q = (h @ f64(w[p + "q"]).T).view(T, H, d + r)
    qr = rotate_part(q[..., d:], m)
    k = (c @ f64(w[p + "uk"]).T).view(T, H, d)
    v = (c @ f64(w[p + "uv"]).T).view(T, H, e)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :d], k) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    pr = softmax_with_sink(scores, window_mask(T, (m.get("mask") or {}).get("size")), f64(w[p + "sink"]))
    o = torch.einsum("hij,jhe->ihe", pr, v).reshape(T, H * e)
    o = o * torch.sigmoid(h @ f64(w[p + "g"]).T)
    return o @ f64(w[p + "o"]).T


def grouped_attention(h, m, w, p, eps):
    """The left branch: values are the keys as projected; one norm over all of q and one over all of k; rotation
    in neighbouring pairs; capped scores; a window; a sink of score zero."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = h @ f64(w[p + "q"]).T
    k = h @ f64(w[p + "k"]).T
    v = k.view(T, G, d)
    q = norm_plain(q, w[p + "q.norm"], eps).view(T, H, d)
    k = norm_plain(k, w[p + "k.norm"], eps).view(T, G, d)
    rot = m.get("rot")
    if rot and rot["dims"]:
        freqs, mag = pair_frequencies(rot["dims"], rot["base"])
        q = rotate(q, torch.arange(T), rot["dims"], freqs, mag, "interleaved")
        k = rotate(k, torch.arange(T), rot["dims"], freqs, mag, "interleaved")
    group = torch.arange(H) // (H // G)
    scores = softcap(torch.einsum("ihd,jhd->hij", q, k[:, group]) * m["scale"], m.get("softcap"))
    pr = softmax_with_sink(scores, window_mask(T, (m.get("mask") or {}).get("size")), torch.zeros(H, dtype=F))
    o = torch.einsum("hij,jhe->ihe", pr, v[:, group]).reshape(T, H * d)
    return o @ f64(w[p + "o"]).T


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


def unit_vectors(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, dk], v [T, H, dv], beta [T, H], g [T, H, dk]. Per head, token by token: S = g S (rows are key
    channels); u = beta (v - S^T k); S = S + k u^T; o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = S * g[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def gated_delta(h, m, w, p, eps):
    """The right branch."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ f64(w[p + "q"]).T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ f64(w[p + "k"]).T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ f64(w[p + "v"]).T, w[p + "v.conv"])).view(T, H, e)
    group = torch.arange(H) // (H // G)
    q = (unit_vectors(q) * d ** -0.5)[:, group]
    k = unit_vectors(k)[:, group]
    beta = torch.sigmoid(h @ f64(w[p + "b"]).T)
    rate = torch.nn.functional.softplus((h @ f64(w[p + "a1"]).T) @ f64(w[p + "a2"]).T + f64(w[p + "dt_bias"])).view(T, H, d)
    g = torch.exp(-torch.exp(f64(w[p + "A_log"]))[None, :, None] * rate)
    o = delta_rule(q, k, v, beta, g)
    o = unit_rms(o, eps) * f64(w[p + "norm"])
    o = o.reshape(T, H * e) * torch.sigmoid((h @ f64(w[p + "g1"]).T) @ f64(w[p + "g2"]).T)
    return o @ f64(w[p + "o"]).T


def parallel_mixer(h, m, w, p, eps):
    left = grouped_attention(h, m["left"], w, p + "left.", eps)
    right = gated_delta(h, m["right"], w, p + "right.", eps)
    return 0.5 * (norm_plain(left, w[p + "left.out"], eps) + norm_plain(right, w[p + "right.out"], eps))


def gated_ffn(h, w, p):
    return (silu(h @ f64(w[p + "gate"]).T) * (h @ f64(w[p + "up"]).T)) @ f64(w[p + "down"]).T


def forward(cfg, w, tokens, keep_layers=False):
    """Logits [T, vocab] of a whole sequence; with keep_layers also the stream after every layer [layers, T, width]."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    latents, kept = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_rows(x, m, w, p + "mix.", eps)
                src = i
            y = latent_attention(x, m, w, p + "mix.", eps, latents[src])
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, m, w, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = norm_one_plus(alpha * x + y, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = norm_one_plus(alpha * x + gated_ffn(x, w, p + "mlp."), w[p + "norm2"], eps)
        if keep_layers:
            kept.append(x.clone())
    logits = norm_one_plus(x, w["final.norm"], eps) @ f64(w["head"]).T
    return (logits, torch.stack(kept)) if keep_layers else logits
