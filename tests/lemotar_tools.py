"""Shared by the Lemotar tests: small configurations that differ from one another in every size and option, weights drawn
so that activations are of order one (attention far from uniform, caps and sinks in reach, decays slow enough for a state
to last, gates neither shut nor open), model folders, and the plain implementation's logits."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, rot_dims=0, base=10000.0, scaling=None, window=None, kv_from=None, scale=None, ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return _entry("latent_attention", m, ff)


def left(heads, kv_heads, dim, rot_dims=0, window=None, softcap=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l, r, ff=None, ranks=(5, 3)):
    e = _entry("parallel", {"left": l, "right": r}, ff)
    e["_ranks"] = list(ranks)       # not a key of the design: the tests' weights are drawn with these ranks (decay, gate)
    return e


def _entry(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff is not None else None}


def model(vocab, width, eps, alpha, scale, layers):
    cfg = {"architecture": "Lemotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    return cfg


CONFIGS = {
    # no size a power of two or a multiple of eight; three heads; part of the rotated part turns, stretched; windows
    # that are no multiple of the page; a reader with a wider window than its writer; a layer without feed-forward;
    # two value heads a q/k head in the delta rule; one tap (no filter state) and two
    "P": model(131, 44, 3e-6, 1.7, 2.5, [
        latent(3, 10, 6, 7, 12, rot_dims=4, base=300.0, scaling=(3.0, 64, 8.0, 1.0), window=9, ff=56),
        parallel(left(6, 3, 10, rot_dims=4, window=17, softcap=4.0, base=300.0), right(4, 2, 5, 7, 2), ranks=(5, 3)),
        latent(2, 6, 6, 9, 12, rot_dims=4, base=300.0, scaling=(3.0, 64, 8.0, 1.0), window=13, kv_from=0, ff=20),
        parallel(left(2, 2, 6), right(3, 3, 6, 4, 1), ff=20, ranks=(2, 7))]),
    # multiples of 16 (the tensor-core kernels' sizes); one kv head; whole heads rotated, not stretched; no embedding
    # factor, alpha one; a latent layer without a window; windows of one page and of three
    "Q": model(200, 64, 1e-5, 1.0, None, [
        parallel(left(4, 1, 32, rot_dims=32, window=16, softcap=30.0, base=250000.0), right(2, 1, 16, 32, 4), ff=96, ranks=(8, 8)),
        latent(4, 32, 16, 32, 32, rot_dims=16, base=10000.0, ff=64),
        latent(2, 16, 16, 64, 32, rot_dims=16, base=10000.0, window=48, kv_from=1, ff=32),
        parallel(left(4, 4, 16, rot_dims=8, window=48), right(1, 1, 32, 16, 3), ranks=(16, 4))]),
    # a latent of 64 with a rotated part of 32 stretched by 8; heads of 64 in the softmax branch; keys of the delta rule
    # wider than a warp and wider than 64; five taps; values narrower and wider than keys
    "R": model(97, 48, 1e-6, 2.5, 6.0, [
        latent(2, 16, 32, 24, 64, rot_dims=32, base=1000.0, scaling=(8.0, 32, 4.0, 1.0), window=40, ff=40),
        parallel(left(2, 2, 64, rot_dims=2, window=8, softcap=8.0, base=50.0, scale=0.2), right(2, 2, 40, 24, 5), ff=40, ranks=(3, 3)),
        parallel(left(2, 1, 8, window=64), right(4, 2, 72, 8, 2), ranks=(4, 6))]),
}
PAGE_SIZES = {"P": 8, "Q": 16, "R": 8}
SEEDS = {"P": 51, "Q": 52, "R": 53}


def clean(cfg: dict) -> dict:
    """The configuration as the design's config.json holds it (without the tests' own keys)."""
    out = json.loads(json.dumps(cfg))
    for e in out["layers"]:
        e.pop("_ranks", None)
    return out


def draw_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> dict:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(n, std, mean=0.0):
        return (mean + std * torch.randn(n, generator=g)).to(dtype)

    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    w = {"embed": (torch.randn(cfg["vocab"], W, generator=g) / scale).to(dtype), "head": mat(cfg["vocab"], W, 2.0),
         "final.norm": vec(W, 0.2)}
    for i, entry in enumerate(cfg["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        w[p + "norm1"] = vec(W, 0.2)
        q = p + "mix."
        if entry["type"] == "latent_attention":
            H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[q + "q"] = mat(H * (d + r), W, 3.0)
            if m.get("kv_from") is None:
                w[q + "dkv"], w[q + "dkv.norm"] = mat(R + r, W, 1.5), vec(R, 0.2, 1.0)
            w[q + "uk"], w[q + "uv"] = mat(H * d, R, 1.5), mat(H * e, R, 1.5)
            w[q + "sink"] = vec(H, 1.0, 0.5)
            w[q + "g"], w[q + "o"] = mat(H * e, W, 1.5), mat(W, H * e)
        else:
            l, r_ = m["left"], m["right"]
            H, G, d = l["heads"], l["kv_heads"], l["dim"]
            a = q + "left."
            w[a + "q"], w[a + "k"], w[a + "o"] = mat(H * d, W, 1.5), mat(G * d, W, 1.5), mat(W, H * d)
            w[a + "q.norm"], w[a + "k.norm"] = vec(H * d, 0.3, 2.0), vec(G * d, 0.3, 2.0)      # scores of several units
            w[a + "out"] = vec(W, 0.2, 1.0)
            H, G, d, e, taps = r_["heads"], r_["kv_heads"], r_["dim"], r_["vdim"], r_["conv"]
            ra, rg = entry.get("_ranks", (5, 3))
            b = q + "right."
            w[b + "q"], w[b + "k"], w[b + "v"] = mat(G * d, W, 1.5), mat(G * d, W, 1.5), mat(H * e, W, 1.5)
            for n, size in (("q", G * d), ("k", G * d), ("v", H * e)):
                c = 0.4 * torch.randn(size, taps, generator=g)
                c[:, -1] += 1.0
                w[b + n + ".conv"] = c.to(dtype)
            w[b + "b"] = mat(H, W, 2.0)
            w[b + "A_log"] = (-1.0 + 2.0 * torch.rand(H, generator=g)).to(dtype)                 # rates of 0.37 to 2.7
            w[b + "dt_bias"] = (-4.0 + 3.5 * torch.rand(H * d, generator=g)).to(dtype)           # steps of 0.02 to 0.5
            w[b + "a1"], w[b + "a2"] = mat(ra, W, 1.5), mat(H * d, ra, 1.0)
            w[b + "g1"], w[b + "g2"] = mat(rg, W, 1.5), mat(H * e, rg, 1.5)
            w[b + "norm"], w[b + "o"], w[b + "out"] = vec(e, 0.2, 1.0), mat(W, H * e), vec(W, 0.2, 1.0)
        if entry["mlp"] is not None:
            ff = entry["mlp"]["ff"]
            w[p + "norm2"] = vec(W, 0.2)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff)
    return w


def write_folder(path, cfg: dict, weights: dict) -> Path:
    from quantinfer_b200.weights import write_safetensors

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(clean(cfg), indent=1))
    write_safetensors(path / "model.safetensors", {k: v.contiguous() for k, v in weights.items()})
    return path


def make(path, name: str):
    """(folder, config, weights) of the named configuration."""
    cfg = CONFIGS[name]
    w = draw_weights(cfg, SEEDS[name])
    return write_folder(path, cfg, w), clean(cfg), w


def plain_rows(cfg: dict, weights: dict, requests: dict) -> dict:
    """{(request, position): logits row} from the plain implementation."""
    from plain import plain_lemotar

    rows = {}
    for rid, toks in requests.items():
        logits = plain_lemotar.forward(cfg, weights, toks).to(torch.float32).numpy()
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows
