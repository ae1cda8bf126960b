"""Shared by the Dulotar tests: small configurations that differ from one another in every size and option, weights drawn
so that activations are of order one (attention far from uniform and its cap in reach, decays slow enough for a state to
last, gates neither shut nor open), model folders, and the plain implementation's logits."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def left(heads, kv_heads, dim, vdim, rot_dims=0, chunk=None, conv=None, softcap=None, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if conv is not None:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(l, r, left_scale=1.0, right_scale=1.0, ff=None, weights_of=None):
    return _entry("parallel", {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}, ff, weights_of)


def mingru(width, ff=None, weights_of=None):
    return _entry("mingru", {"width": width}, ff, weights_of)


def wkv(heads, dim, ff=None, weights_of=None, rank=6):
    e = _entry("wkv", {"heads": heads, "dim": dim}, ff, weights_of)
    e["_rank"] = rank          # not a key of the design: the tests' weights are drawn with this rank
    return e


def _entry(kind, mixer, ff, weights_of):
    e = {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff is not None else None}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def model(vocab, width, eps, scale, taps, layers):
    cfg = {"architecture": "Dulotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    return cfg


CONFIGS = {
    # no size a power of two or a multiple of eight; three kv heads; values smaller than keys; part of a head rotated; a
    # chunk that is no multiple of the page; five taps on the mixers' inputs, two on q, k, v; a layer that runs twice
    # with another's weights, between layers of other kinds
    "U": model(131, 44, 3e-6, 2.5, 5, [
        parallel(left(6, 3, 10, 6, rot_dims=4, chunk=9, conv=2, softcap=4.0, base=300.0), right(3, 5, 7, (0.5, 0.9, 0.97)), 0.8, 1.3, ff=56),
        wkv(3, 6, rank=5),
        mingru(30, ff=20),
        wkv(3, 6, weights_of=1, rank=5),
        mingru(30, ff=20, weights_of=2)]),
    # multiples of 16; one kv head; whole heads rotated; no cap, no convolution on q, k, v; one tap on the inputs (no state);
    # branch factors of one; a chunk of one page
    "V": model(200, 64, 1e-5, 1.0, 1, [
        mingru(64),
        parallel(left(4, 1, 32, 16, rot_dims=32, chunk=16, base=250000.0), right(2, 16, 32, (0.8, 0.999)), ff=96),
        parallel(left(4, 4, 16, 32, rot_dims=8, chunk=48, conv=4, softcap=30.0), right(1, 32, 16, (0.95,)), 1.5, 0.25),
        wkv(2, 32, ff=128, rank=16)]),
    # no input convolution at all; no chunks (every earlier key is seen); no rotation; keys wider than a warp's lanes in the
    # recurrences' state; heads of 64 (the padded sizes of the tensor-core kernel)
    "W": model(97, 48, 1e-6, 6.0, None, [
        parallel(left(2, 2, 64, 64, conv=3, softcap=8.0, scale=0.2), right(2, 40, 24, (0.7, 0.93)), 1.1, 0.6, ff=40),
        wkv(1, 40, rank=3),
        parallel(left(2, 1, 8, 8, rot_dims=2, chunk=8, base=50.0), right(2, 8, 8, (0.9, 0.6)), 0.5, 2.0, weights_of=None)]),
}
PAGE_SIZES = {"U": 8, "V": 16, "W": 8}
SEEDS = {"U": 41, "V": 42, "W": 43}


def clean(cfg: dict) -> dict:
    """The configuration as the design's config.json holds it (without the tests' own keys)."""
    out = json.loads(json.dumps(cfg))
    for e in out["layers"]:
        e.pop("_rank", None)
    return out


def draw_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> dict:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    taps = (cfg.get("canon") or {}).get("taps")

    def mat(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(n, std, mean=0.0):
        return (mean + std * torch.randn(n, generator=g)).to(dtype)

    def norm(name):
        return {name: vec(W, 0.2, 1.0), name + ".b": vec(W, 0.1)}

    w = {"embed": (torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"]).to(dtype), "head": mat(cfg["vocab"], W, 2.0)}
    w.update(norm("final.norm"))
    for i, entry in enumerate(cfg["layers"]):
        if entry.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", entry["mixer"]
        w.update(norm(p + "norm1"))
        if taps is not None:
            w[p + "canon1"] = (0.4 * torch.randn(W, taps, generator=g)).to(dtype)
        if entry["type"] == "parallel":
            l, r = m["left"], m["right"]
            H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            q = p + "mix.left."
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "o"] = mat(H * d, W, 2.5), mat(G * d, W, 2.5), mat(G * dv, W), mat(W, H * dv)
            if l.get("conv"):
                for n, size in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    c = 0.4 * torch.randn(size, l["conv"], generator=g)
                    c[:, -1] += 1.0                      # mostly the current token, so that rotation and scores keep their meaning
                    w[q + n + ".conv"] = c.to(dtype)
            Hr, dr, dvr = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(Hr * dr, W, 1.5), mat(Hr * dr, W, 1.5), mat(Hr * dvr, W, 1.5), mat(Hr * dvr, W, 1.5)
            w[q + "o"], w[q + "norm"] = mat(W, Hr * dvr), vec(Hr * dvr, 0.2, 1.0)
        elif entry["type"] == "mingru":
            n = m["width"]
            q = p + "mix."
            w[q + "z"], w[q + "x"], w[q + "g"], w[q + "o"] = mat(n, W, 1.5), mat(n, W, 1.5), mat(n, W, 1.5), mat(W, n)
            w[q + "z.b"], w[q + "x.b"] = vec(n, 0.5, -1.0), vec(n, 0.3)        # gates mostly small: the state lasts
        else:
            H, d, rank = m["heads"], m["dim"], entry.get("_rank", 6)
            q = p + "mix."
            for s in ("r", "k", "v", "g", "w"):
                w[q + "mu." + s] = torch.rand(W, generator=g).to(dtype)
            w[q + "r"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(H * d, W, 1.5), mat(H * d, W, 1.5), mat(H * d, W, 1.5), mat(H * d, W, 1.5)
            w[q + "w1"], w[q + "w2"] = mat(rank, W, 1.5), mat(H * d, rank, 1.0)
            w[q + "w0"] = (-0.5 - 3.5 * torch.rand(H * d, generator=g)).to(dtype)      # decays of 0.55 to 0.98 a step
            w[q + "u"] = (0.5 * torch.randn(H, d, generator=g)).to(dtype)
            w[q + "norm"], w[q + "o"] = vec(H * d, 0.2, 1.0), mat(W, H * d)
        if entry["mlp"] is not None:
            w.update(norm(p + "norm2"))
            ff = entry["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W, 1.5), mat(W, ff)
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
    from plain import plain_dulotar

    rows = {}
    for rid, toks in requests.items():
        logits = plain_dulotar.forward(cfg, weights, toks).to(torch.float32).numpy()
        for p in range(len(toks)):
            rows[(rid, p)] = logits[p]
    return rows
