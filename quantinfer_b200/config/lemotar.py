"""Typed configuration of the Lemotar design, read from the keys of its config.json.

A small decoder-only model whose norms come AFTER the sums: x <- norm(alpha x + sublayer(x)), the norm an RMS norm
with a weight stored around zero (gain 1 + w). Two mixers. (1) Attention over a cached latent with a sliding window, a
learned sink per head, an output gate, a rotated part in half-split pairs whose frequencies may be stretched (YaRN);
a layer may read another layer's cached latent. (2) Two branches side by side on one input: softmax attention over
grouped heads whose values are the keys as projected, with one RMS norm over all of q and one over all of k, rotation in
neighbouring pairs, capped scores, a sliding window and one added to the softmax's denominator; and a gated delta rule
over a matrix state per head (short convolutions with silu on q, k, v; unit vectors; a decay per head and key channel;
a gated RMS norm per head). Each branch's output passes an RMS norm over the model width; half their sum is the
mixer's. The feed-forward is gated with silu.

config.json keys (every size, and every constant that can differ between models):

    architecture            "Lemotar"
    vocab, width
    norm.eps                eps of every RMS norm (the unit vectors of the delta rule have their own, fixed below)
    postln_alpha            alpha
    embedding.scale         factor on the embedding's rows
    layers[i]               {type: "latent_attention" | "parallel", mixer: {...}, mlp: {kind: "dense", ff} or null}
      latent_attention      {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {base, dims, scaling: {factor, original,
                             fast, slow} (optional)}, mask: {size} (optional), kv_from: j (optional)}
      parallel              {left: {heads, kv_heads, dim, vdim, scale, softcap (optional), rot: {base, dims} (optional),
                             mask: {size} (optional)}, right: {heads, kv_heads, dim, vdim, conv}}

Tensor names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,g,o}`, or
`l<i>.mix.left.{q,k,q.norm,k.norm,o,out}` and `l<i>.mix.right.{q,k,v,q.conv,k.conv,v.conv,b,A_log,a1,a2,dt_bias,g1,g2,
norm,o,out}`; `l<i>.mlp.{gate,up,down}`; `final.norm`, `head`. The design sets no limit on positions.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from ..errors import ConfigError
from .bebuvik import UNLIMITED_POSITIONS, _get
from .spec import (EmbeddingSpec, FeedForwardSpec, GatedAttentionSpec, GatedDeltaSpec, HeadSpec, LatentAttentionSpec, LayerCall,
                   ModelSpec, NormSpec, ParallelMixersSpec, PostNormLayerSpec, RotarySpec)

ARCHITECTURE = "Lemotar"

# constants the design fixes
FFN_ACTIVATION = "silu"
LATENT_PAIRING = "half_split"      # coordinate i turns with coordinate i + dims / 2
LEFT_PAIRING = "interleaved"       # coordinate 2i turns with coordinate 2i + 1
LEFT_SINK = "zero"                 # one is added to the softmax's denominator
UNIT_EPS = 1e-6                    # inside the root of the delta rule's unit vectors
BRANCH_SUM_SCALE = 0.5             # half the sum of the two branches


@dataclass(frozen=True)
class LemotarStretch:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LemotarLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    stretch: object = None     # LemotarStretch or None
    window: object = None      # None: every earlier position
    kv_from: object = None     # None: the layer projects its own latent


@dataclass(frozen=True)
class LemotarSoftmaxBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: object = None
    rot_base: float = 10000.0
    rot_dims: int = 0
    window: object = None


@dataclass(frozen=True)
class LemotarDeltaBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class LemotarParallel:
    left: LemotarSoftmaxBranch
    right: LemotarDeltaBranch


@dataclass(frozen=True)
class LemotarLayer:
    kind: str                  # "latent_attention" | "parallel"
    mixer: object
    ff: object = None          # the feed-forward's inner width; None: no feed-forward


@dataclass(frozen=True)
class LemotarConfig:
    vocab: int
    width: int
    norm_eps: float
    alpha: float
    embedding_scale: float
    layers: tuple
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "LemotarConfig":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        if d.get("architecture", ARCHITECTURE) != ARCHITECTURE and ARCHITECTURE not in (d.get("architectures") or []):
            raise ConfigError(f"this is not a {ARCHITECTURE} configuration")
        layers_in = d.get("layers")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError("config.json `layers` must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json `layers[{i}]` must be an object")
            m = _get(entry, "mixer", dict, where)
            mw = where + "mixer."
            kind = entry.get("type")
            if kind == "latent_attention":
                rot = _get(m, "rot", dict, mw, required=False)
                sc = _get(rot, "scaling", dict, mw + "rot.", required=False) if rot is not None else None
                mask = _get(m, "mask", dict, mw, required=False)
                sw = mw + "rot.scaling."
                mixer = LemotarLatent(
                    heads=_get(m, "heads", int, mw), dim=_get(m, "dim", int, mw), rot_dim=_get(m, "rot_dim", int, mw),
                    vdim=_get(m, "vdim", int, mw), kv_rank=_get(m, "kv_rank", int, mw), scale=_get(m, "scale", float, mw),
                    rot_base=_get(rot, "base", float, mw + "rot.") if rot is not None else 10000.0,
                    rot_dims=_get(rot, "dims", int, mw + "rot.") if rot is not None else 0,
                    stretch=LemotarStretch(_get(sc, "factor", float, sw), _get(sc, "original", float, sw), _get(sc, "fast", float, sw),
                                           _get(sc, "slow", float, sw)) if sc is not None else None,
                    window=_get(mask, "size", int, mw + "mask.") if mask is not None else None,
                    kv_from=_get(m, "kv_from", int, mw, required=False))
            elif kind == "parallel":
                l, r = _get(m, "left", dict, mw), _get(m, "right", dict, mw)
                lw, rw = mw + "left.", mw + "right."
                rot = _get(l, "rot", dict, lw, required=False)
                mask = _get(l, "mask", dict, lw, required=False)
                mixer = LemotarParallel(
                    left=LemotarSoftmaxBranch(
                        heads=_get(l, "heads", int, lw), kv_heads=_get(l, "kv_heads", int, lw), dim=_get(l, "dim", int, lw),
                        vdim=_get(l, "vdim", int, lw), scale=_get(l, "scale", float, lw),
                        softcap=_get(l, "softcap", float, lw, required=False),
                        rot_base=_get(rot, "base", float, lw + "rot.") if rot is not None else 10000.0,
                        rot_dims=_get(rot, "dims", int, lw + "rot.") if rot is not None else 0,
                        window=_get(mask, "size", int, lw + "mask.") if mask is not None else None),
                    right=LemotarDeltaBranch(heads=_get(r, "heads", int, rw), kv_heads=_get(r, "kv_heads", int, rw),
                                             dim=_get(r, "dim", int, rw), vdim=_get(r, "vdim", int, rw), conv=_get(r, "conv", int, rw)))
            else:
                raise ConfigError(f"config.json `{where}type` is {kind!r}; this design's mixers are 'latent_attention' and 'parallel'")
            mlp_in, ff = entry.get("mlp"), None
            if mlp_in is not None:
                if not isinstance(mlp_in, dict) or mlp_in.get("kind") != "dense":
                    raise ConfigError(f"config.json `{where}mlp` must be null or an object of kind 'dense'")
                ff = _get(mlp_in, "ff", int, where + "mlp.")
            layers.append(LemotarLayer(kind, mixer, ff))
        emb = _get(d, "embedding", dict, "", required=False)
        cfg = cls(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                  norm_eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
                  alpha=_get(d, "postln_alpha", float, "", required=False, default=1.0),
                  embedding_scale=_get(emb, "scale", float, "embedding.", required=False, default=1.0) if emb is not None else 1.0,
                  layers=tuple(layers), raw=copy.deepcopy(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        if self.raw:
            return copy.deepcopy(self.raw)
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "postln_alpha": self.alpha, "embedding": {"scale": self.embedding_scale}, "layers": []}
        for layer in self.layers:
            m = layer.mixer
            if layer.kind == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
                if m.rot_dims:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                    if m.stretch is not None:
                        s = m.stretch
                        mixer["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                l, r = m.left, m.right
                left = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale}
                if l.softcap is not None:
                    left["softcap"] = l.softcap
                if l.rot_dims:
                    left["rot"] = {"base": l.rot_base, "dims": l.rot_dims}
                if l.window is not None:
                    left["mask"] = {"size": l.window}
                mixer = {"left": left, "right": {"heads": r.heads, "kv_heads": r.kv_heads, "dim": r.dim, "vdim": r.vdim, "conv": r.conv}}
            d["layers"].append({"type": layer.kind, "mixer": mixer,
                                "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff is not None else None})
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Lemotar `vocab` and `width` must be greater than zero")
        if self.norm_eps <= 0.0:
            raise ConfigError("Lemotar `norm.eps` must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.kind == "latent_attention":
                if min(m.heads, m.dim, m.vdim, m.kv_rank) <= 0:
                    raise ConfigError(f"Lemotar layer {i}: heads, dim, vdim and kv_rank must be greater than zero")
                if m.rot_dims % 2 or m.rot_dims > m.rot_dim:
                    raise ConfigError(f"Lemotar layer {i}: rot.dims ({m.rot_dims}) must be even and within rot_dim ({m.rot_dim})")
                if (m.rot_dims and m.rot_base <= 1.0) or m.scale <= 0.0:
                    raise ConfigError(f"Lemotar layer {i}: rot.base must be above one and scale positive")
                s = m.stretch
                if s is not None and (s.factor < 1.0 or min(s.original, s.fast, s.slow) <= 0.0):
                    raise ConfigError(f"Lemotar layer {i}: rot.scaling needs a factor of at least one and positive original, fast and slow")
                if m.window is not None and m.window <= 0:
                    raise ConfigError(f"Lemotar layer {i}: mask.size must be positive")
                if m.kv_from is not None:
                    if not 0 <= m.kv_from < i or self.layers[m.kv_from].kind != "latent_attention":
                        raise ConfigError(f"Lemotar layer {i}: kv_from ({m.kv_from}) must name an earlier latent-attention layer")
                    src = self.layers[m.kv_from].mixer
                    if src.kv_from is not None:
                        raise ConfigError(f"Lemotar layer {i}: kv_from names layer {m.kv_from}, which has no latent projection of its own")
                    if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims, src.stretch) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims, m.stretch):
                        raise ConfigError(f"Lemotar layer {i}: its latent size and rotation differ from those of layer {m.kv_from}, whose cache it reads")
            else:
                l, r = m.left, m.right
                if min(l.heads, l.kv_heads, l.dim, l.vdim) <= 0 or l.heads % l.kv_heads:
                    raise ConfigError(f"Lemotar layer {i}: left.heads must be a positive multiple of left.kv_heads, dim and vdim positive")
                if l.vdim != l.dim:
                    raise ConfigError(f"Lemotar layer {i}: the left branch's values are its keys, so left.vdim ({l.vdim}) must equal left.dim ({l.dim})")
                if l.rot_dims % 2 or l.rot_dims > l.dim:
                    raise ConfigError(f"Lemotar layer {i}: left.rot.dims ({l.rot_dims}) must be even and within dim ({l.dim})")
                if (l.rot_dims and l.rot_base <= 0.0) or l.scale <= 0.0:
                    raise ConfigError(f"Lemotar layer {i}: left.rot.base and left.scale must be positive")
                if l.window is not None and l.window <= 0:
                    raise ConfigError(f"Lemotar layer {i}: left.mask.size must be positive")
                if l.softcap is not None and l.softcap <= 0.0:
                    raise ConfigError(f"Lemotar layer {i}: left.softcap must be positive")
                if min(r.heads, r.kv_heads, r.dim, r.vdim) <= 0 or r.heads % r.kv_heads:
                    raise ConfigError(f"Lemotar layer {i}: right.heads must be a positive multiple of right.kv_heads, dim and vdim positive")
                if not 1 <= r.conv <= 16:
                    raise ConfigError(f"Lemotar layer {i}: right.conv must lie in 1..16")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"Lemotar layer {i}: mlp.ff must be greater than zero")

    # ---- the model as data --------------------------------------------------

    def to_model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name):
            return NormSpec(w, eps, name, "rmsnorm_one_plus")

        layers, order, entry_of = [], [], {}
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.kind == "latent_attention":
                s = m.stretch
                position = RotarySpec(m.rot_dims, m.rot_base, LATENT_PAIRING,
                                      stretch=(s.factor, s.original, s.fast, s.slow) if s is not None else None) if m.rot_dims else None
                mixer = LatentAttentionSpec(
                    hidden_size=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank,
                    position=position, norm_eps=eps, scale=m.scale, window=m.window, sink=True, shares_latent=m.kv_from is not None,
                    prefix=p + "mix.", out_gate=True)
            else:
                l, r = m.left, m.right
                left = GatedAttentionSpec(
                    hidden_size=w, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim, value_dim=l.dim,
                    position=RotarySpec(l.rot_dims, l.rot_base, LEFT_PAIRING) if l.rot_dims else None, scale=l.scale, chunk=None,
                    window=l.window, bias=False, out_gate=False, prefix=p + "mix.left.", softcap=l.softcap, sink=LEFT_SINK,
                    values_from_keys=True, qk_norm="whole", qk_norm_eps=eps)
                right = GatedDeltaSpec(hidden_size=w, heads=r.heads, kv_heads=r.kv_heads, head_dim=r.dim, value_dim=r.vdim,
                                       conv_taps=r.conv, norm_eps=eps, unit_eps=UNIT_EPS, prefix=p + "mix.right.")
                mixer = ParallelMixersSpec(left, right, prefix=p + "mix.", out_norm_names=(p + "mix.left.out", p + "mix.right.out"),
                                           out_norm_eps=eps, sum_scale=BRANCH_SUM_SCALE, hidden_size=w)
            ffn = FeedForwardSpec(w, layer.ff, FFN_ACTIVATION, p + "mlp.", names=("gate", "up", "down")) if layer.ff is not None else None
            layers.append(PostNormLayerSpec(mixer_norm=norm(p + "norm1"), mixer=mixer, ffn_norm=norm(p + "norm2") if ffn is not None else None,
                                            ffn=ffn, alpha=self.alpha))
            if layer.kind == "latent_attention" and m.kv_from is not None:
                order.append(LayerCall(i, entry_of[m.kv_from], False))
            else:
                entry_of[i] = len(entry_of)
                order.append(LayerCall(i, entry_of[i], True))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w, max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, w, "", weight_name="embed", scale=self.embedding_scale), layers=tuple(layers),
            order=tuple(order), final_norm=norm("final.norm"), head=HeadSpec(self.vocab, w, False, "", weight_name="head"),
            eos_token_id=None)
        spec.validate()
        return spec
