"""Typed configuration of the Dulotar design, read from the keys of its config.json.

A small decoder-only model of pre-norm layers (layer norm with gain and bias) whose mixers are recurrent or part
recurrent: a gated recurrence per channel (minGRU), time mixing over a matrix state with a decay per key channel
(RWKV style), or two branches side by side: softmax attention over a chunk of the sequence (grouped heads, a short
convolution on q, k and v, rotation in interleaved pairs, capped scores) plus linear attention with one constant
decay a head. Every mixer reads h + conv(h), a causal convolution of the normalised stream over time. The
feed-forward, where a layer has one, is dense with a squared relu. A layer may run with another layer's weights.

config.json keys (every size, and every constant that can differ between models):

    architecture            "Dulotar"
    vocab, width
    norm.eps                eps of the layer norms and of the RMS norms inside mixers
    embedding.scale         factor on the embedding's rows
    canon.taps              taps of the input convolution of every layer's mixer (absent: no such convolution)
    layers[i]               {type: "parallel" | "mingru" | "wkv", mixer: {...}, mlp: {kind: "dense", ff} or null,
                             weights_of: j (optional: run with layer j's tensors, state and cache of its own)}
      parallel mixer        {left: {heads, kv_heads, dim, vdim, scale, conv, softcap, rot: {base, dims}, mask: {size}},
                             right: {heads, dim, vdim, decay: [one a head]}, left_scale, right_scale}
      mingru mixer          {width}
      wkv mixer             {heads, dim}        (the rank of the decay's two projections is the shape of `mix.w1`)

Tensor names: `embed`, `l<i>.norm1|norm2` (each with `.b`), `l<i>.canon1`, `l<i>.mix.left.{q,k,v,o}` and
`l<i>.mix.left.{q,k,v}.conv`, `l<i>.mix.right.{q,k,v,g,o,norm}`, or `l<i>.mix.{z,z.b,x,x.b,g,o}`, or
`l<i>.mix.{mu.r,mu.k,mu.v,mu.g,mu.w,r,k,v,g,w1,w2,w0,u,norm,o}`; `l<i>.mlp.{up,down}`; `final.norm` (`.b`), `head`.
The design sets no limit on positions.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field

from ..errors import ConfigError
from .bebuvik import UNLIMITED_POSITIONS, _get
from .spec import (ConvPreNormLayerSpec, DenseFeedForwardSpec, EmbeddingSpec, GatedAttentionSpec, HeadSpec, LayerCall,
                   LightningAttentionSpec, MinGRUSpec, ModelSpec, NormSpec, ParallelMixersSpec, RotarySpec, ShortConvSpec,
                   TimeMixSpec)

ARCHITECTURE = "Dulotar"

# constants the design fixes
FFN_ACTIVATION = "relu2"           # the square of relu
ROTATION_PAIRING = "interleaved"   # coordinate 2i turns with coordinate 2i + 1


@dataclass(frozen=True)
class DulotarSoftmaxBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: object = None            # taps of the convolution on q, k, v; None: none
    softcap: object = None
    rot_base: float = 10000.0
    rot_dims: int = 0
    chunk: object = None           # mask.size; None: every earlier position


@dataclass(frozen=True)
class DulotarLinearBranch:
    heads: int
    dim: int
    vdim: int
    decay: tuple


@dataclass(frozen=True)
class DulotarParallel:
    left: DulotarSoftmaxBranch
    right: DulotarLinearBranch
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DulotarMinGRU:
    width: int


@dataclass(frozen=True)
class DulotarWKV:
    heads: int
    dim: int


@dataclass(frozen=True)
class DulotarLayer:
    kind: str                      # "parallel" | "mingru" | "wkv"
    mixer: object
    ff: object = None              # the dense feed-forward's inner width; None: no feed-forward
    weights_of: object = None      # the layer whose tensors this one runs with; None: its own


@dataclass(frozen=True)
class DulotarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    canon_taps: object             # None: no input convolution
    layers: tuple
    raw: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, d: dict) -> "DulotarConfig":
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
            if kind == "parallel":
                l, r = _get(m, "left", dict, mw), _get(m, "right", dict, mw)
                lw, rw = mw + "left.", mw + "right."
                rot = _get(l, "rot", dict, lw, required=False)
                mask = _get(l, "mask", dict, lw, required=False)
                decay = r.get("decay")
                if not isinstance(decay, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise ConfigError(f"config.json `{rw}decay` must be a list of numbers, one a head")
                mixer = DulotarParallel(
                    left=DulotarSoftmaxBranch(
                        heads=_get(l, "heads", int, lw), kv_heads=_get(l, "kv_heads", int, lw), dim=_get(l, "dim", int, lw),
                        vdim=_get(l, "vdim", int, lw), scale=_get(l, "scale", float, lw),
                        conv=_get(l, "conv", int, lw, required=False), softcap=_get(l, "softcap", float, lw, required=False),
                        rot_base=_get(rot, "base", float, lw + "rot.") if rot is not None else 10000.0,
                        rot_dims=_get(rot, "dims", int, lw + "rot.") if rot is not None else 0,
                        chunk=_get(mask, "size", int, lw + "mask.") if mask is not None else None),
                    right=DulotarLinearBranch(heads=_get(r, "heads", int, rw), dim=_get(r, "dim", int, rw),
                                              vdim=_get(r, "vdim", int, rw), decay=tuple(float(x) for x in decay)),
                    left_scale=_get(m, "left_scale", float, mw, required=False, default=1.0),
                    right_scale=_get(m, "right_scale", float, mw, required=False, default=1.0))
            elif kind == "mingru":
                mixer = DulotarMinGRU(_get(m, "width", int, mw))
            elif kind == "wkv":
                mixer = DulotarWKV(heads=_get(m, "heads", int, mw), dim=_get(m, "dim", int, mw))
            else:
                raise ConfigError(f"config.json `{where}type` is {kind!r}; this design's mixers are 'parallel', 'mingru' and 'wkv'")
            mlp_in, ff = entry.get("mlp"), None
            if mlp_in is not None:
                if not isinstance(mlp_in, dict) or mlp_in.get("kind") != "dense":
                    raise ConfigError(f"config.json `{where}mlp` must be null or an object of kind 'dense'")
                ff = _get(mlp_in, "ff", int, where + "mlp.")
            layers.append(DulotarLayer(kind, mixer, ff, _get(entry, "weights_of", int, where, required=False)))
        canon = _get(d, "canon", dict, "", required=False)
        emb = _get(d, "embedding", dict, "", required=False)
        cfg = cls(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                  norm_eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
                  embedding_scale=_get(emb, "scale", float, "embedding.", required=False, default=1.0) if emb is not None else 1.0,
                  canon_taps=_get(canon, "taps", int, "canon.") if canon is not None else None,
                  layers=tuple(layers), raw=copy.deepcopy(d))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        if self.raw:
            return copy.deepcopy(self.raw)
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "layers": []}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        for layer in self.layers:
            m = layer.mixer
            if layer.kind == "parallel":
                l, r = m.left, m.right
                left = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale}
                if l.conv is not None:
                    left["conv"] = l.conv
                if l.softcap is not None:
                    left["softcap"] = l.softcap
                if l.rot_dims:
                    left["rot"] = {"base": l.rot_base, "dims": l.rot_dims}
                if l.chunk is not None:
                    left["mask"] = {"size": l.chunk}
                mixer = {"left": left, "left_scale": m.left_scale, "right_scale": m.right_scale,
                         "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "decay": list(r.decay)}}
            elif layer.kind == "mingru":
                mixer = {"width": m.width}
            else:
                mixer = {"heads": m.heads, "dim": m.dim}
            entry = {"type": layer.kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff is not None else None}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            d["layers"].append(entry)
        return d

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Dulotar `vocab` and `width` must be greater than zero")
        if self.norm_eps <= 0.0:
            raise ConfigError("Dulotar `norm.eps` must be positive")
        if self.canon_taps is not None and not 1 <= self.canon_taps <= 16:
            raise ConfigError("Dulotar `canon.taps` must lie in 1..16")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.kind == "parallel":
                l, r = m.left, m.right
                if min(l.heads, l.kv_heads, l.dim, l.vdim) <= 0 or l.heads % l.kv_heads:
                    raise ConfigError(f"Dulotar layer {i}: left.heads must be a positive multiple of left.kv_heads, dim and vdim positive")
                if l.rot_dims % 2 or l.rot_dims > l.dim:
                    raise ConfigError(f"Dulotar layer {i}: left.rot.dims ({l.rot_dims}) must be even and within dim ({l.dim})")
                if (l.rot_dims and l.rot_base <= 0.0) or l.scale <= 0.0:
                    raise ConfigError(f"Dulotar layer {i}: left.rot.base and left.scale must be positive")
                if l.chunk is not None and l.chunk <= 0:
                    raise ConfigError(f"Dulotar layer {i}: left.mask.size must be positive")
                if l.conv is not None and not 1 <= l.conv <= 16:
                    raise ConfigError(f"Dulotar layer {i}: left.conv must lie in 1..16")
                if l.softcap is not None and l.softcap <= 0.0:
                    raise ConfigError(f"Dulotar layer {i}: left.softcap must be positive")
                if min(r.heads, r.dim, r.vdim) <= 0 or len(r.decay) != r.heads:
                    raise ConfigError(f"Dulotar layer {i}: right needs positive sizes and one decay a head")
                if not all(0.0 <= x <= 1.0 for x in r.decay):
                    raise ConfigError(f"Dulotar layer {i}: right.decay must lie in 0..1")
            elif layer.kind == "mingru":
                if m.width <= 0:
                    raise ConfigError(f"Dulotar layer {i}: mixer.width must be greater than zero")
            elif min(m.heads, m.dim) <= 0:
                raise ConfigError(f"Dulotar layer {i}: heads and dim must be greater than zero")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"Dulotar layer {i}: mlp.ff must be greater than zero")
            j = layer.weights_of
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].weights_of is not None:
                    raise ConfigError(f"Dulotar layer {i}: weights_of must name another layer that has tensors of its own")
                other = self.layers[j]
                if (other.kind, other.mixer, other.ff) != (layer.kind, layer.mixer, layer.ff):
                    raise ConfigError(f"Dulotar layer {i}: a layer that runs with layer {j}'s weights must equal it in every size")

    # ---- the model as data --------------------------------------------------

    def to_model_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name):
            return NormSpec(w, eps, name, "layernorm")

        layers, index_of = [], {}
        for i, layer in enumerate(self.layers):
            if layer.weights_of is not None:
                continue
            p, m = f"l{i}.", layer.mixer
            if layer.kind == "parallel":
                l, r = m.left, m.right
                left = GatedAttentionSpec(
                    hidden_size=w, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim, value_dim=l.vdim,
                    position=RotarySpec(l.rot_dims, l.rot_base, ROTATION_PAIRING) if l.rot_dims else None, scale=l.scale,
                    chunk=l.chunk, window=None, bias=False, out_gate=False, prefix=p + "mix.left.", conv_taps=l.conv,
                    softcap=l.softcap, out_scale=m.left_scale)
                right = LightningAttentionSpec(hidden_size=w, heads=r.heads, head_dim=r.dim, value_dim=r.vdim, decays=r.decay,
                                               norm_eps=eps, out_scale=m.right_scale, prefix=p + "mix.right.")
                mixer = ParallelMixersSpec(left, right, prefix=p + "mix.")
            elif layer.kind == "mingru":
                mixer = MinGRUSpec(w, m.width, prefix=p + "mix.")
            else:
                mixer = TimeMixSpec(w, m.heads, m.dim, decay_rank=None, norm_eps=eps, prefix=p + "mix.")
            ffn = DenseFeedForwardSpec(w, layer.ff, FFN_ACTIVATION, p + "mlp.") if layer.ff is not None else None
            conv = ShortConvSpec(w, self.canon_taps, (p + "canon1",), residual=True) if self.canon_taps is not None else None
            index_of[i] = len(layers)
            layers.append(ConvPreNormLayerSpec(mixer_norm=norm(p + "norm1"), mixer=mixer,
                                               ffn_norm=norm(p + "norm2") if ffn is not None else None, ffn=ffn, conv=conv))
        order = tuple(LayerCall(index_of[layer.weights_of if layer.weights_of is not None else i], entry, True)
                      for entry, (i, layer) in enumerate(enumerate(self.layers)))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w, max_positions=UNLIMITED_POSITIONS,
            embedding=EmbeddingSpec(self.vocab, w, "", weight_name="embed", scale=self.embedding_scale), layers=tuple(layers),
            order=order, final_norm=norm("final.norm"), head=HeadSpec(self.vocab, w, False, "", weight_name="head"),
            eos_token_id=None)
        spec.validate()
        return spec
