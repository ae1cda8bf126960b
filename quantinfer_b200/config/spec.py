"""Descriptions of a model as data: parts with their sizes and constants, the
layers they form, and the order in which layers run.

An architecture's config class turns its config.json into a :class:`ModelSpec`.
Nothing below the spec knows which architecture it came from: parts are built
from their spec alone (`parts.registry.build_*`). The reference keeps the same
split between a config and an architecture-neutral description
(crates/quantinfer-model/src/semantic.rs:39-57,91-103: per-layer attention,
normalisation, activation and positional specs).

Each spec carries `kind`, the key under which the part's class is registered,
and `prefix`, prepended to the part's local tensor names to give the names in
the weight files.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    """`kind` "rmsnorm": gain per coordinate, tensor `prefix + "weight"`. "rmsnorm_scalar": one gain for all
    coordinates, the tensor named `prefix` itself, of shape []. "dyt": dynamic tanh, tanh(alpha x) w + b with no
    statistic of the row (eps unused): w is the tensor named `prefix` itself, b `prefix + ".b"`, alpha
    `prefix + ".alpha"` of shape []. "layernorm": (x - mean) / sqrt(variance + eps) * w + b with the variance the mean
    squared deviation; w is the tensor named `prefix` itself, b `prefix + ".b"`."""

    size: int
    eps: float
    prefix: str = ""
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding over the first `rotary_dim` dimensions of each head, angle of pair p =
    position * theta^(-2p / rotary_dim). `pairing` says which two elements pair p is:
    "half_split" (p, p + rotary_dim / 2) or "interleaved" (2p, 2p + 1)."""

    head_dim: int
    rotary_dim: int
    theta: float
    max_positions: int
    kind: str = "rope_half_split"
    pairing: str = "half_split"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over a paged key/value cache."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec]
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None      # None: all earlier keys; n: the last n keys
    scale: Optional[float] = None     # None: head_dim ** -0.5
    prefix: str = ""
    kind: str = "attention"


@dataclass(frozen=True)
class FeedForwardSpec:
    """Gated feed-forward: down(act(gate(x)) * up(x))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    prefix: str = ""
    kind: str = "gated_mlp"
    names: Optional[tuple] = None     # (gate, up, down) tensor names after the prefix; None: the *_proj.weight names


@dataclass(frozen=True)
class RotarySpec:
    """Rotary encoding whose angles are computed where they are used (no table, so no limit on
    positions): pair i of the first `rotary_dim` coordinates of a part turns by position *
    theta^(-2i / rotary_dim). `pairing` as for :class:`PositionSpec`."""

    rotary_dim: int
    theta: float
    pairing: str = "interleaved"
    kind: str = "rope_direct"
    stretch: Optional[tuple] = None   # (factor, original, fast, slow): pairs that turn fewer than `slow` times over
                                      # `original` positions have their frequency divided by `factor`, pairs that turn
                                      # more than `fast` times keep it, a linear ramp over the pair's number lies
                                      # between (YaRN); cos and sin are then multiplied by 0.1 ln(factor) + 1


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention over a cached low-rank latent: a position caches `kv_rank` numbers (normalised,
    gain per coordinate) and a rotated key part of `rot_dim` numbers that all heads share; per head the
    key's plain part (`head_dim` numbers) and the value (`value_dim`) are projections of the latent.
    `shares_latent`: the layer has no latent projection and reads the cache entry of another layer.
    `sink`: the softmax's denominator holds one more learned term per head."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    value_dim: int
    kv_rank: int
    position: Optional[RotarySpec]
    norm_eps: float
    scale: float
    window: Optional[int] = None
    sink: bool = False
    shares_latent: bool = False
    prefix: str = ""
    kind: str = "latent_attention"
    out_gate: bool = False            # the concatenated heads are multiplied by sigmoid(W_g x) (`g`) before the output projection


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    """Feed-forward without a gate: down(act(up(x)))."""

    hidden_size: int
    intermediate_size: int
    activation: str = "gelu_tanh"
    prefix: str = ""
    kind: str = "dense_mlp"


@dataclass(frozen=True)
class ShortConvSpec:
    """A bank of short causal convolutions over time that read one input: filter k has `taps` weights per
    channel, stored as the tensor `names[k]` of shape [width, taps]; out_k = (input if `residual`) +
    filter_k(input). The last taps - 1 inputs are a request's state."""

    width: int
    taps: int
    names: tuple
    residual: bool = True
    kind: str = "short_conv"


@dataclass(frozen=True)
class ParallelLayerSpec:
    """One block with one norm whose output feeds the mixer and the feed-forward side by side:
    h = norm(x); x += gate_m * mixer(conv_m(h)) + gate_f * ffn(conv_f(h)). `conv` (optional) is the bank
    of input convolutions, one filter per sublayer; `gate_names` (optional) are the prefixes of the sigmoid
    gates' projections of h, one per sublayer ("<name>" the matrix, "<name>.b" the bias). `ffn` may be None."""

    norm: NormSpec
    mixer: object
    ffn: object
    conv: Optional[ShortConvSpec] = None
    gate_names: Optional[tuple] = None
    kind: str = "parallel_gated"

    # what the model reads of any layer spec
    @property
    def mixer_norm(self):
        return self.norm


@dataclass(frozen=True)
class BigramEmbeddingSpec:
    """Token embedding plus a row of a hashed bigram table [buckets + 1, hidden]: row (previous * mul_prev +
    current * mul_cur) mod buckets, the last row for a sequence's first token."""

    vocab_size: int
    hidden_size: int
    buckets: int
    mul_prev: int
    mul_cur: int
    table_name: str = "embed"
    bigram_name: str = "bigram"
    prefix: str = ""
    kind: str = "bigram_embedding"


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Causal grouped-query attention whose projections have biases (q, k, v and the output; tensors `q`, `k`,
    `v`, `o`, each with `.b`), whose values may have another size than its keys, and whose concatenated heads are
    multiplied by sigmoid(W_g x) (`g`, when `out_gate`) before the output projection. `chunk`: a query sees only
    the keys of its own chunk of that many positions, counted from the sequence's start; `window`: the last n keys;
    both None: every earlier key. `position`: a :class:`RotarySpec` over the first coordinates of each head, or None."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    position: Optional[RotarySpec]
    scale: float
    chunk: Optional[int] = None
    window: Optional[int] = None
    bias: bool = True
    out_gate: bool = True
    prefix: str = ""
    kind: str = "gated_attention"
    conv_taps: Optional[int] = None    # n: q, k and v each pass a causal convolution of n taps per channel right after their
                                       # projection (tensors `q.conv`, `k.conv`, `v.conv` [channels, n], no bias); the last
                                       # n - 1 projected rows are a request's state
    softcap: Optional[float] = None    # c: a score s becomes c tanh(s / c) before the softmax
    out_scale: float = 1.0             # a factor on what the mixer hands on (applied before the output projection)
    sink: Optional[str] = None         # the softmax's denominator holds one more term exp(b_h) a head, with no key and no
                                       # value: "zero": b_h = 0 (one is added); "learned": b is the tensor `sink` [heads]
    values_from_keys: bool = False     # there is no `v`: a position's value is its key as projected (before any norm and
                                       # rotation), so value_dim equals head_dim
    qk_norm: Optional[str] = None      # "whole": q (all heads at once) and k (likewise) each pass one RMS norm over the whole
                                       # projection before the rotation, gains `q.norm` [heads head_dim], `k.norm`
    qk_norm_eps: float = 1e-6


@dataclass(frozen=True)
class MinGRUSpec:
    """A gated recurrence per channel whose gates read only the current token: z = sigmoid(W_z x + b_z),
    u = W_x x + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u) below; S_t = (1 - z) S_(t-1) + z c;
    out = W_o (S_t * silu(W_g x)). Tensors `z`, `z.b`, `x`, `x.b`, `g`, `o` after the prefix; S is 32-bit state."""

    hidden_size: int
    width: int
    prefix: str = ""
    kind: str = "mingru"


@dataclass(frozen=True)
class TimeMixSpec:
    """Time mixing over a matrix state per head with a decay per head and key channel (RWKV style). Each of r, k, v,
    g, w reads its own mix of the token's input with its predecessor's, x + (x' - x) mu_s (`mu.r` ...); r, k, v are
    projections of theirs to `heads` x `head_dim`; gate = silu(W_g mix_g); decay = exp(-exp(W_w2 tanh(W_w1 mix_w) +
    w0)) (`w1` [rank, hidden], `w2` [heads head_dim, rank], `w0`); o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t (`u`
    [heads, head_dim]); S_t = diag(decay_t) S_(t-1) + k_t v_t^T; every head's o over its root mean square, times
    `norm`, times the gate, W_o. The state (32-bit) is S and the predecessor's input."""

    hidden_size: int
    heads: int
    head_dim: int
    decay_rank: int
    norm_eps: float
    prefix: str = ""
    kind: str = "time_mix"


@dataclass(frozen=True)
class LightningAttentionSpec:
    """Linear attention over a matrix state per head with one constant decay a head: q = silu(W_q x), k = silu(W_k x)
    (`heads` x `head_dim`), v = silu(W_v x) (`heads` x `value_dim`); S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t;
    the concatenated heads pass one RMS norm with gain (`norm`), times sigmoid(W_g x), W_o. `out_scale`: a factor on
    what the mixer hands on (applied before the output projection)."""

    hidden_size: int
    heads: int
    head_dim: int
    value_dim: int
    decays: tuple
    norm_eps: float
    out_scale: float = 1.0
    prefix: str = ""
    kind: str = "lightning_attention"


@dataclass(frozen=True)
class ParallelMixersSpec:
    """Two mixers side by side that read the same input; their outputs are added. Each branch's own factor is a field of
    its spec (`out_scale`). At most one branch keeps pages; every other state is of fixed size. `out_norm_names`
    (left, right): each branch's output first passes an RMS norm over the model width with the gain of that name (eps
    `out_norm_eps`); `sum_scale` multiplies the sum."""

    left: object
    right: object
    prefix: str = ""
    kind: str = "parallel_mixers"
    out_norm_names: Optional[tuple] = None
    out_norm_eps: float = 1e-6
    sum_scale: float = 1.0
    hidden_size: Optional[int] = None  # needed with `out_norm_names` (the gains' size)


@dataclass(frozen=True)
class GatedDeltaSpec:
    """A matrix state per head that is decayed per key channel and corrected towards each token's value (gated delta
    rule). q, k = projections to `kv_heads` x `head_dim`, v to `heads` x `value_dim` (head h reads q/k head
    floor(h / (heads / kv_heads))); each passes a causal convolution of `conv_taps` taps per channel (`q.conv` ...,
    no bias) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + `unit_eps`)), q times head_dim^(-1/2);
    beta = sigmoid(W_b x) a head; decay = exp(-exp(A_log_h) softplus(W_a2 W_a1 x + dt_bias)) per head and key
    channel; S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; every head's o over its root mean
    square (eps `norm_eps`) times `norm` [value_dim] times sigmoid(W_g2 W_g1 x); W_o. The ranks of the two low-rank
    pairs are read from `a1` and `g1`. State (32-bit): S, and the convolutions' last taps - 1 inputs."""

    hidden_size: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    conv_taps: int
    norm_eps: float
    unit_eps: float = 1e-6
    prefix: str = ""
    kind: str = "gated_delta"


@dataclass(frozen=True)
class PostNormLayerSpec:
    """The block whose norms come after the sums: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ffn(x)). The
    sublayers read the stream itself. `ffn` (with its norm) may be None."""

    mixer_norm: NormSpec
    mixer: object
    ffn_norm: Optional[NormSpec]
    ffn: object
    alpha: float = 1.0
    kind: str = "postnorm"


@dataclass(frozen=True)
class ConvPreNormLayerSpec:
    """The pre-norm block whose mixer reads h + conv(h) instead of h = norm1(x): x += mixer(h + conv(h));
    x += ffn(norm2(x)). `conv` None: the plain pre-norm block; `ffn` (with its norm) may be None."""

    mixer_norm: NormSpec
    mixer: object
    ffn_norm: Optional[NormSpec]
    ffn: object
    conv: Optional[ShortConvSpec] = None
    kind: str = "prenorm_conv"


@dataclass(frozen=True)
class StateSpaceSpec:
    """A selective state-space mixer with one decay a head: `heads` heads of `head_dim` channels, a state of
    `state` x `head_dim` numbers a head, B and C shared by the heads of a group (`groups`), an input convolution of
    `conv_taps` taps with bias and silu over x | B | C, the gate silu(z) before an RMS norm in `norm_groups` equal
    parts. Tensors after the prefix: `in` [2 inner + 2 groups state + heads, hidden], `conv` [channels, taps],
    `conv.b`, `dt_bias`, `A_log`, `D` [heads], `norm` [inner], `o` [hidden, inner]."""

    hidden_size: int
    heads: int
    head_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    prefix: str = ""
    kind: str = "mamba2"


@dataclass(frozen=True)
class ClampedGLUSpec:
    """Feed-forward down(g sigmoid(alpha g) (u + 1)) with g = min(gate(x), limit), u = clamp(up(x), -limit, limit);
    no biases; tensors `gate`, `up`, `down` after the prefix."""

    hidden_size: int
    intermediate_size: int
    limit: float
    alpha: float = 1.702
    prefix: str = ""
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class MoESpec:
    """Mixture of `experts` small feed-forwards of the :class:`ClampedGLUSpec` form (`e<k>.gate` and so on), of which
    a token uses `top`: scores = softmax of the router's logits over all experts (32-bit); the choice is by score +
    `correction`, the weights are the chosen scores over their sum (+ 1e-20) times `router_scale`. `shared`
    (optional) runs for every token and is added."""

    hidden_size: int
    experts: int
    top: int
    router_scale: float
    expert: ClampedGLUSpec            # its prefix is the feed-forward's; expert k's tensors follow `e<k>.`
    shared: Optional[ClampedGLUSpec] = None
    prefix: str = ""
    kind: str = "moe"


@dataclass(frozen=True)
class SandwichLayerSpec:
    """One block with a norm before AND after each sublayer and a multiplier on what joins the stream:
    x += m * post1(mixer(pre1(x))); x += m * post2(ffn(pre2(x))). `ffn` (with its norms) may be None."""

    mixer_norm: NormSpec
    mixer_post_norm: NormSpec
    mixer: object
    ffn_norm: Optional[NormSpec]
    ffn_post_norm: Optional[NormSpec]
    ffn: object
    residual_mult: float = 1.0
    kind: str = "sandwich"


@dataclass(frozen=True)
class ReentrySpec:
    """What a pass of a looped stretch of layers begins with: x <- W [x ; x0], x0 the embedding's output,
    W the tensor `weight_name` [hidden, 2 hidden]."""

    hidden_size: int
    weight_name: str
    kind: str = "concat_proj"


@dataclass(frozen=True)
class LayerSpec:
    """One block: x += mixer(norm(x)); x += ffn(norm(x)) for kind `prenorm`."""

    mixer_norm: NormSpec
    mixer: object          # a mixer spec (AttentionSpec or any registered kind)
    ffn_norm: NormSpec
    ffn: object            # a feed-forward spec
    kind: str = "prenorm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache entry `cache`.

    Naming a layer twice reuses its weights. `writes_cache=False` makes the
    call read a cache entry that an earlier call filled, without adding to it.
    """

    layer: int
    cache: int
    writes_cache: bool = True
    reenter: bool = False      # the model's re-entry part (ModelSpec.reentry) runs right before this call


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    prefix: str = ""
    kind: str = "embedding"
    weight_name: Optional[str] = None   # the tensor's full name when it is not prefix + "weight"
    scale: float = 1.0                  # the row is multiplied by this (32-bit) on its way into the stream


@dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int
    tied: bool              # True: the head is the embedding table
    prefix: str = ""
    kind: str = "lm_head"
    softcap: Optional[float] = None     # c: logits = c * tanh(logits / c)
    weight_name: Optional[str] = None   # the tensor's full name when it is not prefix + "weight"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: tuple
    order: tuple
    final_norm: NormSpec
    head: HeadSpec
    eos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)
    reentry: Optional[ReentrySpec] = None

    def cache_entries(self) -> int:
        return 1 + max(call.cache for call in self.order) if self.order else 0

    def validate(self) -> None:
        from ..errors import ConfigError

        if not self.layers or not self.order:
            raise ConfigError("a model needs at least one layer and one entry in its run order")
        written = set()
        for i, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {call.layer}, the model has {len(self.layers)}")
            if call.cache < 0:
                raise ConfigError(f"run order entry {i} has a negative cache entry")
            if call.reenter and self.reentry is None:
                raise ConfigError(f"run order entry {i} re-enters, but the model has no re-entry part")
            if call.writes_cache:
                if call.cache in written:
                    raise ConfigError(f"run order entry {i}: cache entry {call.cache} already has a writer")
                written.add(call.cache)
            elif call.cache not in written:
                raise ConfigError(f"run order entry {i} reads cache entry {call.cache} before any layer wrote it")
        if written != set(range(self.cache_entries())):
            raise ConfigError("cache entries must be numbered 0..n-1 and each needs a writer")
