"""Arrangement of a layer's parts: the pre-norm residual block.

    h = h + mixer(norm1(h)) ; h = h + ffn(norm2(h))

The residual stream `resid` is 32-bit; each part's output `delta` is added by
the next norm's fused kernel, so an add never runs alone
(crates/quantinfer-runtime/src/qwen3/mod.rs:117-138: residual :126, norm :127,
attention :128-129, add :130, norm :131-135, feed-forward and add :136-137).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, build_part, part_class, register_part
from .linear import Linear


class PreNormBlock(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime)
        self._parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        for cat, sub in (("norm", spec.mixer_norm), ("mixer", spec.mixer),
                         ("norm", spec.ffn_norm), ("ffn", spec.ffn)):
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, resid, delta, batch, cache):
        x = self.mixer_norm(resid, delta)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm(resid, a)
        return resid, self.ffn.forward(x)


class ConvPreNormBlock(Part):
    """The pre-norm block whose mixer reads the normalised stream plus a causal convolution of it over time:

        h = norm1(x) ; x = x + mixer(h + conv(h)) ; x = x + ffn(norm2(x))

    The norm's output stays 32-bit on its way into the convolution, whose last taps - 1 inputs are the block's state of
    fixed size; the convolution's output comes in the activation type. Without `conv` in the spec this is the plain
    pre-norm block; the feed-forward (with its norm) may be absent. A mixer that keeps state of fixed size beside its
    pages says so with `state_need`, which the block passes on."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.conv = build_part("conv", spec.conv, runtime) if spec.conv is not None else None
        self.ffn = build_part("ffn", spec.ffn, runtime) if spec.ffn is not None else None
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime) if spec.ffn is not None else None
        if self.conv is not None and len(spec.conv.names) != 1:
            raise ConfigError("prenorm_conv: one input filter (the mixer's)")
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.conv, self.ffn_norm, self.ffn) if p is not None)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        subs = [("norm", spec.mixer_norm), ("mixer", spec.mixer)]
        if spec.conv is not None:
            subs.append(("conv", spec.conv))
        if spec.ffn is not None:
            subs += [("norm", spec.ffn_norm), ("ffn", spec.ffn)]
        for cat, sub in subs:
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.conv.state_need() if self.conv is not None else None

    def mixer_state_need(self):
        return getattr(self.mixer, "state_need", lambda: None)()

    def forward(self, resid, delta, batch, cache):
        if self.conv is not None:
            wide = getattr(self.mixer_norm, "wide_output", False)      # a norm that can hand its result on in 32-bit does
            h = self.mixer_norm(resid, delta, out_dtype=torch.float32) if wide else self.mixer_norm(resid, delta)
            (x,), _ = self.conv.forward(h, batch, cache.block_state)
        else:
            x = self.mixer_norm(resid, delta)
        y = self.mixer.forward(x, batch, cache)
        if self.ffn is None:
            return resid, y
        return resid, self.ffn.forward(self.ffn_norm(resid, y))


class ParallelGatedBlock(Part):
    """One norm, two sublayers side by side, gated:

        h = norm(x) ; x = x + gate_m * mixer(conv_m(h)) + gate_f * ffn(conv_f(h))
        gate_k = sigmoid(h . Wg_k^T + b_k)          conv_k(h) = h + filter_k(h) over time

    The norm's output stays 32-bit: it is the input of the convolutions (whose state is 32-bit) and is
    written once more in the activation type for the gates' projection, which reads it unfiltered. The gates'
    matrices are stacked at load, so one product gives both; the two biases, the sigmoids, the products with
    the sublayers' outputs and their sum are one kernel whose 32-bit result the next norm adds to the stream.
    The input convolutions are optional (absent from the spec: h goes to the sublayers as it is); so is the
    feed-forward. The gates are what makes this block: a spec without them is refused."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.norm = build_part("norm", spec.norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime) if spec.ffn is not None else None
        self.conv = build_part("conv", spec.conv, runtime) if spec.conv is not None else None
        n_sub = 2 if self.ffn is not None else 1
        if self.conv is not None and len(spec.conv.names) != n_sub:
            raise ConfigError("parallel_gated: one input filter per sublayer")
        if spec.gate_names is not None and len(spec.gate_names) != n_sub:
            raise ConfigError("parallel_gated: one gate per sublayer")
        if spec.gate_names is None:
            raise ConfigError("parallel_gated: the spec names no gates")
        h = spec.norm.size
        self.gates = Linear(runtime, n_sub * h, h, spec.gate_names[0] + "+")
        self.gate_bias = None
        self._parts = tuple(p for p in (self.norm, self.mixer, self.ffn, self.conv) if p is not None)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        subs = [("norm", spec.norm), ("mixer", spec.mixer)]
        if spec.ffn is not None:
            subs.append(("ffn", spec.ffn))
        if spec.conv is not None:
            subs.append(("conv", spec.conv))
        for cat, sub in subs:
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        h = spec.norm.size
        for name in spec.gate_names or ():
            needs[name] = TensorNeed((h, h))
            needs[name + ".b"] = TensorNeed((h,), "matrix", "zeros")
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)
        names = self.spec.gate_names
        if names is not None:
            ws = [tensors[n] for n in names]
            if len({w.dtype for w in ws}) > 1:
                ws = [w.to(torch.float32) for w in ws]
            self.gates.load(torch.cat(ws, dim=0))
            self.gate_bias = [self._gain(tensors[n + ".b"]) for n in names]

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.conv.state_need() if self.conv is not None else None

    def forward(self, resid, delta, batch, cache):
        rt = self.runtime
        n, width = resid.shape
        two = self.ffn is not None
        if self.conv is not None:
            h = torch.empty((n, width), dtype=torch.float32, device=resid.device)
            kernels.add_rmsnorm(resid, delta, self.norm.gain, self.norm.spec.eps, h)
            ins, hb = self.conv.forward(h, batch, cache.block_state, want_copy=rt.dtype != torch.float32)
            if hb is None:
                hb = h
        else:
            hb = self.norm(resid, delta)
            ins = [hb, hb]
        y_m = self.mixer.forward(ins[0], batch, cache)
        y_f = self.ffn.forward(ins[1]) if two else None
        out = torch.empty((n, width), dtype=torch.float32, device=resid.device)
        g = self.gates(hb)
        kernels.gated_sum(g, self.gate_bias[0], self.gate_bias[1] if two else None, y_m, y_f, out)
        return resid, out


class SandwichBlock(Part):
    """A norm before AND after each sublayer, and a multiplier on what joins the stream:

        x = x + m * post1(mixer(pre1(x))) ;  x = x + m * post2(ffn(pre2(x)))

    Nothing is added by a kernel of its own: a sublayer's output travels as a :class:`PostNormed` (with its
    post-norm, the multiplier and the mixer's unapplied output bias) to the next pre-norm, in this block or the
    next one, or to the model's final norm, which does post-norm, addition and its own norm in one pass when both
    norms are elementwise (dynamic tanh). The feed-forward, with its two norms, may be absent."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.norm1 = build_part("norm", spec.mixer_norm, runtime)
        self.norm1b = build_part("norm", spec.mixer_post_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime) if spec.ffn is not None else None
        self.norm2 = build_part("norm", spec.ffn_norm, runtime) if spec.ffn is not None else None
        self.norm2b = build_part("norm", spec.ffn_post_norm, runtime) if spec.ffn is not None else None
        for n in (self.norm1b, self.norm2b):
            if n is not None and not hasattr(n, "add_into"):
                raise ConfigError("sandwich: a post-norm must be a norm that can be applied to a sublayer's output (add_into)")
        self._parts = tuple(p for p in (self.norm1, self.norm1b, self.mixer, self.norm2, self.norm2b, self.ffn) if p is not None)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        subs = [("norm", spec.mixer_norm), ("norm", spec.mixer_post_norm), ("mixer", spec.mixer)]
        if spec.ffn is not None:
            subs += [("norm", spec.ffn_norm), ("norm", spec.ffn_post_norm), ("ffn", spec.ffn)]
        for cat, sub in subs:
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, resid, delta, batch, cache):
        from .norm import PostNormed

        m = self.spec.residual_mult
        h = self.norm1(resid, delta)
        y = self.mixer.forward(h, batch, cache)
        pending = PostNormed(y, self.norm1b, m, getattr(self.mixer, "out_bias", None))
        if self.ffn is None:
            return resid, pending
        h = self.norm2(resid, pending)
        return resid, PostNormed(self.ffn.forward(h), self.norm2b, m)


class PostNormBlock(Part):
    """The block whose norms come after the sums and replace the stream:

        x = norm1(alpha * x + mixer(x)) ;  x = norm2(alpha * x + ffn(x))

    The sublayers read the stream itself. Sum, norm and the stream's copy in the activation type (what the next sublayer's
    projections read) are one kernel; the block hands that copy on to the next block as a :class:`StreamCopy`. The
    feed-forward, with its norm, may be absent. The norms must offer `renorm` (the form that replaces the stream)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.mixer_norm = build_part("norm", spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", spec.mixer, runtime)
        self.ffn = build_part("ffn", spec.ffn, runtime) if spec.ffn is not None else None
        self.ffn_norm = build_part("norm", spec.ffn_norm, runtime) if spec.ffn is not None else None
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "renorm"):
                raise ConfigError("postnorm: a norm after the sum must be able to replace the stream (renorm)")
        if hasattr(self.mixer, "keep_partials"):
            self.mixer.keep_partials = True       # the norm's kernel adds a split product's partial sums itself
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        subs = [("norm", spec.mixer_norm), ("mixer", spec.mixer)]
        if spec.ffn is not None:
            subs += [("norm", spec.ffn_norm), ("ffn", spec.ffn)]
        for cat, sub in subs:
            needs.update(part_class(cat, sub).needs_of_spec(sub))
        return needs

    def load(self, tensors):
        for p in self._parts:
            p.load(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def mixer_state_need(self):
        return getattr(self.mixer, "state_need", lambda: None)()

    def forward(self, resid, delta, batch, cache):
        from .norm import StreamCopy, settle

        if isinstance(delta, StreamCopy):
            x = delta.x
        else:
            pending = settle(resid, delta)
            if pending is not None:          # a block of another kind came before: its output joins the stream first
                kernels.scaled_sum(resid, pending, 1.0, 1.0, resid)
            if self.runtime.dtype == torch.float32:
                x = resid
            else:
                x = torch.empty(resid.shape, dtype=self.runtime.dtype, device=resid.device)
                kernels.convert(resid, x)
        x = self.mixer_norm.renorm(resid, self.mixer.forward(x, batch, cache), self.spec.alpha)
        if self.ffn is not None:
            x = self.ffn_norm.renorm(resid, self.ffn.forward(x), self.spec.alpha)
        return resid, StreamCopy(x)


register_part("block", "postnorm", PostNormBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "prenorm_conv", ConvPreNormBlock)
register_part("block", "parallel_gated", ParallelGatedBlock)
