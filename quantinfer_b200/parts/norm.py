"""RMSNorm with the residual add fused in.

    x = resid + delta ; resid = x ; out = (x / sqrt(mean(x^2) + eps)) * gain

The gain multiplies as stored (no `1 + g`), and one eps serves every norm of
the model, as in the reference (backends/cpu/src/backend.rs:172-193; placement
crates/quantinfer-runtime/src/qwen3/mod.rs:127,131-135,370-372). Sums are 32-bit.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorNeed
from .base import Part, register_part


def sum_partials(delta, dtype=None):
    """`delta` as one [tokens, hidden] tensor: the K-split partial sums [splits, tokens, hidden]
    of a projection added in split order (32-bit), or `delta` itself when it is already whole.
    For norms that have no kernel that adds the partial sums itself."""
    if delta is None or delta.dim() == 2:
        return delta
    total = delta[0].clone()
    for k in range(1, delta.shape[0]):
        total += delta[k]
    return total if dtype is None else total.to(dtype)


class PostNormed:
    """A sublayer's output that has not joined the residual stream yet: the stream is to receive
    `mult * post(y + bias)`, `post` a norm applied AFTER the sublayer (None: y + bias as it is). A block hands
    this on as its `delta`, so that the next norm's kernel does the post-norm, the addition and its own norm in one
    pass; `apply` does the addition alone, for whoever cannot fuse it."""

    def __init__(self, y, post=None, mult: float = 1.0, bias=None):
        self.y, self.post, self.mult, self.bias = y, post, mult, bias

    def apply(self, resid):
        """resid += mult * post(y + bias); returns None (nothing is pending any more)."""
        if self.post is not None:
            self.post.add_into(resid, self.y, self.bias, self.mult)
        else:
            kernels.dyt(resid, self.y, self.bias)
        return None


class StreamCopy:
    """Nothing is pending: the stream is up to date, and `x` is the stream once more in the activation type, as the
    norm that wrote the stream last left it beside it, for whoever reads the stream next."""

    def __init__(self, x):
        self.x = x

    def apply(self, resid):
        return None


def settle(resid, delta):
    """`delta` as something every norm takes: a pending :class:`PostNormed` is added to the stream now; a
    :class:`StreamCopy` has nothing to add."""
    return delta.apply(resid) if isinstance(delta, (PostNormed, StreamCopy)) else delta


class RMSNorm(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.gain = None

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix + "weight": TensorNeed((spec.size,), "gain", "gain")}

    def load(self, tensors):
        self.gain = self._gain(tensors[self.spec.prefix + "weight"])

    def forward(self, resid, delta, rows=None, write_resid=True):
        delta = settle(resid, delta)
        n = resid.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        kernels.add_rmsnorm(resid, delta, self.gain, self.spec.eps, out, rows=rows, write_resid=write_resid)
        return out

    __call__ = forward


class OnePlusRMSNorm(RMSNorm):
    """RMS norm whose weight is stored around zero: out = x / sqrt(mean(x^2) + eps) * (1 + w), w the tensor named by the
    spec's `prefix` itself. 1 + w is formed once, in 32-bit, at load. Besides the pre-norm form of every norm it offers
    the form that comes AFTER a sum and replaces the stream (`renorm`)."""

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix: TensorNeed((spec.size,), "gain", "zeros")}

    def load(self, tensors):
        self.gain = self._gain(tensors[self.spec.prefix].to(torch.float32) + 1.0)

    def renorm(self, resid, delta, alpha: float):
        """resid <- norm(alpha * resid + delta), in place and in 32-bit; returns the new stream in the activation type
        (the stream itself when that type is float32)."""
        delta = settle(resid, delta)
        copy = None if self.runtime.dtype == torch.float32 else torch.empty(resid.shape, dtype=self.runtime.dtype, device=resid.device)
        kernels.scale_add_rmsnorm(resid, delta, alpha, self.gain, self.spec.eps, copy)
        return resid if copy is None else copy


class ScalarRMSNorm(RMSNorm):
    """RMS norm whose gain is ONE number for all coordinates, stored as a tensor of shape [] under the
    spec's `prefix` itself. The number is spread over a gain vector at load, so the fused kernels of the
    per-coordinate norm serve it unchanged."""

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix: TensorNeed((), "gain", "gain")}

    def load(self, tensors):
        g = tensors[self.spec.prefix].to(torch.float32).reshape(1)
        self.gain = self._gain(g.expand(self.spec.size))


class DynamicTanh(Part):
    """Dynamic tanh in the place of a norm: out = tanh(alpha x) w + b, elementwise, with no mean or variance of the
    row (the spec's eps is unused). w is the tensor named by the spec's `prefix` itself, b `prefix.b`, alpha
    `prefix.alpha` of shape []; all are used in 32-bit, alpha from device memory. Being elementwise, it fuses with
    everything around it: as a pre-norm it takes the pending output of the sublayer before it (`delta`, plain or a
    :class:`PostNormed` with ITS post-norm, multiplier and unapplied bias), adds it to the stream and normalises the
    result in one launch; as a post-norm it is applied by whoever consumes the `PostNormed` that names it."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.w = self.b = self.alpha = None

    @classmethod
    def needs_of_spec(cls, spec):
        p = spec.prefix
        return {p: TensorNeed((spec.size,), "gain", "gain"), p + ".b": TensorNeed((spec.size,), "gain", "zeros"),
                p + ".alpha": TensorNeed((), "gain", "gain")}

    def load(self, tensors):
        p = self.spec.prefix
        self.w, self.b = self._gain(tensors[p]), self._gain(tensors[p + ".b"])
        self.alpha = self._gain(tensors[p + ".alpha"].reshape(1))

    def params(self):
        return (self.w, self.b, self.alpha)

    def add_into(self, resid, y, bias=None, mult: float = 1.0):
        """resid += mult * dyt(y + bias)."""
        kernels.dyt(resid, y, bias, post=self.params(), mult=mult)

    def forward(self, resid, delta, rows=None, write_resid=True):
        n = resid.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        y = bias = post = None
        mult = 1.0
        if isinstance(delta, PostNormed):
            if delta.post is not None and not isinstance(delta.post, DynamicTanh):
                delta = delta.apply(resid)        # a post-norm of another kind cannot ride in this kernel
            else:
                y, bias, mult = delta.y, delta.bias, delta.mult
                post = delta.post.params() if delta.post is not None else None
        if delta is not None and not isinstance(delta, PostNormed):
            y = delta
        kernels.dyt(resid, y, bias, post=post, mult=mult, pre=self.params(), out=out, rows=rows,
                    write_resid=write_resid and rows is None)
        return out

    __call__ = forward


class LayerNorm(Part):
    """Layer norm with gain and bias, the residual add fused in: x = resid + delta; out = (x - mean) / sqrt(var + eps) * w
    + b, var the mean squared deviation (two 32-bit sums over the row). w is the tensor named by the spec's `prefix`
    itself, b `prefix.b`. `out_dtype` float32 keeps the result in 32-bit for a consumer that wants it so (an input
    convolution whose state is 32-bit)."""

    wide_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.gain = self.bias = None

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix: TensorNeed((spec.size,), "gain", "gain"), spec.prefix + ".b": TensorNeed((spec.size,), "gain", "zeros")}

    def load(self, tensors):
        self.gain, self.bias = self._gain(tensors[self.spec.prefix]), self._gain(tensors[self.spec.prefix + ".b"])

    def forward(self, resid, delta, rows=None, write_resid=True, out_dtype=None):
        delta = settle(resid, delta)
        n = resid.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=out_dtype or self.runtime.dtype, device=resid.device)
        kernels.add_layernorm(resid, delta, self.gain, self.bias, self.spec.eps, out, rows=rows, write_resid=write_resid)
        return out

    __call__ = forward


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "dyt", DynamicTanh)
register_part("norm", "rmsnorm_scalar", ScalarRMSNorm)
register_part("norm", "rmsnorm_one_plus", OnePlusRMSNorm)
