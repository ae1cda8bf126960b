"""Causal grouped-query attention with biased projections, an output gate and chunks.

    [q | k | v | g] = x . W^T                 (the four projections stacked at load: one product)
    q | k | v       = conv(q | k | v)         (optional: a causal convolution over time per channel, `conv_taps` taps)
    q, k            = rotate(q + b_q, p), rotate(k + b_k, p)      over the first `rotary_dim` coordinates of a head
    cache[p]        = (k, v + b_v)            values may have another size than keys
    a               = softmax(cap(q k^T * scale) over the visible keys) v          cap(s) = c tanh(s / c), optional
    y               = (a * sigmoid(g) * out_scale) . Wo^T (+ b_o)

Biases, the gate, the convolution, the cap and the factor are each optional (fields of the spec). So are: a sink (the
softmax's denominator holds exp(b_h) once more, b zero or the learned tensor `sink`); one RMS norm over the whole of q
and one over the whole of k before the rotation (`q.norm`, `k.norm`); values that are the keys as projected, before
norm and rotation (no `v` then). The convolution's
last taps - 1 projected rows are the mixer's state of fixed size BESIDE its pages (`state_need`, handed back as
`cache.mixer_state`).

Visible keys of the query at position i: j <= i, within the last `window` positions if the spec has a window, and
within i's own chunk (floor(i / chunk) = floor(j / chunk), chunks counted from the sequence's first position, not
from where a step began) if it has chunks. The cache need carries both, so pages of chunks a request has left go
back to the pool at once.

The biases of q, k and v are added where the projection's row is read next (the rotation and cache-write kernel);
the gate is applied where the attention's result is written; the output projection's bias is left unapplied and
offered as `out_bias`, which a block's next norm adds in its own pass. Angles are computed where they are used,
position * theta^(-2i / rotary_dim) in 32-bit: no table, no limit on positions.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import PagedKVNeed, StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class GatedAttention(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} kv heads")
        for name, v in (("window", s.window), ("chunk", s.chunk)):
            if v is not None and v <= 0:
                raise ConfigError(f"gated_attention: {name} must be positive or None")
        self.H, self.G, self.d, self.dv = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        self.v_from_k = bool(getattr(s, "values_from_keys", False))
        self.sink_kind, self.qk_norm = getattr(s, "sink", None), getattr(s, "qk_norm", None)
        if self.v_from_k and (self.dv != self.d or getattr(s, "conv_taps", None) is not None or s.bias):
            raise ConfigError("gated_attention: values that are the keys have the keys' size, no bias and no convolution")
        if self.sink_kind not in (None, "zero", "learned") or self.qk_norm not in (None, "whole"):
            raise ConfigError(f"gated_attention: sink {self.sink_kind!r} / qk_norm {self.qk_norm!r} are not known")
        self.sink = self.q_gain = self.k_gain = None
        self.qkv_cols = (self.H + self.G) * self.d + (0 if self.v_from_k else self.G * self.dv)
        self.proj = Linear(runtime, self.qkv_cols + (self.H * self.dv if s.out_gate else 0), s.hidden_size, s.prefix + "q+k+v+g")
        if self.sink_kind == "zero":
            self.sink = torch.zeros(self.H, dtype=torch.float32, device=runtime.device)
        self.o = Linear(runtime, s.hidden_size, self.H * self.dv, s.prefix + "o")
        self.bias = self.out_bias = self.inv_freq = self.conv_w = None
        self.taps = getattr(s, "conv_taps", None)
        if self.taps is not None and not 1 <= self.taps <= 16:
            raise ConfigError(f"gated_attention: a convolution of {self.taps} taps (1..16)")
        pos = s.position
        self.rot = pos.rotary_dim if pos is not None else 0
        self.interleaved = pos is not None and pos.pairing == "interleaved"
        if pos is not None:
            if pos.pairing not in ("half_split", "interleaved") or pos.rotary_dim % 2 or not 0 < pos.rotary_dim <= s.head_dim:
                raise ConfigError(f"gated_attention: a rotation over {pos.rotary_dim} of {s.head_dim} coordinates ({pos.pairing})")
            exponent = (2.0 * torch.arange(self.rot // 2, dtype=torch.float64)) / float(self.rot)
            self.inv_freq = torch.pow(torch.tensor(float(pos.theta), dtype=torch.float64), -exponent).to(torch.float32).to(runtime.device)

    @classmethod
    def needs_of_spec(cls, s):
        p, H, G, d, dv, w = s.prefix, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.hidden_size
        needs = {p + "q": TensorNeed((H * d, w)), p + "k": TensorNeed((G * d, w))}
        if not getattr(s, "values_from_keys", False):
            needs[p + "v"] = TensorNeed((G * dv, w))
        if getattr(s, "qk_norm", None) == "whole":
            needs.update({p + "q.norm": TensorNeed((H * d,), "gain", "gain"), p + "k.norm": TensorNeed((G * d,), "gain", "gain")})
        if getattr(s, "sink", None) == "learned":
            needs[p + "sink"] = TensorNeed((H,), "gain", "normal")
        if s.out_gate:
            needs[p + "g"] = TensorNeed((H * dv, w))
        needs[p + "o"] = TensorNeed((w, H * dv))
        if getattr(s, "conv_taps", None) is not None:
            needs.update({p + "q.conv": TensorNeed((H * d, s.conv_taps)), p + "k.conv": TensorNeed((G * d, s.conv_taps)),
                          p + "v.conv": TensorNeed((G * dv, s.conv_taps))})
        if s.bias:
            needs.update({p + "q.b": TensorNeed((H * d,), "matrix", "zeros"), p + "k.b": TensorNeed((G * d,), "matrix", "zeros"),
                          p + "v.b": TensorNeed((G * dv,), "matrix", "zeros"), p + "o.b": TensorNeed((w,), "matrix", "zeros")})
        return needs

    def load(self, tensors):
        p, s = self.spec.prefix, self.spec
        ws = [tensors[p + n] for n in ("q", "k") + (() if self.v_from_k else ("v",)) + (("g",) if s.out_gate else ())]
        if self.qk_norm == "whole":
            self.q_gain, self.k_gain = self._gain(tensors[p + "q.norm"]), self._gain(tensors[p + "k.norm"])
        if self.sink_kind == "learned":
            self.sink = self._gain(tensors[p + "sink"])
        if len({t.dtype for t in ws}) > 1:
            ws = [t.to(torch.float32) for t in ws]
        self.proj.load(torch.cat(ws, dim=0))
        self.o.load(tensors[p + "o"])
        if self.taps is not None:
            w = torch.cat([tensors[p + n + ".conv"].to(torch.float32) for n in ("q", "k", "v")], dim=0)
            self.conv_w = self._gain(w.t().unsqueeze(0))          # [1, taps, q | k | v channels]
        if s.bias:
            self.bias = self._gain(torch.cat([tensors[p + n + ".b"].to(torch.float32) for n in ("q", "k", "v")]))
            self.out_bias = self._gain(tensors[p + "o.b"])

    def cache_need(self):
        return PagedKVNeed(self.G, self.d, self.spec.window, self.dv if self.dv != self.d else None, self.spec.chunk)

    def state_need(self):
        """The convolution's state: the last taps - 1 rows of q | k | v as projected (32-bit), beside the pages."""
        if self.taps is None or self.taps < 2:
            return None
        return StateNeed((self.taps - 1, self.qkv_cols), torch.float32)

    def forward(self, x, batch, cache):
        rt, s = self.runtime, self.spec
        n = x.shape[0]
        table = batch.block_tables[cache.group]
        proj = self.proj(x)
        if self.taps is not None:
            conved = torch.empty((n, self.qkv_cols), dtype=x.dtype, device=x.device)
            kernels.short_conv(proj[:, :self.qkv_cols], self.conv_w, cache.mixer_state, [conved], None, batch.token_req, batch.q_start,
                               batch.start_pos, batch.slot_ids, residual=False)
            gate_src, proj = proj, conved
        else:
            gate_src = proj
        q = torch.empty((n, self.H * self.d), dtype=x.dtype, device=x.device)
        kernels.bias_rope_kv(proj, self.bias, q, self.inv_freq, self.rot, self.interleaved, batch.positions, batch.token_req,
                             table, cache.page_size, cache.k_pages if cache.writes else None,
                             cache.v_pages if cache.writes else None, self.H, self.G, self.d, self.dv, rt.status,
                             q_gain=self.q_gain, k_gain=self.k_gain, norm_eps=getattr(s, "qk_norm_eps", 0.0),
                             values_from_keys=self.v_from_k)
        out = torch.empty((n, self.H * self.dv), dtype=x.dtype, device=x.device)
        gate = gate_src[:, self.qkv_cols:] if s.out_gate else None
        kernels.gated_attention(q, out, cache.k_pages, cache.v_pages, table, batch, self.H, self.G, self.d, self.dv, s.scale,
                                s.window or 0, s.chunk or 0, gate, rt.status, softcap=getattr(s, "softcap", None) or 0.0,
                                out_scale=getattr(s, "out_scale", 1.0), sink=self.sink)
        return self.o(out, keep_partials=True)


register_part("mixer", "gated_attention", GatedAttention)
