"""Linear attention over a matrix state per head with one constant decay a head (lightning attention).

    [q | k | v | g] = x . W^T                 (the four projections stacked at load: one product)
    q, k, v = silu(q), silu(k), silu(v)       heads x head_dim, heads x head_dim, heads x value_dim
    S_t = decay_h S_(t-1) + k_t v_t^T         o_t = S_t^T q_t                                  (32-bit, per head)
    y = (rmsnorm(o over all heads) * norm * sigmoid(g) * out_scale) . Wo^T

A request's state of fixed size is S for every head, one row of 32-bit numbers in its slot, zero at a sequence's start.
"""

from __future__ import annotations

import torch

from .. import kernels
from . import segments
from ..cache.needs import StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class LightningAttention(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if min(s.heads, s.head_dim, s.value_dim) <= 0 or len(s.decays) != s.heads:
            raise ConfigError("lightning_attention: sizes must be greater than zero, with one decay a head")
        self.qk, self.inner = s.heads * s.head_dim, s.heads * s.value_dim
        self.proj = Linear(runtime, 2 * self.qk + 2 * self.inner, s.hidden_size, s.prefix + "q+k+v+g")
        self.o = Linear(runtime, s.hidden_size, self.inner, s.prefix + "o")
        self.decays = torch.tensor([float(d) for d in s.decays], dtype=torch.float32, device=runtime.device)
        self.gain = None

    @classmethod
    def needs_of_spec(cls, s):
        p, h, qk, inner = s.prefix, s.hidden_size, s.heads * s.head_dim, s.heads * s.value_dim
        return {p + "q": TensorNeed((qk, h)), p + "k": TensorNeed((qk, h)), p + "v": TensorNeed((inner, h)), p + "g": TensorNeed((inner, h)),
                p + "norm": TensorNeed((inner,), "gain", "gain"), p + "o": TensorNeed((h, inner))}

    def load(self, tensors):
        p = self.spec.prefix
        ws = [tensors[p + n] for n in ("q", "k", "v", "g")]
        if len({t.dtype for t in ws}) > 1:
            ws = [t.to(torch.float32) for t in ws]
        self.proj.load(torch.cat(ws, dim=0))
        self.o.load(tensors[p + "o"])
        self.gain = self._gain(tensors[p + "norm"])

    def cache_need(self):
        s = self.spec
        return StateNeed((s.heads * s.value_dim * s.head_dim,), torch.float32)

    def forward(self, x, batch, cache):
        s = self.spec
        n = x.shape[0]
        proj = self.proj(x)
        qk, inner = self.qk, self.inner
        S = cache.state.unflatten(1, (s.heads, s.value_dim, s.head_dim))
        o = torch.empty((n, inner), dtype=torch.float32, device=x.device)
        segments.matrix_state_scan("head_decay", proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + inner], S, o, batch,
                                   s.heads, s.head_dim, s.value_dim, head_decay=self.decays)
        y = torch.empty((n, inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_rmsnorm(o, proj[:, 2 * qk + inner:], self.gain, s.norm_eps, y, 1, gate="sigmoid", out_scale=s.out_scale)
        return self.o(y, keep_partials=True)


register_part("mixer", "lightning_attention", LightningAttention)
