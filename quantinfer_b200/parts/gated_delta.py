"""A matrix state per head that is decayed per key channel and corrected towards each token's value (gated delta rule).

    [q | k | v | b] = x . W^T                  (stacked at load: one product; q, k: kv_heads x head_dim, v: heads x value_dim)
    q | k | v       = silu(conv(q | k | v))    a causal convolution over time per channel, `conv_taps` taps, no bias
    q, k            = q / sqrt(sum q^2 + unit_eps) * head_dim^(-1/2),  k / sqrt(sum k^2 + unit_eps)       per head
    beta            = sigmoid(b)               one a head
    w               = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias))      per head and key channel
    S' = diag(w) S ;  u = beta (v - S'^T k) ;  S = S' + k u^T ;  o = S^T q      per head, token by token, 32-bit
    y = (o / rms(o) per head * norm * sigmoid(W_g2 (W_g1 x))) . Wo^T

Head h reads the q/k head floor(h / (heads / kv_heads)). The two low-rank pairs share their products: a1 and g1 are
stacked into one projection, a2 and g2 into one block-diagonal one, so the decay's logits and the gate's come out of
one product side by side; the ranks are read from the tensors. Unit vectors, beta, softplus and both exponentials are
evaluated in 32-bit inside the recurrence kernel while it stages a token's operands.

A request's state of fixed size: S [heads, value_dim, head_dim] (32-bit, zero at a sequence's start) is the mixer's own
entry; the convolutions' last taps - 1 projected rows of q | k | v (32-bit) lie beside it (`state_need`).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import StateNeed
from ..errors import ConfigError, WeightError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class GatedDelta(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if min(s.heads, s.kv_heads, s.head_dim, s.value_dim) <= 0 or s.heads % s.kv_heads:
            raise ConfigError("gated_delta: sizes must be greater than zero and heads a multiple of kv_heads")
        if not 1 <= s.conv_taps <= 16:
            raise ConfigError(f"gated_delta: a convolution of {s.conv_taps} taps (1..16)")
        if s.head_dim > 256:
            raise ConfigError(f"gated_delta: keys of {s.head_dim} are beyond the recurrence kernel (256)")
        self.qk, self.inner, self.decays = s.kv_heads * s.head_dim, s.heads * s.value_dim, s.heads * s.head_dim
        self.conv_cols = 2 * self.qk + self.inner
        self.proj = Linear(runtime, self.conv_cols + s.heads, s.hidden_size, s.prefix + "q+k+v+b")
        self.o = Linear(runtime, s.hidden_size, self.inner, s.prefix + "o")
        self.low = self.high = None         # built at load: their ranks come from the tensors
        self.conv_w = self.gain = self.a_log = self.dt_bias = None

    @classmethod
    def needs_of_spec(cls, s):
        p, h = s.prefix, s.hidden_size
        qk, inner, decays = s.kv_heads * s.head_dim, s.heads * s.value_dim, s.heads * s.head_dim
        return {p + "q": TensorNeed((qk, h)), p + "k": TensorNeed((qk, h)), p + "v": TensorNeed((inner, h)),
                p + "q.conv": TensorNeed((qk, s.conv_taps)), p + "k.conv": TensorNeed((qk, s.conv_taps)),
                p + "v.conv": TensorNeed((inner, s.conv_taps)), p + "b": TensorNeed((s.heads, h)),
                p + "A_log": TensorNeed((s.heads,), "gain", "zeros"), p + "dt_bias": TensorNeed((decays,), "gain", "zeros"),
                p + "a1": TensorNeed((None, h)), p + "a2": TensorNeed((decays, None)),
                p + "g1": TensorNeed((None, h)), p + "g2": TensorNeed((inner, None)),
                p + "norm": TensorNeed((s.value_dim,), "gain", "gain"), p + "o": TensorNeed((h, inner))}

    def load(self, tensors):
        p, s, rt = self.spec.prefix, self.spec, self.runtime

        def stacked(names):
            ws = [tensors[p + n] for n in names]
            if len({t.dtype for t in ws}) > 1:
                ws = [t.to(torch.float32) for t in ws]
            return ws

        self.proj.load(torch.cat(stacked(("q", "k", "v", "b")), dim=0))
        self.o.load(tensors[p + "o"])
        a1, g1, a2, g2 = stacked(("a1", "g1", "a2", "g2"))
        ra, rg = a1.shape[0], g1.shape[0]
        if a2.shape[1] != ra or g2.shape[1] != rg:
            raise WeightError(f"{p}a1/a2 or {p}g1/g2: the two halves of a low-rank pair must share their rank")
        self.low = Linear(rt, ra + rg, s.hidden_size, p + "a1+g1")
        self.low.load(torch.cat([a1, g1], dim=0))
        high = torch.zeros((self.decays + self.inner, ra + rg), dtype=a2.dtype)
        high[:self.decays, :ra] = a2
        high[self.decays:, ra:] = g2
        self.high = Linear(rt, self.decays + self.inner, ra + rg, p + "a2+g2")
        self.high.load(high)
        w = torch.cat([tensors[p + n + ".conv"].to(torch.float32) for n in ("q", "k", "v")], dim=0)
        self.conv_w = self._gain(w.t().unsqueeze(0))              # [1, taps, q | k | v channels]
        self.gain = self._gain(tensors[p + "norm"].to(torch.float32).repeat(s.heads))
        self.a_log, self.dt_bias = self._gain(tensors[p + "A_log"]), self._gain(tensors[p + "dt_bias"])

    def cache_need(self):
        s = self.spec
        return StateNeed((s.heads * s.value_dim * s.head_dim,), torch.float32)

    def state_need(self):
        """The convolutions' state: the last taps - 1 rows of q | k | v as projected (32-bit)."""
        if self.spec.conv_taps < 2:
            return None
        return StateNeed((self.spec.conv_taps - 1, self.conv_cols), torch.float32)

    def forward(self, x, batch, cache):
        s = self.spec
        n = x.shape[0]
        qk, inner, decays = self.qk, self.inner, self.decays
        proj = self.proj(x)
        conved = torch.empty((n, self.conv_cols), dtype=x.dtype, device=x.device)
        kernels.short_conv(proj[:, :self.conv_cols], self.conv_w, cache.mixer_state, [conved], None, batch.token_req, batch.q_start,
                           batch.start_pos, batch.slot_ids, residual=False, act="silu")
        logits = self.high(self.low(x))                         # [n, decay logits | gate logits]
        S = cache.state.unflatten(1, (s.heads, s.value_dim, s.head_dim))
        o = torch.empty((n, inner), dtype=torch.float32, device=x.device)
        kernels.matrix_state_scan("delta", conved[:, :qk], conved[:, qk:2 * qk], conved[:, 2 * qk:], S, o, batch.q_start, batch.start_pos,
                                  batch.slot_ids, s.heads, s.head_dim, s.value_dim, log_decay=logits[:, :decays], decay_bias=self.dt_bias,
                                  head_decay=self.a_log, beta=proj[:, self.conv_cols:], qk_heads=s.kv_heads, unit_eps=s.unit_eps,
                                  q_scale=float(s.head_dim) ** -0.5)
        y = torch.empty((n, inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_rmsnorm(o, logits[:, decays:], self.gain, s.norm_eps, y, s.heads, gate="sigmoid")
        return self.o(y, keep_partials=True)


register_part("mixer", "gated_delta", GatedDelta)
