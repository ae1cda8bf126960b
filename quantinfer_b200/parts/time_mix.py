"""Time mixing over a matrix state per head, with a decay per head and key channel (RWKV style).

    mix_s = x + (x' - x) * mu_s               s in r, k, v, g, w; x' the previous token's x (zeros at a sequence's start)
    r, k, v = W_r mix_r, W_k mix_k, W_v mix_v (heads x head_dim each)          gate = silu(W_g mix_g)
    decay = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))                             (32-bit from the projection's output on)
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t       S_t = diag(decay_t) S_(t-1) + k_t v_t^T         (32-bit, per head)
    y = (o / rms(o) per head * norm * gate) . Wo^T

A request's state of fixed size is one row of 32-bit numbers in its slot: the previous token's x, then S for every head.
The rank of the decay's two projections is read from `w1` when the spec leaves it open.
"""

from __future__ import annotations

import torch

from .. import kernels
from . import segments
from ..cache.needs import StateNeed
from ..errors import ConfigError, WeightError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear

MIXES = ("r", "k", "v", "g", "w")


class TimeMix(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if min(s.heads, s.head_dim) <= 0:
            raise ConfigError("time_mix: heads and head_dim must be greater than zero")
        self.inner = s.heads * s.head_dim
        self.r, self.k, self.v, self.g = (Linear(runtime, self.inner, s.hidden_size, s.prefix + n) for n in ("r", "k", "v", "g"))
        self.o = Linear(runtime, s.hidden_size, self.inner, s.prefix + "o")
        self.w1 = self.w2 = None           # built at load: their rank may come from the tensors
        self.mu = self.w0 = self.u = self.gain = None

    @classmethod
    def needs_of_spec(cls, s):
        p, h, inner, rank = s.prefix, s.hidden_size, s.heads * s.head_dim, s.decay_rank
        needs = {p + "mu." + n: TensorNeed((h,), "matrix", "zeros") for n in MIXES}
        needs.update({p + n: TensorNeed((inner, h)) for n in ("r", "k", "v", "g")})
        needs.update({p + "w1": TensorNeed((rank, h)), p + "w2": TensorNeed((inner, rank)), p + "w0": TensorNeed((inner,), "matrix", "zeros"),
                      p + "u": TensorNeed((s.heads, s.head_dim), "matrix", "zeros"), p + "norm": TensorNeed((inner,), "gain", "gain"),
                      p + "o": TensorNeed((h, inner))})
        return needs

    def load(self, tensors):
        p, s = self.spec.prefix, self.spec
        for lin, n in ((self.r, "r"), (self.k, "k"), (self.v, "v"), (self.g, "g"), (self.o, "o")):
            lin.load(tensors[p + n])
        rank = tensors[p + "w1"].shape[0]
        if tensors[p + "w2"].shape[1] != rank:
            raise WeightError(f"{p}w1 has {rank} rows, {p}w2 has {tensors[p + 'w2'].shape[1]} columns: the decay's rank must be one number")
        self.w1 = Linear(self.runtime, rank, s.hidden_size, p + "w1")
        self.w2 = Linear(self.runtime, self.inner, rank, p + "w2")
        self.w1.load(tensors[p + "w1"])
        self.w2.load(tensors[p + "w2"])
        self.mu = self._gain(torch.stack([tensors[p + "mu." + n].to(torch.float32) for n in MIXES]))
        self.w0, self.u, self.gain = self._gain(tensors[p + "w0"]), self._gain(tensors[p + "u"].reshape(-1)), self._gain(tensors[p + "norm"])

    def cache_need(self):
        s = self.spec
        return StateNeed((s.hidden_size + s.heads * s.head_dim * s.head_dim,), torch.float32)

    def forward(self, x, batch, cache):
        s = self.spec
        n, h = x.shape
        state = cache.state
        prev, S = state[:, :h], state[:, h:].unflatten(1, (s.heads, s.head_dim, s.head_dim))
        mixes = torch.empty((len(MIXES), n, h), dtype=x.dtype, device=x.device)
        kernels.token_shift(x, self.mu, prev, mixes, batch.token_req, batch.q_start, batch.start_pos, batch.slot_ids)
        r, k, v, g = self.r(mixes[0]), self.k(mixes[1]), self.v(mixes[2]), self.g(mixes[3])
        low = self.w1(mixes[4])
        kernels.activation(low, low, "tanh")
        log_decay = self.w2(low)
        o = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        segments.matrix_state_scan("channel_decay", r, k, v, S, o, batch, s.heads, s.head_dim, s.head_dim, log_decay=log_decay,
                                   decay_bias=self.w0, bonus=self.u)
        y = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_rmsnorm(o, g, self.gain, s.norm_eps, y, s.heads, gate="silu")
        return self.o(y, keep_partials=True)


register_part("mixer", "time_mix", TimeMix)
