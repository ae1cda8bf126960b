"""A gated recurrence per channel whose gates read only the current token (minGRU).

    [pz | px | pg] = x . W^T                  (the three projections stacked at load: one product)
    z = sigmoid(pz + b_z)     u = px + b_x     c = u + 1/2 where u >= 0, sigmoid(u) below
    S_t = (1 - z_t) S_(t-1) + z_t c_t         (32-bit, per channel)
    y = (S_t * silu(pg)) . Wo^T

A request's state is one row of `width` 32-bit numbers in its slot, zero at a sequence's start. The recurrence is
linear in S, so the kernel cuts an entry of many tokens into slices that run side by side and chains them.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


class MinGRU(Part):
    TOKENS_A_SLICE = 16      # an entry is cut so that a slice has at least this many tokens (at most 32 slices)

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.width <= 0:
            raise ConfigError("mingru: the width must be greater than zero")
        self.proj = Linear(runtime, 3 * spec.width, spec.hidden_size, spec.prefix + "z+x+g")
        self.o = Linear(runtime, spec.hidden_size, spec.width, spec.prefix + "o")
        self.bz = self.bx = None

    @classmethod
    def needs_of_spec(cls, s):
        p, w, h = s.prefix, s.width, s.hidden_size
        return {p + "z": TensorNeed((w, h)), p + "z.b": TensorNeed((w,), "matrix", "zeros"), p + "x": TensorNeed((w, h)),
                p + "x.b": TensorNeed((w,), "matrix", "zeros"), p + "g": TensorNeed((w, h)), p + "o": TensorNeed((h, w))}

    def load(self, tensors):
        p = self.spec.prefix
        ws = [tensors[p + n] for n in ("z", "x", "g")]
        if len({t.dtype for t in ws}) > 1:
            ws = [t.to(torch.float32) for t in ws]
        self.proj.load(torch.cat(ws, dim=0))
        self.o.load(tensors[p + "o"])
        self.bz, self.bx = self._gain(tensors[p + "z.b"]), self._gain(tensors[p + "x.b"])

    def cache_need(self):
        return StateNeed((self.spec.width,), torch.float32)

    def forward(self, x, batch, cache):
        w = self.spec.width
        proj = self.proj(x)
        out = torch.empty((x.shape[0], w), dtype=x.dtype, device=x.device)
        slices = 1 if batch.all_decode else max(1, min(32, batch.max_q_len // self.TOKENS_A_SLICE))
        kernels.mingru_scan(proj, self.bz, self.bx, cache.state, out, batch.q_start, batch.start_pos, batch.slot_ids, w, slices)
        return self.o(out, keep_partials=True)


register_part("mixer", "mingru", MinGRU)
