"""Two mixers side by side that read the same input; the sum of their outputs is the mixer's.

Each branch is a mixer of any registered kind with its own tensors; a factor on a branch is a field of that branch's
spec (applied by the branch before its output projection, so the sum needs no factors). At most one branch keeps
pages: its need is this mixer's `cache_need`. Everything else the branches keep is of fixed size: a branch's own
entry (when its `cache_need` is a StateNeed) and what a branch keeps beside its pages (`state_need`) are laid side by
side in ONE row of 32-bit numbers, this mixer's `state_need`, and each branch is handed its part of it.

With `out_norm_names` in the spec each branch's output first passes an RMS norm over the model width (a gain per branch),
and `sum_scale` multiplies the sum; norms, factor and sum are one kernel, which also adds the partial sums of the
branches' output projections.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheView
from ..cache.needs import StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, build_part, part_class, register_part


def _floats(need) -> int:
    if need.dtype is not torch.float32:
        raise ConfigError("parallel_mixers: the branches' state of fixed size must be 32-bit")
    n = 1
    for d in need.shape:
        n *= d
    return n


class ParallelMixers(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.branches = (build_part("mixer", spec.left, runtime), build_part("mixer", spec.right, runtime))
        # where each branch's states lie in the shared row: (own entry, beside its pages), each (offset, need) or None
        self._paged, self._layout, at = None, [], 0
        for i, b in enumerate(self.branches):
            own, beside = b.cache_need(), getattr(b, "state_need", lambda: None)()
            if own is not None and not isinstance(own, StateNeed):
                if self._paged is not None:
                    raise ConfigError("parallel_mixers: only one branch may keep pages")
                self._paged, own = (i, own), None
            spans = []
            for need in (own, beside):
                spans.append((at, need) if need is not None else None)
                if need is not None:
                    at += (_floats(need) + 3) // 4 * 4          # every part starts at a 16-byte boundary
            self._layout.append(spans)
        self._floats = at
        self.out_gains = None
        names = getattr(spec, "out_norm_names", None)
        if names is not None and (len(names) != 2 or not getattr(spec, "hidden_size", None)):
            raise ConfigError("parallel_mixers: norms on the branches' outputs need two gain names and the model width")

    @classmethod
    def needs_of_spec(cls, spec):
        needs = {}
        for sub in (spec.left, spec.right):
            needs.update(part_class("mixer", sub).needs_of_spec(sub))
        for name in getattr(spec, "out_norm_names", None) or ():
            needs[name] = TensorNeed((spec.hidden_size,), "gain", "gain")
        return needs

    def load(self, tensors):
        for b in self.branches:
            b.load(tensors)
        names = getattr(self.spec, "out_norm_names", None)
        if names is not None:
            self.out_gains = tuple(self._gain(tensors[n]) for n in names)

    def cache_need(self):
        return self._paged[1] if self._paged is not None else None

    def state_need(self):
        return StateNeed((self._floats,), torch.float32) if self._floats else None

    def _part_of(self, row, span):
        if span is None:
            return None
        at, need = span
        flat = row[:, at:at + _floats(need)]
        return flat.unflatten(1, tuple(need.shape)) if len(need.shape) != 1 else flat

    def forward(self, x, batch, cache):
        row = cache.mixer_state
        outs = []
        for i, b in enumerate(self.branches):
            own, beside = self._layout[i]
            if self._paged is not None and self._paged[0] == i:
                view = CacheView(cache.entry, cache.group, cache.page_size, cache.k_pages, cache.v_pages, None, cache.writes,
                                 mixer_state=self._part_of(row, beside))
            else:
                view = CacheView(cache.entry, state=self._part_of(row, own), writes=cache.writes, mixer_state=self._part_of(row, beside))
            outs.append(b.forward(x, batch, view))      # whole, or K-split partial sums [parts, n, h]: added in 32-bit below
        out = torch.empty(outs[0].shape[-2:], dtype=torch.float32, device=x.device)
        scale = getattr(self.spec, "sum_scale", 1.0)
        if self.out_gains is not None:
            kernels.normed_sum(outs[0], outs[1], self.out_gains[0], self.out_gains[1], self.spec.out_norm_eps, scale, out)
        else:
            kernels.scaled_sum(outs[0], outs[1], scale, scale, out)
        return out


register_part("mixer", "parallel_mixers", ParallelMixers)
