"""A selective state-space mixer with one decay a head (the state-space-duality form of Mamba).

    [z | xBC | dt] = x . W_in^T                     z: inner, xBC: inner + 2 groups state, dt: heads; inner = heads * head_dim
    xBC            = silu(conv(xBC) + b_conv)       causal, per channel, `taps` taps, zeros before the sequence's start
    dt             = softplus(dt + dt_bias)         a = exp(-exp(A_log) * dt)             (32-bit, per head)
    S_t            = a_t S_(t-1) + dt_t B_t x_t^T   y_t = S_t^T C_t + D x_t              (32-bit; S is state x head_dim a head)
    y              = rmsnorm_groups(y * silu(z)) * g                                      (the gate comes before the norm)
    out            = y . W_o^T

B and C belong to the head's group. A request's state of fixed size is ONE row of 32-bit numbers in its slot: the
last taps - 1 inputs of the convolution, then S for every head; the cache manager zeroes it when the request
opens, copies it aside before a step and back if the step fails. The kernels take zeros at position 0 whatever
the slot holds, read the state at a step entry's first token and write it after its last, so one launch serves
whole prompts, portions cut anywhere and single decode tokens, side by side in one batch.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import StateNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from . import segments
from .base import Part, register_part
from .linear import Linear


class Mamba2(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if min(s.heads, s.head_dim, s.state, s.groups, s.conv_taps, s.norm_groups) <= 0:
            raise ConfigError("mamba2: every size must be greater than zero")
        if s.heads % s.groups:
            raise ConfigError(f"mamba2: {s.heads} heads are not a multiple of {s.groups} groups")
        self.inner = s.heads * s.head_dim
        if self.inner % s.norm_groups:
            raise ConfigError(f"mamba2: {self.inner} channels do not split into {s.norm_groups} equal parts")
        self.channels = self.inner + 2 * s.groups * s.state
        self.inp = Linear(runtime, self.inner + self.channels + s.heads, s.hidden_size, s.prefix + "in")
        self.o = Linear(runtime, s.hidden_size, self.inner, s.prefix + "o")
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.gain = None
        self.conv_floats = (s.conv_taps - 1) * self.channels

    @classmethod
    def needs_of_spec(cls, s):
        p, inner = s.prefix, s.heads * s.head_dim
        ch = inner + 2 * s.groups * s.state
        return {p + "in": TensorNeed((inner + ch + s.heads, s.hidden_size)), p + "conv": TensorNeed((ch, s.conv_taps)),
                p + "conv.b": TensorNeed((ch,), "matrix", "zeros"), p + "dt_bias": TensorNeed((s.heads,)),
                p + "A_log": TensorNeed((s.heads,)), p + "D": TensorNeed((s.heads,), "gain", "gain"),
                p + "norm": TensorNeed((inner,), "gain", "gain"), p + "o": TensorNeed((s.hidden_size, inner))}

    def load(self, tensors):
        p = self.spec.prefix
        self.inp.load(tensors[p + "in"])
        self.o.load(tensors[p + "o"])
        self.conv_w = self._gain(tensors[p + "conv"].to(torch.float32).t().unsqueeze(0))       # [1, taps, channels]
        self.conv_b = self._gain(tensors[p + "conv.b"].reshape(1, -1))
        self.dt_bias, self.a_log = self._gain(tensors[p + "dt_bias"]), self._gain(tensors[p + "A_log"])
        self.d_skip, self.gain = self._gain(tensors[p + "D"]), self._gain(tensors[p + "norm"])

    def cache_need(self):
        s = self.spec
        return StateNeed((self.conv_floats + s.heads * s.head_dim * s.state,), torch.float32)

    SEGMENT, SEGMENT_FROM = segments.SEGMENT, segments.SEGMENT_FROM

    def _segments(self, batch):
        """The step's entries cut into segments when one of them is long (`segments.entry_segments`)."""
        return segments.entry_segments(batch, self.SEGMENT, self.SEGMENT_FROM)

    def forward(self, x, batch, cache):
        s = self.spec
        n = x.shape[0]
        proj = self.inp(x)
        state = cache.state                                   # float32 [slots, conv inputs | S]
        conv_state = state[:, :self.conv_floats].unflatten(1, (s.conv_taps - 1, self.channels)) if s.conv_taps > 1 else None
        ssm_state = state[:, self.conv_floats:].unflatten(1, (s.heads, s.head_dim, s.state))
        xbc = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        kernels.short_conv(proj[:, self.inner:self.inner + self.channels], self.conv_w, conv_state, [xbc], None, batch.token_req,
                           batch.q_start, batch.start_pos, batch.slot_ids, residual=False, bias=self.conv_b, act="silu")
        y = torch.empty((n, self.inner), dtype=torch.float32, device=x.device)
        raw_dt = proj[:, self.inner + self.channels:]
        seg = self._segments(batch)
        if seg is None:
            kernels.ssm_scan(xbc, raw_dt, self.dt_bias, self.a_log, self.d_skip, ssm_state, y,
                             batch.q_start, batch.start_pos, batch.slot_ids, s.heads, s.groups, s.head_dim, s.state)
        else:
            # long entries: segments side by side (see csrc/ssm.cu): each from zero, the chain of their states, each again
            seg_q_start, entry_seg, zeros, ones, rows, longest = seg
            local = torch.empty((rows.numel(), s.heads, s.head_dim, s.state), dtype=torch.float32, device=x.device)
            kernels.ssm_scan(xbc, raw_dt, self.dt_bias, self.a_log, self.d_skip, local, None, seg_q_start, zeros, rows,
                             s.heads, s.groups, s.head_dim, s.state, long_entries=True)
            kernels.ssm_chain(local, ssm_state, raw_dt, self.dt_bias, self.a_log, seg_q_start, entry_seg, batch.start_pos,
                              batch.slot_ids, longest)
            kernels.ssm_scan(xbc, raw_dt, self.dt_bias, self.a_log, self.d_skip, local, y, seg_q_start, ones, rows,
                             s.heads, s.groups, s.head_dim, s.state, write_state=False, long_entries=True)
        g = torch.empty((n, self.inner), dtype=x.dtype, device=x.device)
        kernels.gated_group_rmsnorm(y, proj[:, :self.inner], self.gain, s.norm_eps, g, s.norm_groups)
        return self.o(g, keep_partials=True)


register_part("mixer", "mamba2", Mamba2)
