"""Causal attention over a cached low-rank latent, with a rotated key part shared by all heads.

    q        = x . Wq^T                    per head [head_dim plain | rot_dim rotated]
    z        = x . Wdkv^T                  kv_rank + rot_dim numbers
    c        = rmsnorm(z[:kv_rank]) * g    the latent (32-bit norm, gain per coordinate)
    kr       = rotate(z[kv_rank:], p)      one rotated key part for all heads
    cache[p] = [c | kr]
    k_h, v_h = Wuk_h c, Wuv_h c            (never formed, see below)
    s_ij     = (q_h(i) . k_h(j) + rotate(qr_h(i), i) . kr(j)) * scale,   j in the window of i
    p_ij     = exp(s_ij) / (sum_j exp(s_ij) + exp(sink_h))
    y        = (concat_h sum_j p_ij v_h(j)) * sigmoid(x . Wg^T) . Wo^T        (the gate is optional)

Keys and values are not expanded: q_h . (Wuk_h c) = (Wuk_h^T q_h) . c, so the plain part of the query is moved
into the latent space by a per-head product, every head then attends over the SAME cached rows (query width
kv_rank + rot_dim, "value" the row's first kv_rank numbers), and the result is taken out of the latent space by
Wuv_h. The projections of q and of the latent are one product over the stacked weights. A layer that shares
another layer's latent has no Wdkv and reads that layer's cache entry with its own Wuk, Wuv, window and sinks.

Every size and constant is a field of the spec. The angles of the rotation are computed in the kernel from
32-bit frequencies, theta^(-2i / rotary_dim), so there is no table and no limit on positions. The pairs are
neighbours (2i, 2i + 1) or halves (i, i + rotary_dim / 2), as the position spec says; its `stretch` (frequencies of
slowly turning pairs divided by a factor, cos and sin enlarged) is applied where the frequencies are made.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.needs import PagedLatentNeed
from ..errors import ConfigError
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear
from .position import direct_frequencies


class LatentAttention(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        s = spec
        if s.window is not None and s.window <= 0:
            raise ConfigError("latent_attention: window must be positive or None")
        pos = s.position
        self.rot_dims = pos.rotary_dim if pos is not None else 0
        if pos is not None and (pos.pairing not in ("interleaved", "half_split") or pos.rotary_dim % 2 or pos.rotary_dim > s.rot_dim):
            raise ConfigError("latent_attention: the rotation must pair coordinates within the rotated part")
        self.H, self.d, self.r, self.e, self.R = s.num_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        self.q_width = self.H * (self.d + self.r)
        self.out_gate = bool(getattr(s, "out_gate", False))
        self.kv_width = 0 if s.shares_latent else self.R + self.r
        n_out = self.q_width + self.kv_width + (self.H * self.e if self.out_gate else 0)
        self.proj = Linear(runtime, n_out, s.hidden_size, s.prefix + "q+dkv+g")
        self.o = Linear(runtime, s.hidden_size, self.H * self.e, s.prefix + "o")
        self.uk_t = self.uv = self.gain = self.sink = self.inv_freq = None
        self.keep_partials = False      # a block whose next norm adds a split product's partial sums itself sets this
        self.half_split = pos is not None and pos.pairing == "half_split"
        self.magnitude = 1.0
        if self.rot_dims:
            if getattr(pos, "stretch", None) is None and not self.half_split:
                # theta^(-2i / dims), exponent and power in 32-bit
                exponent = (2.0 * torch.arange(self.rot_dims // 2, dtype=torch.float32)) / torch.tensor(float(self.rot_dims), dtype=torch.float32)
                self.inv_freq = torch.pow(torch.tensor(float(pos.theta), dtype=torch.float32), -exponent).to(runtime.device)
            else:
                freqs, self.magnitude = direct_frequencies(pos)
                self.inv_freq = freqs.to(runtime.device)

    @classmethod
    def needs_of_spec(cls, s):
        p, H = s.prefix, s.num_heads
        needs = {p + "q": TensorNeed((H * (s.head_dim + s.rot_dim), s.hidden_size))}
        if not s.shares_latent:
            needs[p + "dkv"] = TensorNeed((s.kv_rank + s.rot_dim, s.hidden_size))
            needs[p + "dkv.norm"] = TensorNeed((s.kv_rank,), "gain", "gain")
        needs[p + "uk"] = TensorNeed((H * s.head_dim, s.kv_rank))
        needs[p + "uv"] = TensorNeed((H * s.value_dim, s.kv_rank))
        if s.sink:
            needs[p + "sink"] = TensorNeed((H,), "gain", "normal")
        if getattr(s, "out_gate", False):
            needs[p + "g"] = TensorNeed((H * s.value_dim, s.hidden_size))
        needs[p + "o"] = TensorNeed((s.hidden_size, H * s.value_dim))
        return needs

    def load(self, tensors):
        s, p, rt = self.spec, self.spec.prefix, self.runtime
        stack = [tensors[p + "q"]] + ([] if s.shares_latent else [tensors[p + "dkv"]]) + ([tensors[p + "g"]] if self.out_gate else [])
        if len({t.dtype for t in stack}) > 1:
            stack = [t.to(torch.float32) for t in stack]
        self.proj.load(torch.cat(stack, dim=0))
        self.o.load(tensors[p + "o"])
        wdt = torch.float32 if rt.dtype == torch.float32 else None
        uk = tensors[p + "uk"].reshape(self.H, self.d, self.R)
        # into the latent space: ql_h = Wuk_h^T q_h, as a product with weight [R, d] per head
        self.uk_t = uk.transpose(1, 2).to(device=rt.device, dtype=wdt or uk.dtype).contiguous()
        uv = tensors[p + "uv"].reshape(self.H, self.e, self.R)
        self.uv = uv.to(device=rt.device, dtype=wdt or uv.dtype).contiguous()
        if not s.shares_latent:
            self.gain = self._gain(tensors[p + "dkv.norm"])
        if s.sink:
            self.sink = self._gain(tensors[p + "sink"])

    def cache_need(self):
        return PagedLatentNeed(self.R + self.r, self.spec.window)

    def forward(self, x, batch, cache):
        rt, s = self.runtime, self.spec
        n = x.shape[0]
        W = self.R + self.r
        table = batch.block_tables[cache.group]
        writes = cache.writes and not s.shares_latent
        z = self.proj(x)                                        # [n, H (d + r) (+ R + r) (+ H e)]
        q = torch.empty((n, self.H, W), dtype=x.dtype, device=x.device)
        kernels.latent_prepare(z, self.q_width if writes else None, q, self.gain, s.norm_eps, self.inv_freq, self.rot_dims,
                               batch.positions, batch.token_req, table, cache.k_pages, self.H, self.d, self.r, self.R, rt.status,
                               half_split=self.half_split, magnitude=self.magnitude)
        kernels.head_linear(z, self.d + self.r, 0, self.d, self.uk_t, q.view(n, self.H * W), W, 0)    # q[:, h, :R] = Wuk_h^T q_h
        o_lat = torch.empty((n, self.H, self.R), dtype=x.dtype, device=x.device)
        ranges = 1
        if batch.all_decode and x.dtype == torch.bfloat16:
            # few query tiles, many keys: the keys of every token are spread over CTAs (a bound on the keys, not the
            # requests' lengths, so that a captured step serves its whole context bucket)
            keys = min(s.window or batch.max_kv_len, batch.max_kv_len)
            ranges = kernels.latent_attention_ranges(n * -(-self.H // 64), keys, W)
        kernels.latent_attention(q, o_lat, cache.k_pages, self.sink, table, batch.q_start, batch.start_pos, batch.positions,
                                 batch.token_req, s.scale, s.window or 0, rt.status, key_ranges=ranges)
        o = torch.empty((n, self.H, self.e), dtype=x.dtype, device=x.device)
        kernels.head_linear(o_lat.view(n, self.H * self.R), self.R, 0, self.R, self.uv, o.view(n, self.H * self.e), self.e, 0)
        o = o.view(n, self.H * self.e)                                          # o_h = Wuv_h (sum_j p_j c_j)
        if self.out_gate:
            kernels.sigmoid_gate(o, z[:, self.q_width + self.kv_width:])
        return self.o(o, keep_partials=self.keep_partials)                      # then Wo


register_part("mixer", "latent_attention", LatentAttention)
