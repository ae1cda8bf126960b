"""Token embedding (a row gather into the 32-bit residual stream) and the
output head (a projection of the normed rows to 32-bit logits).

A tied head uses the embedding table itself: [vocab, hidden] is already the
[out, in] layout the projection reads (the reference materialises a transposed
copy, crates/quantinfer-runtime/src/qwen3/loader.rs:59; the gather is
backends/cpu/src/backend.rs:282-298, the head crates/quantinfer-runtime/src/qwen3/mod.rs:369-378).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorNeed
from .base import Part, register_part
from .linear import Linear


def _weight_name(spec) -> str:
    return getattr(spec, "weight_name", None) or spec.prefix + "weight"


class Embedding(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.table = Linear(runtime, spec.vocab_size, spec.hidden_size, _weight_name(spec))

    @classmethod
    def needs_of_spec(cls, spec):
        return {_weight_name(spec): TensorNeed((spec.vocab_size, spec.hidden_size), "table")}

    def load(self, tensors):
        self.table.load(tensors[_weight_name(self.spec)])

    def forward(self, token_ids):
        out = torch.empty((token_ids.numel(), self.spec.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embedding(self.table.weight, token_ids, out, self.runtime.status, scale=getattr(self.spec, "scale", 1.0))
        return out

    __call__ = forward


class LMHead(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.proj = None if spec.tied else Linear(runtime, spec.vocab_size, spec.hidden_size, _weight_name(spec))
        self.softcap = getattr(spec, "softcap", None)

    @classmethod
    def needs_of_spec(cls, spec):
        if spec.tied:
            return {}
        return {_weight_name(spec): TensorNeed((spec.vocab_size, spec.hidden_size))}

    def load(self, tensors):
        if not self.spec.tied:
            self.proj.load(tensors[_weight_name(self.spec)])

    def tie(self, embedding: Embedding):
        self.proj = embedding.table

    def forward(self, x):
        logits = self.proj(x, out_dtype=torch.float32)
        if self.softcap is not None and logits.numel():
            kernels.softcap(logits, self.softcap)      # c * tanh(logits / c), in place, 32-bit
        return logits

    __call__ = forward


class BigramEmbedding(Part):
    """Token embedding plus a row of a hashed bigram table: x = table[t] + bigram[(prev * mul_prev + t * mul_cur)
    mod buckets], and the table's last row (number `buckets`) for a sequence's first token. The previous token
    of a step's first token is the request's state: one int32 word a slot, which the kernel reads and advances,
    so the part needs the step's arrays and its state (`forward(ids, batch, view)`)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.table = Linear(runtime, spec.vocab_size, spec.hidden_size, spec.prefix + spec.table_name)
        self.bigram = Linear(runtime, spec.buckets + 1, spec.hidden_size, spec.prefix + spec.bigram_name)

    @classmethod
    def needs_of_spec(cls, spec):
        return {spec.prefix + spec.table_name: TensorNeed((spec.vocab_size, spec.hidden_size), "table"),
                spec.prefix + spec.bigram_name: TensorNeed((spec.buckets + 1, spec.hidden_size), "table")}

    def load(self, tensors):
        a, b = tensors[self.spec.prefix + self.spec.table_name], tensors[self.spec.prefix + self.spec.bigram_name]
        if a.dtype != b.dtype:
            a, b = a.to(torch.float32), b.to(torch.float32)
        self.table.load(a)
        self.bigram.load(b)

    def state_need(self):
        from ..cache.needs import StateNeed

        return StateNeed((1,), torch.int32)

    def forward(self, token_ids, batch, view):
        s = self.spec
        out = torch.empty((token_ids.numel(), s.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embedding_bigram(self.table.weight, self.bigram.weight, token_ids, batch.positions, batch.token_req,
                                 batch.q_start, batch.slot_ids, view.state, out, s.buckets, s.mul_prev, s.mul_cur,
                                 self.runtime.status)
        return out

    __call__ = forward


register_part("embedding", "embedding", Embedding)
register_part("embedding", "bigram_embedding", BigramEmbedding)
register_part("head", "lm_head", LMHead)
