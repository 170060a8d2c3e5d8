"""A per-layer input that depends on the token itself, as a feed-forward.

    e = table[token][offset : offset + D]          a slice of a table that all layers share (``bind_shared``)
    out += (act(h . W_gate^T) * e) . W_proj^T      act = gelu in its tanh form; D = ``intermediate_size``

The table is a tensor of the model, not of the layer (``ModelSpec.shared_tensors``); the layer's slice starts at
``offset``.  Two small products with the gate kernel between them.
"""
from __future__ import annotations

from typing import List

from ..weights.loader import WeightSpec
from .. import kernels as K
from . import linear
from .base import FEED_FORWARDS, FeedForward


class TokenTableInput(FeedForward):
    def __init__(self, spec):
        if spec.activation != "gelu_tanh":
            raise ValueError(f"activation '{spec.activation}' is not supported (only 'gelu_tanh')")
        self.spec = spec
        self.D, self.offset, self.table_name = spec.intermediate_size, int(spec.option("offset", 0)), spec.option("table")
        if self.D <= 0 or self.offset < 0 or not self.table_name:
            raise ValueError("a token-table input needs a table's name, an offset and a positive size")
        self.w_gate = self.w_proj = self.table = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p = self.spec, prefix + self.spec.prefix
        return [WeightSpec(p + s.name("gate", "gate"), (self.D, s.hidden_size)), WeightSpec(p + s.name("proj", "proj"), (s.hidden_size, self.D))]

    def bind(self, get) -> None:
        s, p = self.spec, self.spec.prefix
        self.w_gate, self.w_proj = get(p + s.name("gate", "gate")), get(p + s.name("proj", "proj"))

    def bind_shared(self, shared) -> None:
        self.table = shared[self.table_name]
        if self.offset + self.D > self.table.shape[1]:
            raise ValueError(f"columns {self.offset}..{self.offset + self.D} of a table {self.table.shape[1]} wide")

    def forward(self, h, ctx, out) -> None:
        T = h.shape[0]
        g = ctx.empty((T, self.D))
        if T <= linear.ROWS_MAX_M and ctx.options.get("small_products", True):      # a decode step: the gate's product and the gate in one kernel
            K.token_gate_rows(h, self.w_gate, self.table, ctx.layout.tokens, self.offset, g, ctx.stream)
        else:
            z = ctx.empty((T, self.D))
            linear.matmul(h, self.w_gate, z, linear.EPI_STORE, ctx)
            K.gelu_mul_table(z, self.table, ctx.layout.tokens, self.offset, g, ctx.stream)
        linear.matmul(g, self.w_proj, out, linear.EPI_ADD, ctx)


FEED_FORWARDS.register("token_table", TokenTableInput)
