"""Parts that add to the embedded rows before the first layer.

`pair_table`: a second table whose row is chosen by the token and the token before it in the
sequence, hashed into a fixed number of buckets:

    row(t) = (token[t-1] * mul_prev + token[t] * mul_cur) mod buckets      for t > 0
    row(0) = buckets                                                      (the table's extra last row)

and x[t] += table[row(t)].  The token before a step's first token is part of the sequence's state
(one int32 per sequence, written by every step with the sequence's last token of the step).
"""
from __future__ import annotations

from .base import EmbedPart, StateNeed, WeightSpec, register_part


class PairTable(EmbedPart):

    def __init__(self, prefix: str, width: int, buckets: int, mul_prev: int, mul_cur: int, table: str = "bigram",
                 init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.buckets, self.mul_prev, self.mul_cur = int(width), int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets <= 0:
            raise ValueError(f"pair table {prefix!r}: {self.buckets} buckets")
        self.table_name, self.init_std = prefix + table, init_std
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.table_name, (self.buckets + 1, self.width), std=self.init_std)]

    def load(self, get, runtime):
        self.table = runtime.table(get(self.table_name))

    def state_need(self):
        return StateNeed((1,), 0, "int32")       # the sequence's last token so far

    def forward(self, ctx, x, state):
        return ctx.ops.pair_table_add(x, ctx.plan, self.table, state, self.mul_prev, self.mul_cur, self.buckets)


register_part("embed", "pair_table", PairTable)
