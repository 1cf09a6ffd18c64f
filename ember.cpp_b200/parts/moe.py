"""Experts chosen by a table: every token id names its `top` experts in a stored integer table
[vocab, top] (the entries of a row differ), each weighing 1/top; there is no router product.

An expert is a small gated feed-forward without biases, `down(silu(gate h) * (up h))`.  An
optional shared expert of the same form (a size of its own) runs for every token and is added.
The experts' matrices are stacked at load ([experts, gate | up, width] and [experts, width, inner]),
the step's (token, choice) pairs are sorted by expert on the device, and two grouped products run
each expert over its own pairs; nothing comes back to the host, so the step replays as a graph.
"""
from __future__ import annotations

from .base import FeedForward, WeightSpec, build_part, register_part
from .spec import PartSpec


class TableExperts(FeedForward):
    needs_tokens = True

    def __init__(self, prefix: str, width: int, vocab: int, experts: int, top: int, inner: int,
                 shared_inner: int = 0, table: str = "table", expert: str = "e{}.", shared: str = "shared.",
                 gate: str = "gate", up: str = "up", down: str = "down", suffix: str = ".weight",
                 init_std: float = 0.02, down_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.vocab, self.experts, self.top, self.inner = int(width), int(vocab), int(experts), int(top), int(inner)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"experts {prefix!r}: top = {self.top} of {self.experts} experts")
        if self.top > 15:
            raise ValueError(f"experts {prefix!r}: top = {self.top}; at most 15 experts a token")
        self.table_name = prefix + table
        self.expert_names = [tuple(prefix + expert.format(e) + n + suffix for n in (gate, up, down)) for e in range(self.experts)]
        self.init_std, self.down_init_std = init_std, down_init_std
        self.shared = None
        if shared_inner:
            self.shared = build_part("ffn", PartSpec("gated", prefix + shared, dict(
                width=width, inner=int(shared_inner), activation="silu", gate=gate, up=up, down=down, suffix=suffix,
                init_std=init_std, down_init_std=down_init_std)))
        self.w_gate_up = self.w_down = self.table = None

    def weight_specs(self):
        specs = [WeightSpec(self.table_name, (self.vocab, self.top), integer=True, below=self.experts)]
        for g, u, d in self.expert_names:
            specs += [WeightSpec(g, (self.inner, self.width), std=self.init_std),
                      WeightSpec(u, (self.inner, self.width), std=self.init_std),
                      WeightSpec(d, (self.width, self.inner), std=self.down_init_std)]
        return specs + (self.shared.weight_specs() if self.shared is not None else [])

    def load(self, get, runtime):
        import torch
        table = get(self.table_name).to(torch.int64)
        if int(table.min()) < 0 or int(table.max()) >= self.experts:
            raise ValueError(f"experts {self.prefix!r}: the table names an expert outside [0, {self.experts})")
        self.table = runtime.index_table(table)
        self.w_gate_up = torch.stack([torch.cat([runtime.matrix(get(g)), runtime.matrix(get(u))]) for g, u, _ in self.expert_names]).contiguous()
        self.w_down = torch.stack([runtime.matrix(get(d)) for _, _, d in self.expert_names]).contiguous()
        if self.shared is not None:
            self.shared.load(get, runtime)

    def stream_weights(self):
        return self.shared.stream_weights() if self.shared is not None else []

    def _chosen(self, ctx, h):
        ops = ctx.ops
        routing = ops.moe_route(ctx.plan.tokens, ctx.plan.T, self.table, self.experts, self.top)
        inner = ops.moe_gate_up(h, self.w_gate_up, routing, out_dtype=ctx.dtype)     # [T * top, inner], silu(g) * u
        y = ops.moe_down(inner, self.w_down, routing)                                 # float32 [T, top, width]
        return [(y[:, k, :], 1.0 / self.top) for k in range(self.top)]

    def branches(self, ctx, h):
        if self.shared is None:
            return self._chosen(ctx, h)
        runs = [lambda: self._chosen(ctx, h), lambda: self.shared.branches(ctx, h)]
        together = getattr(ctx.ops, "side_by_side", None)     # (one-token steps: the shared expert beside the chosen ones)
        chosen, shared = together(runs) if together is not None and ctx.plan.all_single else [run() for run in runs]
        return chosen + shared

    def forward(self, ctx, h, residual):
        x = residual
        for rows, f in self.branches(ctx, h):
            x = x + f * rows
        return x


register_part("ffn", "table_experts", TableExperts)
