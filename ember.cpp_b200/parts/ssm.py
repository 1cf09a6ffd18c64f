"""Mamba-2 (the state-space duality layer) as a mixer with per-sequence state and no cache.

One input projection makes, side by side, a gate z, the channels x | B | C and a step size per
head.  x, B and C pass a short causal convolution over the sequence (one filter per channel, the
last tap on the current token, zeros before the sequence's start) and silu.  Per head, with a
state S of `state` x `vdim` float32 values that starts at zero:

    dt_t = softplus(dt_t + dt_bias)          a_t = exp(-exp(A_log) * dt_t)
    S_t  = a_t * S_(t-1) + dt_t * B_t x_t^T     y_t = S_t^T C_t + D * x_t

(head h reads the B and C of group h // (heads / groups)).  y is multiplied by silu(z), divided by
its root mean square in `norm_groups` equal parts of a row, multiplied by a gain, and projected
out.  Step sizes, decays, the recurrence and its state, the gate and the norm are float32 in
every mode; the projections and the convolution with its silu are in the compute type.

What a sequence carries from step to step: S of every head, and the last `conv` - 1 rows that
entered the convolution (`StateNeed`s "ssm" and "conv"; the cache keeps a row of each per slot).
"""
from __future__ import annotations

from .base import Mixer, StateNeed, WeightSpec, register_part


class Mamba2(Mixer):

    def __init__(self, prefix: str, width: int, heads: int, vdim: int, groups: int, state: int, conv: int,
                 norm_groups: int, eps: float, proj: str = "in", conv_name: str = "conv", conv_bias: str = "conv.b",
                 dt_bias: str = "dt_bias", a_log: str = "A_log", skip: str = "D", norm: str = "norm", out: str = "o",
                 init_std: float = 0.02, out_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.heads, self.vdim, self.groups = int(width), int(heads), int(vdim), int(groups)
        self.state, self.taps, self.norm_groups, self.eps = int(state), int(conv), int(norm_groups), float(eps)
        if self.heads <= 0 or self.groups <= 0 or self.heads % self.groups:
            raise ValueError(f"mamba2 {prefix!r}: {self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.vdim
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2 {prefix!r}: {self.inner} channels do not split into {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"mamba2 {prefix!r}: a convolution of {self.taps} taps is not in [1, 16]")
        if not 1 <= self.state <= 256:
            raise ValueError(f"mamba2 {prefix!r}: a state of {self.state} rows is not in [1, 256]")
        self.channels = self.inner + 2 * self.groups * self.state      # x | B | C, what the convolution sees
        self.proj_width = 2 * self.inner + 2 * self.groups * self.state + self.heads
        self.names = {k: prefix + v for k, v in dict(proj=proj, conv=conv_name, conv_bias=conv_bias, dt_bias=dt_bias,
                                                     a_log=a_log, skip=skip, norm=norm, out=out).items()}
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_out = None

    def weight_specs(self):
        n = self.names
        return [WeightSpec(n["proj"], (self.proj_width, self.width), std=self.init_std),
                WeightSpec(n["conv"], (self.channels, self.taps), std=0.3),
                WeightSpec(n["conv_bias"], (self.channels,), std=0.1),
                WeightSpec(n["dt_bias"], (self.heads,), mean=-1.0, std=0.5),
                WeightSpec(n["a_log"], (self.heads,), mean=-0.5, std=0.5),
                WeightSpec(n["skip"], (self.heads,), mean=1.0, std=0.2),
                WeightSpec(n["norm"], (self.inner,), mean=1.0, std=0.1),
                WeightSpec(n["out"], (self.width, self.inner), std=self.out_init_std)]

    def load(self, get, runtime):
        import torch
        n = self.names
        w = runtime.matrix(get(n["proj"]))
        # rows of zeros up to a multiple of 8: every row of the projection's output then starts on 16 bytes
        self.proj_stride = -(-self.proj_width // 8) * 8
        if self.proj_stride != self.proj_width:
            w = torch.cat([w, torch.zeros((self.proj_stride - self.proj_width, self.width), dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.conv_w = runtime.vector(get(n["conv"]))          # [channels, taps], float32
        self.conv_b = runtime.vector(get(n["conv_bias"]))
        self.dt_bias = runtime.vector(get(n["dt_bias"]))
        self.a_log = runtime.vector(get(n["a_log"]))
        self.skip = runtime.vector(get(n["skip"]))
        self.norm_w = runtime.vector(get(n["norm"]))

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        need = {"ssm": StateNeed((self.heads, self.vdim, self.state))}     # S transposed: a value channel's row of states
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps - 1, self.channels))       # the rows before the step's first, oldest first
        return need

    def _mix(self, ctx, h, app):
        ops = ctx.ops
        proj = ops.linear(h, self.w_in, None, out_dtype=ctx.dtype)                       # [T, z | x B C | dt (| 0)]
        xbc = ops.conv_silu(proj, self.inner, self.channels, self.conv_w, self.conv_b, app.state.get("conv"), ctx.plan)
        y = ops.ssd_scan(xbc, proj, 2 * self.inner + 2 * self.groups * self.state, self.dt_bias, self.a_log, self.skip,
                         app.state["ssm"], ctx.plan, self.heads, self.vdim, self.groups, self.state)
        return ops.gated_group_norm(y, proj, 0, self.norm_w, self.norm_groups, self.eps, ctx.dtype)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "mamba2", Mamba2)
