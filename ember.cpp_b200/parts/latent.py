"""Attention whose keys and values are expanded from a cached low-rank row (multi-head latent
attention: DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient Mixture-of-Experts
Language Model").

Queries go through a low-rank row of their own: c_q = rmsnorm(W_dq h), q = W_uq c_q, per head
`dim` plain dimensions followed by `rot_dim` rotated ones.  W_dkv h gives `kv_rank` values, which
after an RMS norm are the row c, and `rot_dim` more, which after the rotation are a key part k_r
that all heads share.  Head h has keys W_uk[h] c (plain part) | k_r and values W_uv[h] c; the score
is (q_plain . k_plain + q_rot . k_r) * scale, causal, with an ordinary softmax.  The cache holds
c and k_r and nothing else: one "key/value head" whose key rows are c (`kv_rank` values) and whose
value rows are k_r (`rot_dim` values).

The step never expands keys or values.  Since q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c, the
query is carried into the row's space (one small product per head), the attention runs over c and
k_r directly with all heads sharing the cached rows, its output is a weighted sum of rows c per
head, and W_uv[h] expands that sum (one small product per head) before the output projection.

A layer with `shares_cache` has no W_dkv: its schedule entry names the entry whose cached rows it
reads (`Application.cache_of`), with its own queries, W_uk, W_uv and output projection.
"""
from __future__ import annotations

from .base import CacheNeed, Mixer, WeightSpec, build_part, register_part
from .spec import PartSpec


class LatentAttention(Mixer):

    def __init__(self, prefix: str, width: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, rotary: dict, shares_cache: bool = False, dq: str = "dq", uq: str = "uq",
                 dkv: str = "dkv", uk: str = "uk", uv: str = "uv", out: str = "o", norm_suffix: str = ".norm",
                 init_std: float = 0.02, out_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.heads, self.dim, self.rot_dim, self.vdim = int(width), int(heads), int(dim), int(rot_dim), int(vdim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.shares_cache = bool(shares_cache)
        if min(self.heads, self.dim, self.rot_dim, self.vdim, self.q_rank, self.kv_rank) <= 0:
            raise ValueError(f"latent attention {prefix!r}: every size is positive")
        if self.kv_rank > 1024 or self.rot_dim > 256:
            raise ValueError(f"latent attention {prefix!r}: a cached row of {self.kv_rank} + {self.rot_dim} values "
                             "(at most 1024 + 256)")
        self.rotary = build_part("position", PartSpec("rotary", prefix, dict(rotary)))
        if self.rotary.dims > self.rot_dim:
            raise ValueError(f"latent attention {prefix!r}: {self.rotary.dims} rotated dimensions of {self.rot_dim}")
        self.names = {n: prefix + s for n, s in dict(dq=dq, uq=uq, dkv=dkv, uk=uk, uv=uv, out=out).items()}
        self.norm_suffix, self.init_std, self.out_init_std = norm_suffix, init_std, out_init_std
        self.q_head = self.dim + self.rot_dim
        self.row = self.kv_rank + self.rot_dim        # what a query head is compared with: c | k_r

    def weight_specs(self):
        n, d = self.names, self.width
        specs = [WeightSpec(n["dq"], (self.q_rank, d), std=self.init_std),
                 WeightSpec(n["dq"] + self.norm_suffix, (self.q_rank,), mean=1.0, std=0.1),
                 WeightSpec(n["uq"], (self.heads * self.q_head, self.q_rank), std=self.init_std)]
        if not self.shares_cache:
            specs += [WeightSpec(n["dkv"], (self.row, d), std=self.init_std),
                      WeightSpec(n["dkv"] + self.norm_suffix, (self.kv_rank,), mean=1.0, std=0.1)]
        return specs + [WeightSpec(n["uk"], (self.heads * self.dim, self.kv_rank), std=self.init_std),
                        WeightSpec(n["uv"], (self.heads * self.vdim, self.kv_rank), std=self.init_std),
                        WeightSpec(n["out"], (d, self.heads * self.vdim), std=self.out_init_std)]

    def load(self, get, runtime):
        import torch
        n = self.names
        down = [runtime.matrix(get(n["dq"]))] + ([] if self.shares_cache else [runtime.matrix(get(n["dkv"]))])
        self.w_down = torch.cat(down).contiguous()            # one product for both down projections
        self.q_norm = runtime.vector(get(n["dq"] + self.norm_suffix))
        self.kv_norm = None if self.shares_cache else runtime.vector(get(n["dkv"] + self.norm_suffix))
        self.w_uq = runtime.matrix(get(n["uq"]))
        # per head: [kv_rank, dim], the transposed key expansion (carries a query into the row's space),
        # and [vdim, kv_rank], the value expansion as stored
        self.w_uk_t = runtime.matrix(get(n["uk"])).view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = runtime.matrix(get(n["uv"])).view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.rotary.load(get, runtime)

    def stream_weights(self):
        return [self.w_down, self.w_uq, self.w_out]

    def cache_need(self):
        return CacheNeed("full", 1, self.kv_rank, 0, 0, self.rot_dim)

    def _attend(self, ctx, h, app):
        import torch
        ops = ctx.ops
        if app.writes_cache == self.shares_cache:
            raise ValueError(f"latent attention {self.prefix!r}: a layer with a down projection of its own writes the "
                             "cache, a layer without one reads another entry's")
        down = ops.linear(h, self.w_down, None, out_dtype=torch.float32)             # [T, q_rank (| kv_rank | rot_dim)]
        # the two norms, the shared key part's rotation and the write of c and k_r into the cache in one launch
        c_q = ops.latent_rows(down, ctx.plan, self.q_rank, self.q_norm, self.kv_norm, self.kv_rank, self.rot_dim, self.eps,
                              self.rotary, app.cache if app.writes_cache else None, ctx.dtype)
        q = ops.linear(c_q, self.w_uq, None, out_dtype=ctx.dtype)                    # [T, heads * (dim | rot_dim)]
        rows = torch.empty((q.shape[0], self.heads * self.row), dtype=ctx.dtype, device=q.device)
        ops.head_linear(q, 0, self.q_head, self.w_uk_t, rows, 0, self.row)           # the plain parts, carried over
        self.rotary.rotate(ctx, q, rows, self.heads, self.dim, self.q_head, self.kv_rank, self.row, self.rot_dim)
        mixed = ops.latent_attention(rows, app.cache, ctx.plan, self.heads, self.kv_rank, self.rot_dim, self.scale, ctx.dtype)
        out = torch.empty((q.shape[0], self.heads * self.vdim), dtype=ctx.dtype, device=q.device)
        return ops.head_linear(mixed, 0, self.kv_rank, self.w_uv, out, 0, self.vdim)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._attend(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._attend(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "latent_attention", LatentAttention)
