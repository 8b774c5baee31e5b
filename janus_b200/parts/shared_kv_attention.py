"""Grouped-query attention whose values are its keys as projected, over the paged cache.

With h the mixer's input: q = Wq h + bq (heads x dim), k = Wk h + bk (kv_heads x dim); the values are k itself, as
projected (there is no value projection).  q and k are then divided by their root mean square over the WHOLE
projection (all heads at once, eps inside the root) and multiplied by a weight of that size; rotary positions turn
the leading dimensions of every head of q and k; score = (q . k) * scale; position i sees j with 0 <= i - j < window
(window 0: every j <= i); softmax; query head i uses key/value head floor(i / (heads / kv_heads)); the
concatenated heads are projected by Wo.

q and k are one stacked product whose float32 accumulators one kernel turns into the queries and the cache rows
(bias, value append, norm, rotation, key append: `ops.qk_norm_rope_cache`); the attention itself is the library's
grouped-query attention (keys and values have the same size here; a head size that its bfloat16 kernels do not take is
stored as the next one they take, with zero columns).  A window lets the cache give pages back.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .attention import _check_kernel_limits, attend_paged, stored_head_size
from .base import KVSpec, Mixer, PartSpec, register_part, shared_part
from .linear import Linear


class SharedKVAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, scale: float, eps: float,
                 window: int = 0, position: Optional[PartSpec] = None, rotary_dims: int = 0, bias: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
        if position is not None and (rotary_dims % 2 or not 0 < rotary_dims <= dim):
            raise ValueError(f"{rotary_dims} rotated dimensions do not fit vectors of size {dim}")
        self.hidden_size, self.nh, self.nkv, self.dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(dim)
        self.scale, self.eps, self.window, self.bias = float(scale), float(eps), int(window), bool(bias)
        self.dtype, self.device = dtype, device
        self.dim_stored = stored_head_size(self.dim, dtype)
        _check_kernel_limits(self.nh, self.nkv, self.dim_stored, dtype)
        self.position = shared_part("position", position, dtype, device) if position is not None else None
        self.rotary_dims = int(rotary_dims) if position is not None else 0
        self.q_width, self.k_width = self.nh * self.dim, self.nkv * self.dim
        self.qk = Linear(hidden_size, self.q_width + self.k_width, dtype, device, name="qk", pad_width=True)
        self.q_only: Optional[Linear] = None             # view of the q rows, for places that read another cache
        self.o = Linear(self.nh * self.dim_stored, hidden_size, dtype, device, name="o", pad_width=True)
        self.bq = self.bk = self.wq = self.wk = None

    def cache_spec(self) -> KVSpec:
        return KVSpec(self.nkv, self.dim_stored, self.window)

    def limit_positions(self, n: int) -> None:
        limit = getattr(self.position, "limit_positions", None)
        if limit is not None:
            limit(n)

    def weight_shapes(self):
        shapes = {"q": ((self.q_width, self.hidden_size), "normal"), "k": ((self.k_width, self.hidden_size), "normal"),
                  "q_norm": ((self.q_width,), "ones"), "k_norm": ((self.k_width,), "ones"),
                  "o": ((self.hidden_size, self.q_width), "normal")}
        if self.bias:
            shapes.update(q_bias=((self.q_width,), "normal"), k_bias=((self.k_width,), "normal"))
        return shapes

    def load(self, q, k, q_norm, k_norm, o, q_bias=None, k_bias=None) -> None:
        self.qk.load([q, k])
        self.q_only = self.qk.first_rows(self.q_width)
        if tuple(o.shape) != (self.hidden_size, self.q_width):
            raise ValueError(f"weight 'o' of shape {tuple(o.shape)} does not fit ({self.hidden_size}, {self.q_width})")
        if self.dim_stored != self.dim:          # zero columns where the stored heads have their extra columns
            wide = torch.zeros((self.hidden_size, self.nh, self.dim_stored), dtype=o.dtype, device=o.device)
            wide[:, :, : self.dim] = o.view(self.hidden_size, self.nh, self.dim)
            o = wide.view(self.hidden_size, self.nh * self.dim_stored)
        self.o.load([o])

        def f32(t, n):
            if tuple(t.shape) != (n,):
                raise ValueError(f"a vector of shape {tuple(t.shape)} does not fit ({n},)")
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.wq, self.wk = f32(q_norm, self.q_width), f32(k_norm, self.k_width)
        if self.bias:
            self.bq, self.bk = f32(q_bias, self.q_width), f32(k_bias, self.k_width)

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        proj = self.qk if writes_cache else self.q_only
        if proj is None or not proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("skv_proj", (tokens, proj.out_features), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        T = x.shape[0]
        ws = ctx.workspace
        group = cache_view.group
        lin = self.qk if writes_cache else self.q_only
        proj = ws.get("skv_proj", (T, lin.out_features), torch.float32)
        lin.forward(x, proj, y_is_zero=scratch_cleared)
        table = self.position.fused_rotary_table() if self.position is not None else None
        q = ws.get("q_rot", (T, self.nh * self.dim_stored), self.dtype)
        ops.qk_norm_rope_cache(proj, self.bq, self.bk, self.wq, self.wk, self.eps, table, self.rotary_dims,
                               ctx.positions, q, group.dest_rows, cache_view.k, cache_view.v, self.nh, self.nkv,
                               self.dim, group.page_size, write_kv=writes_cache, stored_dim=self.dim_stored)
        attn = ws.get("attn_out", (T, self.nh * self.dim_stored), self.dtype)
        attend_paged(q, cache_view.k, cache_view.v, attn, ctx, group, self.nh, self.nkv, self.dim_stored, self.window,
                     self.scale)
        self.o.forward_add(attn, residual)


register_part("mixer", "shared_kv_attention", SharedKVAttention)
