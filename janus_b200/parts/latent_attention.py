"""Latent attention: keys and values are made from one small vector per token, and only that vector is cached.

With h the mixer's input: q = Wq h (heads x dim); c = rms_norm(Wdkv h) (size rank, a plain weight, eps inside the
root) is the token's latent; per head k = Wuk c (dim), v = Wuv c (vdim); score = (q . k) * scale; position i sees
every j <= i; softmax; the concatenated heads are projected by Wo.  There are no positions.  A layer may have no
Wdkv of its own and attend over the latents another layer cached (a place of the schedule that reads an earlier
place's cache), with its own Wuk, Wuv, queries and output.

Since k and v are linear in c, the products with Wuk and Wuv move to the other side of the attention:
  q . (Wuk_h c) = (Wuk_h^T q_h) . c          and          sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j),
so the attention is multi-query attention over the cached latents themselves (one key/value head of size rank whose
values are its keys), with queries Wuk_h^T Wq_h h and output Wo_h Wuv_h o_h.  Both pairs of matrices are multiplied
once when the weights are loaded (in float64, then rounded to the engine dtype), so a step runs two products, one
small kernel (queries to the engine dtype, the latent's norm and its append to the pages) and the library's
grouped-query attention with head size rank.  Cached per token: rank numbers, whatever the heads.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .attention import _check_kernel_limits, attend_paged, stored_head_size
from .base import KVSpec, Mixer, register_part
from .linear import Linear


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, rank: int, scale: float, eps: float,
                 own_latent: bool = True, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device = torch.device("cuda")):
        self.hidden_size, self.nh, self.dim, self.vdim, self.rank = (int(hidden_size), int(num_heads), int(dim),
                                                                      int(vdim), int(rank))
        self.scale, self.eps, self.own_latent = float(scale), float(eps), bool(own_latent)
        self.dtype, self.device = dtype, device
        # the attention runs with head size rank and one kv head (a rank that the bfloat16 kernels do not take is
        # stored as the next size they take: zero rows in the queries' matrix, zero columns in the output's)
        self.rank_stored = stored_head_size(self.rank, dtype)
        _check_kernel_limits(self.nh, 1, self.rank_stored, dtype)
        self.q_width = self.nh * self.rank_stored
        # rows: the queries in latent space, then (own latent) the latent's projection
        self.proj = Linear(hidden_size, self.q_width + (self.rank if self.own_latent else 0), dtype, device,
                           name="q_dkv" if self.own_latent else "q", pad_width=True)
        self.q_only: Optional[Linear] = None
        self.o = Linear(self.q_width, hidden_size, dtype, device, name="o", pad_width=True)
        self.norm_weight: Optional[torch.Tensor] = None

    def cache_spec(self) -> Optional[KVSpec]:
        return KVSpec(1, self.rank_stored, values_are_keys=True) if self.own_latent else None

    def weight_shapes(self):
        shapes = {"q": ((self.nh * self.dim, self.hidden_size), "normal"),
                  "uk": ((self.nh * self.dim, self.rank), "normal"), "uv": ((self.nh * self.vdim, self.rank), "normal"),
                  "o": ((self.hidden_size, self.nh * self.vdim), "normal")}
        if self.own_latent:
            shapes.update(dkv=((self.rank, self.hidden_size), "normal"), dkv_norm=((self.rank,), "ones"))
        return shapes

    def load(self, q, uk, uv, o, dkv=None, dkv_norm=None) -> None:
        H, d, e, r, W = self.nh, self.dim, self.vdim, self.rank, self.hidden_size
        for name, t, shape in (("q", q, (H * d, W)), ("uk", uk, (H * d, r)), ("uv", uv, (H * e, r)), ("o", o, (W, H * e))):
            if tuple(t.shape) != shape:
                raise ValueError(f"weight '{name}' of shape {tuple(t.shape)} does not fit {shape}")
        f64 = lambda t: t.to(device=self.device, dtype=torch.float64)      # noqa: E731
        # queries into latent space: rows [head][rank] = Wuk_h^T Wq_h
        rp = self.rank_stored
        q_latent = torch.zeros((H, rp, W), dtype=torch.float64, device=self.device)
        q_latent[:, :r] = torch.einsum("hdr,hdw->hrw", f64(uk).view(H, d, r), f64(q).view(H, d, W))
        q_latent = q_latent.reshape(H * rp, W)
        # the output from latent space: columns [head][rank] = Wo_h Wuv_h
        o_latent = torch.zeros((W, H, rp), dtype=torch.float64, device=self.device)
        o_latent[:, :, :r] = torch.einsum("whe,her->whr", f64(o).view(W, H, e), f64(uv).view(H, e, r))
        o_latent = o_latent.reshape(W, H * rp)
        if self.own_latent:
            if dkv is None or dkv_norm is None or tuple(dkv_norm.shape) != (r,):
                raise ValueError("a latent attention layer with a latent of its own needs 'dkv' and 'dkv_norm'")
            self.proj.load([q_latent, f64(dkv)])
            self.norm_weight = dkv_norm.to(device=self.device, dtype=torch.float32).contiguous()
        else:
            self.proj.load([q_latent])
        self.q_only = self.proj.first_rows(self.q_width)
        self.o.load([o_latent])

    def _linear(self, writes_cache: bool) -> Linear:
        if writes_cache and not self.own_latent:
            raise ValueError("this latent attention layer has no latent of its own: it must read another place's cache")
        return self.proj if writes_cache else self.q_only

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        lin = self._linear(writes_cache)
        if lin is None or not lin.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("latent_proj", (tokens, lin.out_features), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        T = x.shape[0]
        ws = ctx.workspace
        group = cache_view.group
        lin = self._linear(writes_cache)
        proj = ws.get("latent_proj", (T, lin.out_features), torch.float32)
        lin.forward(x, proj, y_is_zero=scratch_cleared)
        q = ws.get("latent_q", (T, self.q_width), self.dtype)
        ops.latent_prep(proj, self.q_width, self.rank, self.norm_weight, self.eps, q, group.dest_rows, cache_view.k,
                        write_c=writes_cache, stored_rank=self.rank_stored)
        attn = ws.get("latent_attn", (T, self.q_width), self.dtype)
        attend_paged(q, cache_view.k, cache_view.k, attn, ctx, group, self.nh, 1, self.rank_stored, 0, self.scale)
        self.o.forward_add(attn, residual)


register_part("mixer", "latent_attention", LatentAttention)
