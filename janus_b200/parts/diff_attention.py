"""Differential attention over the paged cache.

Every query head has two attention maps over the same values.  With h the mixer's input:
q = Wq h (heads x 2 x dim, a head's rows are [map 1, map 2]), k = Wk h (kv_heads x 2 x dim), v = Wv h
(kv_heads x vdim); query head i uses key/value head floor(i / (heads / kv_heads)).  Optionally a short causal
convolution over time runs on every channel of q, k and v right after the projection
(y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence's start; the last taps - 1 projected
values of a sequence are state), then rotary positions turn the leading dimensions of every q and k vector.
Scores are (q . k) * scale; position i sees j <= i with i - j < window or j < keep_first (window 0: all);
softmax per map; o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number per
layer; o is divided by its root mean square over the head's vdim values (eps inside the root, no weight) and
multiplied by (1 - diff); the concatenated heads are projected by Wo.

The cache keeps the two maps of a key/value head as neighbouring key heads of size dim and the values with
heads and a size of their own (`KVSpec.n_value_heads`, `value_dim`); a window gives pages back once every
later query has left them, except those of the kept first keys.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..kernels import ops
from .base import KVSpec, Mixer, PartSpec, StateSpec, register_part, shared_part
from .linear import Linear


class DifferentialAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 diff: float, eps: float, conv_taps: int = 0, window: int = 0, keep_first: int = 0,
                 position: Optional[PartSpec] = None, rotary_dims: int = 0,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
        if not 1 <= vdim <= 256:
            raise ValueError(f"a value size of {vdim} is not supported by the attention kernel (1 to 256)")
        if position is not None and (rotary_dims % 2 or not 0 < rotary_dims <= dim):
            raise ValueError(f"{rotary_dims} rotated dimensions do not fit vectors of size {dim}")
        self.hidden_size, self.nh, self.nkv = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim = int(dim), int(vdim)
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.taps = int(conv_taps) if conv_taps and conv_taps > 1 else (1 if conv_taps == 1 else 0)
        self.window, self.keep_first = int(window), int(keep_first) if window else 0
        self.dtype, self.device = dtype, device
        self.position = shared_part("position", position, dtype, device) if position is not None else None
        self.rotary_dims = int(rotary_dims) if position is not None else 0
        self.q_width, self.k_width, self.v_width = self.nh * 2 * self.dim, self.nkv * 2 * self.dim, self.nkv * self.vdim
        self.channels = self.q_width + self.k_width + self.v_width
        self.qkv = Linear(hidden_size, self.channels, dtype, device, name="qkv", pad_width=True)
        self.o = Linear(self.nh * self.vdim, hidden_size, dtype, device, name="o", pad_width=True)
        self.conv_weight: Optional[torch.Tensor] = None
        self.lam = self.diff

    def cache_spec(self) -> Tuple:
        kv = KVSpec(2 * self.nkv, self.dim, self.window, self.keep_first, n_value_heads=self.nkv, value_dim=self.vdim)
        if self.taps > 1:
            return (kv, StateSpec((self.taps - 1, self.channels)))
        return kv

    def limit_positions(self, n: int) -> None:
        limit = getattr(self.position, "limit_positions", None)
        if limit is not None:
            limit(n)

    def weight_shapes(self):
        shapes = {"q": ((self.q_width, self.hidden_size), "normal"), "k": ((self.k_width, self.hidden_size), "normal"),
                  "v": ((self.v_width, self.hidden_size), "normal"),
                  "o": ((self.hidden_size, self.nh * self.vdim), "normal"),
                  "lq1": ((self.dim,), "normal"), "lk1": ((self.dim,), "normal"),
                  "lq2": ((self.dim,), "normal"), "lk2": ((self.dim,), "normal")}
        if self.taps:
            shapes.update(q_conv=((self.q_width, self.taps), "normal"), k_conv=((self.k_width, self.taps), "normal"),
                          v_conv=((self.v_width, self.taps), "normal"))
        return shapes

    def load(self, q, k, v, o, lq1, lk1, lq2, lk2, q_conv=None, k_conv=None, v_conv=None) -> None:
        self.qkv.load([q, k, v])
        self.o.load([o])
        f = [t.to(torch.float32).cpu() for t in (lq1, lk1, lq2, lk2)]
        # one number per layer, made once in float32
        self.lam = float(torch.exp((f[0] * f[1]).sum()) - torch.exp((f[2] * f[3]).sum()) + self.diff)
        if self.taps:
            w = torch.cat([t.to(torch.float32) for t in (q_conv, k_conv, v_conv)], dim=0)
            if tuple(w.shape) != (self.channels, self.taps):
                raise ValueError(f"convolution weights of shape {tuple(w.shape)} do not fit ({self.channels}, {self.taps})")
            self.conv_weight = w.to(self.device).contiguous()

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the read before this mixer clears it in the same launch."""
        if not self.qkv.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("diff_qkv", (tokens, self.channels), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("differential attention writes its own keys and values; it cannot read another place's")
        T = x.shape[0]
        ws = ctx.workspace
        group = cache_view.group
        proj = ws.get("diff_qkv", (T, self.channels), torch.float32)
        self.qkv.forward(x, proj, y_is_zero=scratch_cleared)
        table = self.position.fused_rotary_table() if self.position is not None else None
        q = ws.get("diff_q", (T, self.q_width), torch.float32)
        ops.conv_rope_cache(proj, self.conv_weight, self.taps, cache_view.state if self.taps > 1 else None,
                            ctx.token_seq, ctx.q_start, ctx.seq_slot, ctx.positions, table, self.rotary_dims, q,
                            group.dest_rows, cache_view.k, cache_view.v, self.nh, self.nkv, self.dim, self.vdim,
                            group.page_size, update_state=ctx.is_decode)
        if self.taps > 1 and not ctx.is_decode:
            ops.conv_state_update(proj, cache_view.state, self.taps, ctx.q_start, ctx.seq_slot, ctx.n_seqs)
        attn = ws.get("diff_attn", (T, self.nh * self.vdim), self.dtype)
        if (self.dtype == torch.bfloat16 and not ctx.is_decode
                and ops.diff_attention_prefill_supported(self.nh, self.nkv, self.dim, self.vdim, group.page_size)):
            # prompt steps in bfloat16: the tensor-core kernel, a tile of tokens x the heads of a key/value head
            ops.diff_attention_prefill(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.q_start, ctx.kv_len,
                                       ctx.n_seqs, ctx.max_q_len, self.nh, self.nkv, self.dim, self.vdim, group.page_size,
                                       self.window, self.keep_first, self.scale, self.lam, self.eps, 1.0 - self.diff)
        else:
            ops.diff_attention(q, cache_view.k, cache_view.v, attn, group.block_table, ctx.token_seq, ctx.positions,
                               self.nh, self.nkv, self.dim, self.vdim, group.page_size, self.window, self.keep_first,
                               self.scale, self.lam, self.eps, 1.0 - self.diff)
        self.o.forward_add(attn, residual)


register_part("mixer", "differential_attention", DifferentialAttention)
