"""Linear attention with a per-head decay ("lightning attention"), a mixer with a state of fixed size.

With h the mixer's input: q = silu(Wq h), k = silu(Wk h) (heads x dim), v = silu(Wv h) (heads x vdim); per
head the state S (dim x vdim, float32, zero at a sequence's start) follows S_t = decay_h S_(t-1) + k_t v_t^T
and the head's output is o_t = S_t^T q_t, with no other scale.  The concatenated heads are divided by their
root mean square (eps inside the root), multiplied by a weight and by sigmoid(Wg h), and projected by Wo.

q, k, v and g are one stacked product whose float32 accumulators the recurrence reads; the state lives in the
cache's fixed-size state area, one [heads, dim, vdim] block per sequence slot, so prompts, portions of prompts
and single tokens all run the same kernel from whatever the steps before left.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..kernels import ops
from .base import Mixer, StateSpec, register_part
from .linear import Linear


class LightningAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 dtype: torch.dtype = torch.bfloat16, device: torch.device = torch.device("cuda")):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays are given for {num_heads} heads")
        if not 1 <= dim <= 256:
            raise ValueError(f"a key size of {dim} is not supported by the recurrence kernel (1 to 256)")
        self.hidden_size, self.nh, self.dim, self.vdim = int(hidden_size), int(num_heads), int(dim), int(vdim)
        self.eps = float(eps)
        self.dtype, self.device = dtype, device
        self.qk_width, self.v_width = self.nh * self.dim, self.nh * self.vdim
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=device)
        # rows of the stacked product: q, k, v, g
        self.proj = Linear(hidden_size, 2 * self.qk_width + 2 * self.v_width, dtype, device, name="qkvg", pad_width=True)
        self.o = Linear(self.v_width, hidden_size, dtype, device, name="o", pad_width=True)
        self.norm_weight: Optional[torch.Tensor] = None

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.nh, self.dim, self.vdim))

    def weight_shapes(self):
        return {"q": ((self.qk_width, self.hidden_size), "normal"), "k": ((self.qk_width, self.hidden_size), "normal"),
                "v": ((self.v_width, self.hidden_size), "normal"), "g": ((self.v_width, self.hidden_size), "normal"),
                "o": ((self.hidden_size, self.v_width), "normal"), "norm": ((self.v_width,), "ones")}

    def load(self, q, k, v, g, o, norm) -> None:
        self.proj.load([q, k, v, g])
        self.o.load([o])
        if tuple(norm.shape) != (self.v_width,):
            raise ValueError(f"norm weight of shape {tuple(norm.shape)} does not fit ({self.v_width},)")
        if self.dtype == torch.float32:
            norm = norm.to(torch.float32)
        self.norm_weight = norm.to(self.device).contiguous()

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projections' float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the read before this mixer clears it in the same launch."""
        if not self.proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("lightning_proj", (tokens, self.proj.out_features), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("a lightning mixer cannot read another place's state: its state is its own")
        T = x.shape[0]
        ws = ctx.workspace
        proj = ws.get("lightning_proj", (T, self.proj.out_features), torch.float32)
        self.proj.forward(x, proj, y_is_zero=scratch_cleared)
        o = ws.get("lightning_o", (T, self.v_width), torch.float32)
        ops.lightning_scan(proj, 0, self.qk_width, 2 * self.qk_width, o, cache_view.state, ctx.q_start, ctx.seq_slot,
                           self.decay, ctx.n_seqs, self.nh, self.dim, self.vdim, ctx.max_q_len, ws)
        gated = ws.get("lightning_gated", (T, self.v_width), self.dtype)
        ops.gated_rmsnorm(o, self.norm_weight, proj[:, 2 * self.qk_width + self.v_width:], self.eps, gated)
        self.o.forward_add(gated, residual)


register_part("mixer", "lightning_attention", LightningAttention)
