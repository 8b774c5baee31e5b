"""The selective state-space mixer in its Mamba-2 form (one scalar decay per head and token), a mixer with a state
of fixed size.

With h the mixer's input, inner = heads * vdim, N the state size and G groups: Win h is laid out as
[z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C together pass a short causal convolution per channel
(weight [channels, taps] whose last column meets the current token, a bias, zeros before a sequence's start) and
SiLU.  dt = softplus(dt + dt_bias); per head h (group floor(h / (heads / G))) the state S (N x vdim, float32, zero at
a sequence's start) follows S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T and y_t = S_t^T C_t + D_h x_t.
The concatenated heads are multiplied by silu(z), divided in each of `norm_groups` equal pieces by the piece's root
mean square (eps inside the root), multiplied by a weight and projected by Wo.

The projection is one product whose float32 accumulators the convolution, the recurrence and the gate read; the
recurrence's state and the convolution's last taps - 1 inputs live side by side in one block of the cache's
fixed-size state area per sequence slot, so prompts, portions of prompts and single tokens all run the same
kernels from whatever the steps before left.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer, StateSpec, register_part
from .linear import Linear


class Mamba2Mixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, vdim: int, state: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device = torch.device("cuda")):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads are not a multiple of {groups} groups")
        if not 1 <= state <= 256:
            raise ValueError(f"a state size of {state} is not supported by the recurrence kernel (1 to 256)")
        if conv_taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {conv_taps}")
        self.hidden_size, self.nh, self.vdim, self.n_state, self.groups = (int(hidden_size), int(num_heads), int(vdim),
                                                                           int(state), int(groups))
        self.taps, self.norm_groups, self.eps = int(conv_taps), int(norm_groups), float(eps)
        self.inner = self.nh * self.vdim
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels do not fall into {self.norm_groups} equal pieces for the norm")
        self.dtype, self.device = dtype, device
        self.bc_width = self.groups * self.n_state
        self.channels = self.inner + 2 * self.bc_width                # what the convolution sees: x, B, C
        self.width = 2 * self.inner + 2 * self.bc_width + self.nh     # z, x, B, C, dt
        self.in_proj = Linear(hidden_size, self.width, dtype, device, name="in", pad_width=True)
        self.o = Linear(self.inner, hidden_size, dtype, device, name="o", pad_width=True)
        # one block of state per slot: the recurrence's [heads, N, vdim], then the convolution's [taps - 1, channels]
        self.scan_floats = self.nh * self.n_state * self.vdim
        self.state_floats = self.scan_floats + (self.taps - 1) * self.channels
        self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_weight = None

    def cache_spec(self) -> StateSpec:
        return StateSpec((self.state_floats,))

    def weight_shapes(self):
        return {"in_proj": ((self.width, self.hidden_size), "normal"), "conv": ((self.channels, self.taps), "normal"),
                "conv_bias": ((self.channels,), "normal"), "dt_bias": ((self.nh,), "normal"),
                "A_log": ((self.nh,), "normal"), "D": ((self.nh,), "ones"), "norm": ((self.inner,), "ones"),
                "o": ((self.hidden_size, self.inner), "normal")}

    def load(self, in_proj, conv, conv_bias, dt_bias, A_log, D, norm, o) -> None:
        self.in_proj.load([in_proj])
        self.o.load([o])

        def f32(name, t, shape):
            if tuple(t.shape) != shape:
                raise ValueError(f"'{name}' of shape {tuple(t.shape)} does not fit {shape}")
            return t.to(device=self.device, dtype=torch.float32).contiguous()

        self.conv_w = f32("conv", conv, (self.channels, self.taps))
        self.conv_b = f32("conv_bias", conv_bias, (self.channels,))
        self.dt_bias, self.a_log, self.d_skip = (f32("dt_bias", dt_bias, (self.nh,)), f32("A_log", A_log, (self.nh,)),
                                                 f32("D", D, (self.nh,)))
        self.norm_weight = f32("norm", norm, (self.inner,))

    def scratch_to_clear(self, ctx, tokens: int, writes_cache: bool = True) -> Optional[torch.Tensor]:
        """The projection's float32 buffer, if this step's product adds slices of K into it (decode-sized steps):
        the launch before this mixer clears it in passing."""
        if not self.in_proj.meets_by_adds(tokens, torch.float32):
            return None
        buf = ctx.workspace.get("mamba2_proj", (tokens, self.width), torch.float32)
        return buf if buf.numel() % 4 == 0 else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True,
                scratch_cleared: bool = False) -> None:
        if not writes_cache:
            raise ValueError("a state-space mixer cannot read another place's state: its state is its own")
        T = x.shape[0]
        ws = ctx.workspace
        state = cache_view.state                                      # float32 [slots, state_floats]
        proj = ws.get("mamba2_proj", (T, self.width), torch.float32)
        self.in_proj.forward(x, proj, y_is_zero=scratch_cleared)
        xbc = ws.get("mamba2_xbc", (T, self.channels), torch.float32)
        ops.causal_conv_silu(proj, self.inner, self.channels, self.conv_w, self.conv_b, self.taps, state,
                             self.scan_floats, ctx.token_seq, ctx.q_start, ctx.seq_slot, xbc, ctx.n_seqs,
                             single_tokens=ctx.is_decode)
        y = ws.get("mamba2_y", (T, self.inner), torch.float32)
        ops.mamba2_scan(xbc, self.inner, self.inner + self.bc_width, proj[:, self.inner + self.channels:],
                        self.dt_bias, self.a_log, self.d_skip, y, state, 0, ctx.q_start, ctx.seq_slot, ctx.n_seqs,
                        self.nh, self.groups, self.n_state, self.vdim, ctx.max_q_len, ws)
        gated = ws.get("mamba2_gated", (T, self.inner), self.dtype)
        ops.gated_group_rmsnorm(y, proj[:, : self.inner], self.norm_weight, self.eps, self.norm_groups, gated)
        self.o.forward_add(gated, residual)


register_part("mixer", "mamba2", Mamba2Mixer)
