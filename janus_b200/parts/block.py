"""Arrangement of a layer's parts.  Pre-norm, as the reference's block:
h1 = x + mixer(norm1(x)); out = h1 + feed_forward(norm2(h1))
(crates/janus-engine/src/model/block.rs:223-233,355-380,447-455).  The parts
add into the float32 residual stream themselves."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import register_part


class PreNormBlock:
    """`parts`: mixer_norm and mixer, and, unless the layer has no feed-forward,
    feed_forward_norm and feed_forward."""

    def __init__(self, parts: dict, hidden_size: int, dtype: torch.dtype):
        unknown = set(parts) - {"mixer_norm", "mixer", "feed_forward_norm", "feed_forward"}
        if unknown:
            raise ValueError(f"the pre_norm arrangement has no use for the parts {sorted(unknown)}")
        try:
            self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
            self.feed_forward = parts.get("feed_forward")
            self.feed_forward_norm = parts["feed_forward_norm"] if self.feed_forward is not None else None
        except KeyError as e:
            raise ValueError(f"the pre_norm arrangement needs the part {e.args[0]!r}") from None
        self.hidden_size, self.dtype = hidden_size, dtype

    def forward(self, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True) -> None:
        x = ctx.workspace.get("normed", (residual.shape[0], self.hidden_size), self.dtype)
        # a mixer may name a scratch buffer that it wants zeroed; the norm before it does that in passing
        wants = getattr(self.mixer, "scratch_to_clear", None)
        scratch = wants(ctx, residual.shape[0], writes_cache) if wants is not None else None
        if scratch is not None:
            self.mixer_norm.forward(residual, x, clear=scratch)
            self.mixer.forward(x, residual, ctx, cache_view, writes_cache, scratch_cleared=True)
        else:
            self.mixer_norm.forward(residual, x)
            self.mixer.forward(x, residual, ctx, cache_view, writes_cache)
        if self.feed_forward is None:
            return
        self.feed_forward_norm.forward(residual, x)
        self.feed_forward.forward(x, residual, ctx)


register_part("arrangement", "pre_norm", PreNormBlock)


class HyperConnectedBlock:
    """Pre-norm with several residual streams: each sublayer reads the normed weighted sum of the
    streams through its connection and its output is mixed back into every stream
    (`parts.connection`).  `parts`: mixer_norm, mixer, mixer_connection, and, unless the layer has
    no feed-forward, feed_forward_norm, feed_forward, feed_forward_connection.  The residual of a
    step is float32 [T, streams * hidden_size]; a sublayer adds its output into a zeroed float32
    [T, hidden_size] buffer, as it would into a single residual stream."""

    def __init__(self, parts: dict, hidden_size: int, dtype: torch.dtype):
        unknown = set(parts) - {"mixer_norm", "mixer", "mixer_connection", "feed_forward_norm", "feed_forward",
                                "feed_forward_connection"}
        if unknown:
            raise ValueError(f"the hyper_pre_norm arrangement has no use for the parts {sorted(unknown)}")
        try:
            self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
            self.mixer_connection = parts["mixer_connection"]
            self.feed_forward = parts.get("feed_forward")
            self.feed_forward_norm = parts["feed_forward_norm"] if self.feed_forward is not None else None
            self.feed_forward_connection = parts["feed_forward_connection"] if self.feed_forward is not None else None
        except KeyError as e:
            raise ValueError(f"the hyper_pre_norm arrangement needs the part {e.args[0]!r}") from None
        self.hidden_size, self.dtype = hidden_size, dtype

    def forward(self, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True) -> None:
        T = residual.shape[0]
        x = ctx.workspace.get("normed", (T, self.hidden_size), self.dtype)
        y = ctx.workspace.get("sublayer_out", (T, self.hidden_size), torch.float32)
        # a sublayer's write waits for the read that follows it (the next sublayer's, also the next layer's) and
        # runs in the same launch; the model flushes the last one before its final norm
        pending = ctx.pending_write
        ctx.pending_write = None
        # a mixer may name a scratch buffer that it wants zeroed; the read before it does that in passing
        wants = getattr(self.mixer, "scratch_to_clear", None)
        scratch = wants(ctx, T, writes_cache) if wants is not None else None
        if pending is not None and pending[1] is y and hasattr(pending[0], "write_then_read"):
            pending[0].write_then_read(residual, y, self.mixer_connection, self.mixer_norm, x, clear2=scratch)
        else:
            if pending is not None:
                pending[0].write(residual, pending[1])
            self.mixer_connection.read(residual, self.mixer_norm, x, clear=y, clear2=scratch)
        if scratch is not None:
            self.mixer.forward(x, y, ctx, cache_view, writes_cache, scratch_cleared=True)
        else:
            self.mixer.forward(x, y, ctx, cache_view, writes_cache)
        last = self.mixer_connection
        if self.feed_forward is not None:
            if hasattr(last, "write_then_read"):
                last.write_then_read(residual, y, self.feed_forward_connection, self.feed_forward_norm, x)
            else:
                last.write(residual, y)
                self.feed_forward_connection.read(residual, self.feed_forward_norm, x, clear=y)
            self.feed_forward.forward(x, y, ctx)
            last = self.feed_forward_connection
        ctx.pending_write = (last, y)


register_part("arrangement", "hyper_pre_norm", HyperConnectedBlock)


class _NormedWrite:
    """A sublayer's output that still has to be normed and added to the residual stream; the arrangement leaves it
    with the step (`ctx.pending_write`) so that the next sublayer's read happens in the same launch."""

    def __init__(self, norm, mult: float):
        self.norm, self.mult = norm, mult

    def write(self, residual: torch.Tensor, y: torch.Tensor) -> None:
        self.norm.add_normed(y, residual, self.mult)

    def write_then_cast(self, residual: torch.Tensor, y: torch.Tensor, x: torch.Tensor, clear=None) -> None:
        self.norm.add_normed(y, residual, self.mult, x_out=x, clear=clear)


class OutputNormBlock:
    """The norm sits on each sublayer's OUTPUT, and what joins the residual stream is multiplied by a constant:
    x <- x + mult * norm1(mixer(x)); x <- x + mult * norm2(feed_forward(x)).  The sublayers read x itself (cast to
    the engine dtype).  `parts`: mixer and mixer_norm, and, unless the layer has no feed-forward, feed_forward and
    feed_forward_norm.  A sublayer adds its output into a zeroed float32 [T, hidden_size] buffer; one launch then
    norms it, adds it to the residual stream, zeroes the buffer and casts the stream for the sublayer that follows
    (also the next layer's mixer: the last sum of a layer waits for it)."""

    def __init__(self, parts: dict, hidden_size: int, dtype: torch.dtype, residual_mult: float = 1.0):
        unknown = set(parts) - {"mixer_norm", "mixer", "feed_forward_norm", "feed_forward"}
        if unknown:
            raise ValueError(f"the output_norm arrangement has no use for the parts {sorted(unknown)}")
        try:
            self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
            self.feed_forward = parts.get("feed_forward")
            self.feed_forward_norm = parts["feed_forward_norm"] if self.feed_forward is not None else None
        except KeyError as e:
            raise ValueError(f"the output_norm arrangement needs the part {e.args[0]!r}") from None
        self.hidden_size, self.dtype, self.mult = hidden_size, dtype, float(residual_mult)
        self._mixer_write = _NormedWrite(self.mixer_norm, self.mult)
        self._ff_write = _NormedWrite(self.feed_forward_norm, self.mult) if self.feed_forward is not None else None

    def forward(self, residual: torch.Tensor, ctx, cache_view, writes_cache: bool = True) -> None:
        T = residual.shape[0]
        x = ctx.workspace.get("normed", (T, self.hidden_size), self.dtype)
        y = ctx.workspace.get("sublayer_out", (T, self.hidden_size), torch.float32)
        pending = ctx.pending_write
        ctx.pending_write = None
        # a mixer may name a scratch buffer that it wants zeroed; the launch before it does that in passing
        wants = getattr(self.mixer, "scratch_to_clear", None)
        scratch = wants(ctx, T, writes_cache) if wants is not None else None
        if pending is not None and pending[1] is y and hasattr(pending[0], "write_then_cast"):
            pending[0].write_then_cast(residual, y, x, clear=scratch)
        else:
            if pending is not None:
                pending[0].write(residual, pending[1])
            if y.numel() % 4 == 0:          # the cast's launch also zeroes the sublayers' buffer
                self.mixer_norm.add_normed(None, residual, self.mult, x_out=x, clear=scratch, clear2=y)
            else:
                y.zero_()
                self.mixer_norm.add_normed(None, residual, self.mult, x_out=x, clear=scratch)
        if scratch is not None:
            self.mixer.forward(x, y, ctx, cache_view, writes_cache, scratch_cleared=True)
        else:
            self.mixer.forward(x, y, ctx, cache_view, writes_cache)
        last = self._mixer_write
        if self.feed_forward is not None:
            last.write_then_cast(residual, y, x)
            self.feed_forward.forward(x, y, ctx)
            last = self._ff_write
        ctx.pending_write = (last, y)


register_part("arrangement", "output_norm", OutputNormBlock)
