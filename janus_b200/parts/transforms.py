"""Transforms of whole tensors of a model (`ModelSpec.embedding_transforms`, `logit_transforms`).

`scale_soft_cap`: t <- cap * tanh(t * scale / cap) in place on float32 (a scale on the logits and
a soft cap that keeps them inside (-cap, cap)); without a cap it is the scale alone."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Transform, register_part


class ScaleSoftCap(Transform):
    def __init__(self, scale: float = 1.0, cap: Optional[float] = None, dtype=None, device=None):
        self.scale = float(scale)
        self.cap = 0.0 if cap is None else float(cap)
        if cap is not None and not self.cap > 0.0:
            raise ValueError(f"a soft cap must be positive, got {cap}")

    def plain_scale(self):
        """The factor, if this transform is a multiplication and nothing else (the model then multiplies where
        it makes the tensor, without a launch of this transform's own); else None."""
        return self.scale if self.cap == 0.0 else None

    def forward(self, t: torch.Tensor, ctx) -> None:
        ops.scale_softcap(t, self.scale, self.cap)


register_part("transform", "scale_soft_cap", ScaleSoftCap)
