"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * (offset + w), float32 inside; offset 0 uses the weight as stored,
offset 1 is for checkpoints that store the weight's deviation from one (``NormSpec.weight_offset``).
With ``NormSpec.groups`` = n > 1 the row is cut into n equal runs and every run is divided by its own root mean square;
the weight still spans the whole row.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:189-200 (eps inside the
sqrt; no ``1 + w``); kernel engine/engine-cuda/kernels/norm_rope.cu:37-80.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..weights.loader import WeightSpec
from .base import NORMS, Norm


class DeferredNorm:
    """An RMS norm that has not run yet: the float32 rows, the norm's weight and eps.  A part that says
    ``folds_norm = True`` may be handed one instead of normalised rows; its first matrix product then takes the
    norm in (the kernel scales by the weight on the way in and by the rows' 1/sqrt(mean(x^2) + eps) on the way
    out), or the part calls ``materialize()`` and goes on as with any tensor."""

    def __init__(self, norm: "RMSNorm", x: torch.Tensor, ctx):
        self.norm, self.x, self.ctx = norm, x, ctx
        self.weight, self.eps = norm.weight, norm.spec.eps
        self.shape, self.dtype = x.shape, ctx.dtype

    def materialize(self) -> torch.Tensor:
        return self.norm.forward(self.x, self.ctx)


def rows_of(h):
    """The normalised rows of ``h``: ``h`` itself, or a deferred norm run now."""
    return h.materialize() if isinstance(h, DeferredNorm) else h


class RMSNorm(Norm):
    def __init__(self, spec):
        self.spec = spec
        self.groups = int(getattr(spec, "groups", 1))
        if self.groups < 1 or spec.size % self.groups:
            raise ValueError(f"{self.groups} groups do not divide a norm over {spec.size} elements")
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        init = "one_plus_normal" if self.spec.weight_offset == 0.0 else "normal"      # a weight stored around zero is drawn around zero
        return [WeightSpec(prefix + self.spec.weight, (self.spec.size,), "vector", (init, 0.1))]

    def bind(self, get) -> None:
        w = get(self.spec.weight)
        # the factor on a row is (offset + stored weight), formed once, in float32
        self.weight = w if self.spec.weight_offset == 0.0 else (w.float() + float(self.spec.weight_offset)).contiguous()

    def deferred(self, x: torch.Tensor, ctx) -> DeferredNorm:
        if self.groups != 1:
            raise ValueError("a norm in groups cannot be folded into a matrix product")
        return DeferredNorm(self, x, ctx)

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``out_dtype``: the dtype of the normed rows where it is not the compute dtype (float32 for a norm inside the residual stream)."""
        n = x.shape[0] if rows is None else rows.numel()
        y = ctx.empty((n, self.spec.size), out_dtype)
        if self.groups > 1:
            K.group_rmsnorm(x, self.weight, y, self.groups, self.spec.eps, ctx.stream, rows)
        else:
            K.rmsnorm(x, self.weight, y, self.spec.eps, ctx.stream, rows)
        return y


NORMS.register("rmsnorm", RMSNorm)


class DynamicTanh(Norm):
    """``dyt``: y = tanh(alpha * x) * w + b, with one learned number alpha: a norm that computes no mean and no variance
    (``eps`` of the spec is not used).  Tensors: the weight under the spec's name, the bias and alpha beside it as
    ``<name>.b`` and ``<name>.alpha`` (alpha a tensor without dimensions).  float32 inside.  The block arrangement that
    scales its sublayers' outputs takes this norm into the kernel that adds them to the residual stream (``triple``)."""

    def __init__(self, spec):
        self.spec = spec
        self.weight = self.bias = self.alpha = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        n = prefix + self.spec.weight
        return [WeightSpec(n, (self.spec.size,), "vector", ("one_plus_normal", 0.1)), WeightSpec(n + ".b", (self.spec.size,), "vector", ("normal", 0.1)),
                WeightSpec(n + ".alpha", (), "vector", ("one_plus_normal", 0.1))]

    def bind(self, get) -> None:
        n = self.spec.weight
        self.weight, self.bias, self.alpha = get(n), get(n + ".b"), get(n + ".alpha").reshape(1)

    def triple(self):
        return self.weight, self.bias, self.alpha

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        y = ctx.empty((n, self.spec.size))
        K.dyt(x, self.weight, self.bias, self.alpha, y, ctx.stream, rows)
        return y


NORMS.register("dyt", DynamicTanh)
