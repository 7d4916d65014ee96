"""Gated MLP as a feed-forward: down(act(gate(x)) * up(x)), added into the residual stream; act is silu or the tanh
form of gelu (``FeedForwardSpec.activation``), applied in the epilogue of the gate-and-up product.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:369-386 with
silu(g) = g / (1 + exp(-g)) (:210-219); its kernels fuse gate, up and SwiGLU in
one launch (engine/engine-cuda/kernels/gemm_quant.cu:2589).  Here the gate and
up matrices are interleaved row by row at bind time ([2F, H]: gate_0, up_0,
gate_1, ...), so that one matrix product has both halves of every pair in the
same tile and applies the activation in its epilogue.  The tensors' names come
from the spec (``FeedForwardSpec.names``): gate_proj / up_proj / down_proj
``.weight`` by default, or one stored [2F, H] tensor (gate rows, then up rows)
under the role "gate_up".
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from .. import kernels as K
from . import linear
from .base import FEED_FORWARDS, FeedForward
from .norm import DeferredNorm, rows_of


class GatedMLP(FeedForward):
    folds_norm = True           # a decode step's gate-and-up product takes the norm before it in

    def __init__(self, spec):
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation '{spec.activation}' is not supported ('silu' or 'gelu_tanh')")
        self.gate = K.GATES[spec.activation]
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.spec = spec
        self.w_gate_up = self.w_down = None

    def _names(self):
        s = self.spec
        names = {role: s.name(role, role + "_proj.weight") for role in ("gate", "up", "down")}
        names["gate_up"] = s.name("gate_up")
        return names

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        if n["gate_up"] is not None:
            first = [WeightSpec(p + n["gate_up"], (2 * s.intermediate_size, s.hidden_size))]
        else:
            first = [WeightSpec(p + n["gate"], (s.intermediate_size, s.hidden_size)),
                     WeightSpec(p + n["up"], (s.intermediate_size, s.hidden_size))]
        return first + [WeightSpec(p + n["down"], (s.hidden_size, s.intermediate_size))]

    def bind(self, get) -> None:
        p, n, F = self.spec.prefix, self._names(), self.spec.intermediate_size
        if n["gate_up"] is not None:
            both = get(p + n["gate_up"])
            gate, up = both[:F], both[F:]
        else:
            gate, up = get(p + n["gate"]), get(p + n["up"])
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * F, self.spec.hidden_size).contiguous()
        del gate, up
        self.w_down = get(p + n["down"])

    def forward(self, h, ctx, out: torch.Tensor) -> None:
        act = ctx.empty((h.shape[0], self.spec.intermediate_size))
        if (isinstance(h, DeferredNorm) and self.gate == K.ACT_SILU and ctx.options.get("gemm", "fast") != "plain" and self.w_gate_up.dtype == torch.bfloat16
                and K.gemm_tc_normed_accepts(h.x, h.weight, self.w_gate_up, act, linear.EPI_SWIGLU, None)):
            K.gemm_tc_normed(h.x, h.weight, h.eps, self.w_gate_up, act, linear.EPI_SWIGLU, ctx.stream)
        else:
            linear.matmul(rows_of(h), self.w_gate_up, act, linear.EPI_SWIGLU, ctx, gate=self.gate)
        linear.matmul(act, self.w_down, out, linear.EPI_ADD, ctx)


FEED_FORWARDS.register("gated_mlp", GatedMLP)


class ActivatedMLP(FeedForward):
    """``mlp``: a feed-forward without a gate, down(act(up(x))), added into the residual stream.  The activation
    (``FeedForwardSpec.activation``) is ``polynorm``: with z the up-projection's row of ``intermediate_size`` elements and
    four learned numbers (a, b, c, e) in one tensor (role "act"),

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,    N(x) = x / sqrt(mean(x^2) + eps)

    powers element by element, the means over the row; ``eps`` is the option "act_eps".  The three means and the result are
    float32 inside one kernel that reads the row twice; tensor names by role: "up", "down", "act"."""

    def __init__(self, spec):
        if spec.activation != "polynorm":
            raise ValueError(f"activation '{spec.activation}' is not supported by the ungated feed-forward ('polynorm')")
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.spec = spec
        self.eps = float(spec.option("act_eps", 1e-6))
        self.w_up = self.w_down = self.coef = None

    def _names(self):
        return {role: self.spec.name(role, role) for role in ("up", "down", "act")}

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        return [WeightSpec(p + n["up"], (s.intermediate_size, s.hidden_size)), WeightSpec(p + n["down"], (s.hidden_size, s.intermediate_size)),
                WeightSpec(p + n["act"], (4,), "vector", ("normal_around", 0.3, 0.5))]

    def bind(self, get) -> None:
        p, n = self.spec.prefix, self._names()
        self.w_up, self.w_down, self.coef = get(p + n["up"]), get(p + n["down"]), get(p + n["act"]).contiguous()

    def forward(self, h, ctx, out: torch.Tensor) -> None:
        h = rows_of(h)
        z = ctx.empty((h.shape[0], self.spec.intermediate_size))
        linear.matmul(h, self.w_up, z, linear.EPI_STORE, ctx)
        K.polynorm(z, self.coef, self.eps, z, ctx.stream)              # in place: a block reads its row before it writes it
        linear.matmul(z, self.w_down, out, linear.EPI_ADD, ctx)


FEED_FORWARDS.register("mlp", ActivatedMLP)
