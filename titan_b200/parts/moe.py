"""Mixture of experts as a feed-forward.

    z = h . W_router^T (float32);  the ``top`` largest entries of z choose a token's experts, and their weights are the
    softmax over the chosen entries only;  out += sum_k weight_k * expert_{e_k}(h)  (+ sigmoid(h . w_sg) * shared(h))
    expert(h) = W_down (silu(W_gate h) * (W_up h))

The router and the shared expert's gate are one float32 product ([E (+1), H]).  Every expert's gate and up rows are
interleaved at bind time ([E, 2F, H]) so that one product applies the activation in its epilogue, as the gated MLP does.
Routing, grouping and the experts' products all happen on the device: nothing is read on the host, so decode steps
are captured as graphs.

Options of the spec beyond experts, top and the shared expert:

* ``routing = "softmax_all"``: scores s = softmax(z) over ALL router outputs; an expert is chosen by s + correction (a
  tensor, ``correction``), and only among the ``keep`` groups (``groups`` equal groups of neighbouring experts) whose
  best such score is largest (the others count as minus infinity); the weights are the chosen experts' s divided by
  their sum (+ 1e-20).  The default (``"top_softmax"``) takes the top logits and the softmax over them alone.
* ``routing = "sigmoid_all"``: scores s = sigmoid(z), each output on its own; the rest as above, with two more options:
  ``group_best`` = n (a group's score is the sum of its n largest s + correction; 1: its best one) and ``renormalize`` =
  False (the weights are the chosen experts' s as they are).
* ``shared_gate`` = False: the shared expert's output is added as it is (no sigmoid gate, no tensor for one).
* ``identity = n``: the last n router outputs are experts without matrices whose output is the input row itself (times
  the weight); they take part in the scores, the groups and the choice like any other.
* ``activation``: ``silu`` (silu(g) u) or ``swish_clamped`` with ``limit``: g' = min(g, limit), u' = clamp(u, -limit, limit),
  g' sigmoid(1.702 g') (u' + 1).

A step with few (token, choice) pairs runs a warp-per-output kernel that reads each chosen
expert's rows once (a decode step is bound by those bytes); larger steps group the pairs by expert
(``moe_plan``) and run tiles of rows of one expert each (``moe_grouped``, CUDA cores: float32, and decode steps of many
sequences); a bfloat16 prompt gathers every expert's rows side by side and runs the tensor-core product expert by
expert, reading the experts' row counts on the host.
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from .. import kernels as K
from . import linear
from .base import FEED_FORWARDS, FeedForward


class MixtureOfExperts(FeedForward):
    def __init__(self, spec):
        s = spec
        if s.activation not in ("silu", "swish_clamped"):
            raise ValueError(f"activation '{s.activation}' is not supported ('silu' or 'swish_clamped')")
        self.spec = s
        self.gate_kind, self.limit = K.GATES[s.activation], float(s.option("limit", 0.0))
        if s.activation == "swish_clamped" and not self.limit > 0:
            raise ValueError("the clamped gate needs a positive limit")
        self.routing = s.option("routing", "top_softmax")
        if self.routing not in ("top_softmax", "softmax_all", "sigmoid_all"):
            raise ValueError(f"routing '{self.routing}' is not known (top_softmax, softmax_all, sigmoid_all)")
        self.scored = self.routing in ("softmax_all", "sigmoid_all")            # scores over all outputs, correction, groups
        self.group_best, self.renormalize = int(s.option("group_best", 1)), bool(s.option("renormalize", True))
        self.shared_gate = bool(s.option("shared_gate", True))
        if self.group_best < 1 or (not self.scored and (self.group_best != 1 or not self.renormalize)):
            raise ValueError("group_best and renormalize are options of the routings that score all outputs")
        self.identity = int(s.option("identity", 0))
        self.groups, self.keep = int(s.option("groups", 1)), int(s.option("keep", 1))
        self.E, self.top, self.F = int(s.option("experts", 0)), int(s.option("top", 0)), s.intermediate_size
        self.shared_F = int(s.option("shared_size", 0))
        if self.E <= 0 or self.identity < 0 or not 0 < self.top <= self.E + self.identity or self.F <= 0:
            raise ValueError(f"a mixture of {self.E} experts of size {self.F}, {self.top} a token")
        self.n_all = self.E + self.identity
        if self.routing == "top_softmax" and (self.identity or self.groups != 1):
            raise ValueError("experts without matrices and groups of experts come with routing 'softmax_all'")
        if self.groups <= 0 or not 0 < self.keep <= self.groups or self.n_all % self.groups or self.top > self.keep * (self.n_all // self.groups):
            raise ValueError(f"{self.groups} groups over {self.n_all} experts, {self.keep} kept, {self.top} experts a token")
        if self.identity and self.shared_F:
            raise ValueError("a shared expert beside experts without matrices is not supported")
        self.correction = None
        self.w_router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None

    def _names(self):
        s = self.spec
        names = {role: s.name(role, role) for role in ("gate", "up", "down", "router")}
        names["expert"] = s.name("expert", "e{}.")              # prefix of expert number {}
        names["shared"] = s.name("shared", "shared.")
        names["shared_gate"] = s.name("shared_gate", "shared.sg")
        names["correction"] = s.name("correction", "correction")
        return names

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        H = s.hidden_size
        specs = []
        for e in range(self.E):
            q = p + n["expert"].format(e)
            specs += [WeightSpec(q + n["gate"], (self.F, H)), WeightSpec(q + n["up"], (self.F, H)), WeightSpec(q + n["down"], (H, self.F))]
        specs.append(WeightSpec(p + n["router"], (self.n_all, H)))
        if self.scored:
            specs.append(WeightSpec(p + n["correction"], (self.n_all,), "vector", ("normal", 0.02)))
        if self.shared_F:
            q = p + n["shared"]
            specs += [WeightSpec(q + n["gate"], (self.shared_F, H)), WeightSpec(q + n["up"], (self.shared_F, H)),
                      WeightSpec(q + n["down"], (H, self.shared_F))]
            if self.shared_gate:
                specs.append(WeightSpec(p + n["shared_gate"], (1, H)))
        return specs

    def bind(self, get) -> None:
        s, p, n = self.spec, self.spec.prefix, self._names()
        H = s.hidden_size
        first = get(p + n["expert"].format(0) + n["gate"])
        self.w_gate_up = torch.empty((self.E, 2 * self.F, H), dtype=first.dtype, device=first.device)
        self.w_down = torch.empty((self.E, H, self.F), dtype=first.dtype, device=first.device)
        for e in range(self.E):
            q = p + n["expert"].format(e)
            self.w_gate_up[e, 0::2] = get(q + n["gate"])
            self.w_gate_up[e, 1::2] = get(q + n["up"])
            self.w_down[e] = get(q + n["down"])
        router = get(p + n["router"])
        if self.scored:
            self.correction = get(p + n["correction"])
        if self.shared_F:
            q = p + n["shared"]
            self.w_router = torch.cat([router, get(p + n["shared_gate"])], dim=0).contiguous() if self.shared_gate else router
            self.ws_gate_up = torch.stack([get(q + n["gate"]), get(q + n["up"])], dim=1).reshape(2 * self.shared_F, H).contiguous()
            self.ws_down = get(q + n["down"])
        else:
            self.w_router = router

    def forward(self, h, ctx, out: torch.Tensor) -> None:
        T, H, top, E = h.shape[0], self.spec.hidden_size, self.top, self.E
        P = T * top
        f32, i32 = torch.float32, torch.int32
        ids, wts = ctx.empty((T, top), i32), ctx.empty((T, top), f32)
        gate = ctx.empty((T,), f32) if self.shared_F and self.shared_gate else None
        n_logits = self.w_router.shape[0]
        z = ctx.empty((T, -(-n_logits // 4) * 4), f32)[:, :n_logits]       # rows of whole 16 bytes: the tensor-core product's output rule
        linear.matmul(h, self.w_router, z, linear.EPI_F32, ctx)
        if self.routing == "softmax_all" and self.group_best == 1 and self.renormalize:
            K.moe_route_all(z, top, self.correction, self.groups, self.keep, ids, wts, ctx.stream)
        elif self.scored:
            K.moe_route_scored(z, top, self.correction, self.groups, self.keep, ids, wts, ctx.stream,
                               sigmoid=self.routing == "sigmoid_all", group_best=self.group_best, renorm=self.renormalize)
        else:
            K.moe_route(z, E, top, gate is not None, ids, wts, gate, ctx.stream)
        shared_y = None
        if self.shared_F:
            act_s = ctx.empty((T, self.shared_F))
            linear.matmul(h, self.ws_gate_up, act_s, linear.EPI_SWIGLU, ctx, gate=self.gate_kind, limit=self.limit)
            shared_y = ctx.empty((T, H), f32)
            linear.matmul(act_s, self.ws_down, shared_y, linear.EPI_F32, ctx)
        act, y = ctx.empty((P, self.F)), ctx.empty((P, H), f32)
        gk = dict(gate=self.gate_kind, limit=self.limit)
        # experts without matrices: their pairs have no row in y, the combining kernel adds the token's own row instead
        same = dict(ids=ids, n_real=E, x=h) if self.identity else {}
        if P <= int(ctx.options.get("moe_rows_pairs", 64)):
            K.moe_rows(h, self.w_gate_up, act, 0, ids, top, ctx.stream, **gk)
            K.moe_rows(act, self.w_down, y, 1, ids, top, ctx.stream)
            K.moe_combine(y, wts, shared_y, gate, out, top, ctx.stream, **same)
            return
        plan = K.moe_plan(ids, self.n_all, ctx.empty((K.MoePlan.size(P, self.n_all),), i32), ctx.stream)
        on_tensor_cores = (not ctx.layout.all_single and h.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain"
                           and P >= int(ctx.options.get("moe_tensor_pairs", 512)))
        if on_tensor_cores:
            # A prompt: every expert's rows side by side, one tensor-core product per expert and matrix.  How many rows
            # each expert got is read on the host (one small copy a layer); steps of single tokens never come here,
            # so they stay free of host reads and are captured as graphs.
            offsets = plan.offsets.tolist()[:E + 1]                      # the rows of experts without matrices lie behind the last run
            xs = ctx.empty((P, H))
            K.moe_gather(h, plan, top, xs, ctx.stream)
            if (K.gemm_tc_accepts(xs[:1], self.w_gate_up[0], act[:1], linear.EPI_SWIGLU)
                    and K.gemm_tc_accepts(act[:1], self.w_down[0], y[:1], linear.EPI_F32)):
                K.gemm_tc_expert_runs(xs, self.w_gate_up, act, self.w_down, y, offsets, ctx.stream, **gk)
            else:
                for e in range(E):
                    a, b = offsets[e], offsets[e + 1]
                    if b > a:
                        linear.matmul(xs[a:b], self.w_gate_up[e], act[a:b], linear.EPI_SWIGLU, ctx, **gk)
                        linear.matmul(act[a:b], self.w_down[e], y[a:b], linear.EPI_F32, ctx)
            K.moe_combine(y, wts, shared_y, gate, out, top, ctx.stream, where=plan.inverse, **same)
        else:
            K.moe_grouped(h, self.w_gate_up, act, 0, plan, top, ctx.stream, **gk)
            K.moe_grouped(act, self.w_down, y, 1, plan, top, ctx.stream)
            K.moe_combine(y, wts, shared_y, gate, out, top, ctx.stream, **same)


FEED_FORWARDS.register("moe", MixtureOfExperts)
