"""The matrix memory of xLSTM (mLSTM) as a mixer: a linear-attention state with an exponential input gate, a sigmoid
forget gate, and a running maximum that keeps both in range.

    [q | k | v | gate] = h . [W_q ; W_k ; W_v ; W_g]^T        one product; q, k: heads x dim; v, gate: heads x value_dim
    [i~ | f~]          = h . [W_i ; W_f]^T + (b_i, b_f)       float32, one number per head each
    i = cap * tanh(i~ / cap);   f = logsigmoid(cap * tanh(f~ / cap))                 logarithms of the two gates
    m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n likewise with k alone;   m <- m'
    o = S^T (q * dim^(-1/2)) / (max(|n . q * dim^(-1/2)|, e^(-m)) + 1e-6)
    y = o / rms_head(o) * w * sigmoid(gate);   out += y . W_o^T                      w [heads * value_dim]

S, n and m start at zero (m at 0, not at minus infinity) and are float32: one row per sequence in a ``state`` cache group,
[S of every head | n of every head | m of every head], zeroed when a slot is handed out and indexed by slot on the device,
so decode steps are captured as graphs.  The recurrence takes a sequence's tokens in order whatever the step brings.
Options (``MixerSpec.extra``): ``value_dim``, ``gate_cap``, ``norm_eps``, ``output_scale``.  Tensor names by role: q, k, v,
g, o, i, f, norm; the gates' biases are ``<i|f name>.b``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, StateGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, Mixer
from .norm import rows_of


class MLstmMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.dk, self.dv = s.num_heads, s.head_dim, int(s.option("value_dim", s.head_dim))
        self.cap = float(s.option("gate_cap", 0.0))
        self.eps = float(s.option("norm_eps", 1e-6))
        self.output_scale = float(s.option("output_scale", 1.0))
        if self.H <= 0 or self.dk <= 0 or self.dv <= 0:
            raise ValueError("the mLSTM mixer needs positive heads, dim and value_dim")
        if self.dk > 256:
            raise ValueError(f"{self.dk} key dimensions a head: the recurrence kernel holds up to 256")
        if not self.cap > 0:
            raise ValueError("the mLSTM mixer needs a positive gate_cap")
        self.state_size = self.H * self.dk * self.dv + self.H * self.dk + self.H
        self.w_in = self.w_if = self.w_o = self.b_i = self.b_f = self.norm_w = None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def _name(self, role: str) -> str:
        return self.spec.name(role, role)

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        p, W, n = prefix + self.spec.prefix, self.spec.hidden_size, self._name
        Nk, Nv = self.H * self.dk, self.H * self.dv
        return [WeightSpec(p + n("q"), (Nk, W)), WeightSpec(p + n("k"), (Nk, W)), WeightSpec(p + n("v"), (Nv, W)),
                WeightSpec(p + n("g"), (Nv, W)), WeightSpec(p + n("o"), (W, Nv)),
                WeightSpec(p + n("norm"), (Nv,), "vector", ("one_plus_normal", 0.1)),
                WeightSpec(p + n("i"), (self.H, W)), WeightSpec(p + n("i") + ".b", (self.H,), "vector", ("normal", 0.5)),
                WeightSpec(p + n("f"), (self.H, W)), WeightSpec(p + n("f") + ".b", (self.H,), "vector", ("normal_around", 0.5, 2.0))]

    def bind(self, get) -> None:
        p = self.spec.prefix
        g = lambda role: get(p + self._name(role))
        self.w_in = torch.cat([g(r) for r in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_if = torch.cat([g("i"), g("f")], dim=0).contiguous()
        self.b_i, self.b_f = get(p + self._name("i") + ".b").contiguous(), get(p + self._name("f") + ".b").contiguous()
        self.norm_w, self.w_o = g("norm").contiguous(), g("o")

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        lay = ctx.layout
        T, H, dk, dv = lay.T, self.H, self.dk, self.dv
        group, index = cache
        if not isinstance(group, StateGroup):
            raise TypeError(f"the mLSTM mixer keeps its state in a 'state' cache group, not in {type(group).__name__}")
        state = group.layer_storage(index)
        h = rows_of(h)
        f32 = torch.float32
        proj = ctx.empty((T, self.w_in.shape[0]))
        linear.matmul(h, self.w_in, proj, linear.EPI_STORE, ctx)
        gates = ctx.empty((T, 2 * H), f32)
        linear.matmul(h, self.w_if, gates, linear.EPI_F32, ctx)
        o = ctx.empty((T, H * dv), f32)
        size = proj.element_size()
        a = K.ScanArgs()
        a.q, a.q_stride = proj.data_ptr(), proj.stride(0)
        a.k, a.k_stride = proj.data_ptr() + H * dk * size, proj.stride(0)
        a.v, a.v_stride = proj.data_ptr() + 2 * H * dk * size, proj.stride(0)
        a.group, a.gates, a.gates_stride = 1, gates.data_ptr(), 2 * H
        a.i_bias, a.f_bias, a.cap, a.q_scale = self.b_i.data_ptr(), self.b_f.data_ptr(), self.cap, float(dk) ** -0.5
        a.out, a.out_stride = o.data_ptr(), H * dv
        a.state, a.state_stride = state.data_ptr(), state.stride(0)
        a.q_start, a.slot_of_seq = lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr()
        a.B, a.H, a.dk, a.dv = lay.B, H, dk, dv
        K.recurrent_scan(a, K.SCAN_MLSTM, proj.dtype, ctx.stream)
        y = ctx.empty((T, H * dv))
        K.head_norm_gate(o, self.norm_w, True, proj[:, 2 * H * dk + H * dv:], y, H, K.GATE_SIGMOID, self.output_scale, self.eps, ctx.stream)
        linear.matmul(y, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("mlstm", MLstmMixer)
