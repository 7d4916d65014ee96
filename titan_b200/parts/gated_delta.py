"""The gated delta rule as a mixer: a linear-attention state that forgets by a per-head decay and is corrected towards
each new value instead of only added to.

    [q | k | v | gate] = h . [W_q ; W_k ; W_v ; W_g]^T        one product; q, k: key_heads x dim; v, gate: heads x value_dim
    [b | a]            = h . [W_b ; W_a]^T                    float32, one number per head each
    q, k, v <- silu(conv(.))                                  a short causal convolution over time per channel, taps [C, n],
                                                              the last tap on the current token, zeros before the start
    q <- q / sqrt(sum q^2 + 1e-6) * dim^(-1/2);  k <- k / sqrt(sum k^2 + 1e-6)          per head
    beta = sigmoid(b);  decay = exp(-exp(A_log) * softplus(a + dt_bias))                 per head
    S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                     per head, S float32 [dim, value_dim]
    y = o / rms(o) * w * silu(gate) * output_scale;  out += y . W_o^T                    w [value_dim], shared by the heads

Value head h reads key head h // (heads / key_heads).  What the mixer asks of the cache is one float32 row per sequence in a
``state`` group: S of every head, then the last n - 1 inputs of the convolution; zeroed when a slot is handed out, indexed by
slot on the device, so decode steps are captured as graphs.  The recurrence takes a sequence's tokens in order whatever the
step brings.  Options (``MixerSpec.extra``): ``value_dim``, ``taps``, ``norm_eps``, ``output_scale`` (a mixer that runs beside
another).  Tensor names by role: q, k, v, g, o, b, a, A_log, dt_bias, norm; the taps are ``<q|k|v name>.conv``.
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


class GatedDeltaMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.G, self.dk = s.num_heads, s.num_kv_heads or s.num_heads, s.head_dim
        self.dv, self.taps = int(s.option("value_dim", s.head_dim)), int(s.option("taps", 1))
        self.eps = float(s.option("norm_eps", 1e-6))
        self.output_scale = float(s.option("output_scale", 1.0))
        if self.H <= 0 or self.G <= 0 or self.H % self.G or self.dk <= 0 or self.dv <= 0:
            raise ValueError(f"the delta-rule mixer needs positive sizes and {self.H} heads a multiple of {self.G} key heads")
        if self.dk > 256:
            raise ValueError(f"{self.dk} key dimensions a head: the recurrence kernel holds up to 256")
        if not 1 <= self.taps <= 64:
            raise ValueError(f"a convolution of {self.taps} taps (1 to 64)")
        self.C = 2 * self.G * self.dk + self.H * self.dv                       # channels that pass the convolution
        self.conv_off = self.H * self.dk * self.dv
        self.state_size = self.conv_off + (self.taps - 1) * self.C
        self.w_in = self.w_ba = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm_w = None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def _name(self, role: str) -> str:
        return self.spec.name(role, role)

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        p, W, n = prefix + self.spec.prefix, self.spec.hidden_size, self._name
        Nk, Nv = self.G * self.dk, self.H * self.dv
        return [WeightSpec(p + n("q"), (Nk, W)), WeightSpec(p + n("q") + ".conv", (Nk, self.taps), "vector", ("normal_around", 0.3, 0.3)),
                WeightSpec(p + n("k"), (Nk, W)), WeightSpec(p + n("k") + ".conv", (Nk, self.taps), "vector", ("normal_around", 0.3, 0.3)),
                WeightSpec(p + n("v"), (Nv, W)), WeightSpec(p + n("v") + ".conv", (Nv, self.taps), "vector", ("normal_around", 0.3, 0.3)),
                WeightSpec(p + n("b"), (self.H, W)), WeightSpec(p + n("A_log"), (self.H,), "vector", ("normal", 0.5)),
                WeightSpec(p + n("norm"), (self.dv,), "vector", ("one_plus_normal", 0.1)),
                WeightSpec(p + n("a"), (self.H, W)), WeightSpec(p + n("dt_bias"), (self.H,), "vector", ("normal", 0.5)),
                WeightSpec(p + n("g"), (Nv, W)), WeightSpec(p + n("o"), (W, Nv))]

    def bind(self, get) -> None:
        p = self.spec.prefix
        g = lambda role: get(p + self._name(role))
        self.w_in = torch.cat([g(r) for r in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_ba = torch.cat([g("b"), g("a")], dim=0).contiguous()
        self.conv = torch.cat([get(p + self._name(r) + ".conv") for r in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w, self.w_o = g("A_log").contiguous(), g("dt_bias").contiguous(), g("norm").contiguous(), g("o")

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        lay = ctx.layout
        T, H, G, dk, dv, C = lay.T, self.H, self.G, self.dk, self.dv, self.C
        group, index = cache
        if not isinstance(group, StateGroup):
            raise TypeError(f"the delta-rule mixer keeps its state in a 'state' cache group, not in {type(group).__name__}")
        state = group.layer_storage(index)
        h = rows_of(h)
        f32 = torch.float32
        proj = ctx.empty((T, self.w_in.shape[0]))
        linear.matmul(h, self.w_in, proj, linear.EPI_STORE, ctx)
        ba = ctx.empty((T, 2 * H), f32)
        linear.matmul(h, self.w_ba, ba, linear.EPI_F32, ctx)
        qkv, gates, o = ctx.empty((T, C), f32), ctx.empty((T, 2 * H), f32), ctx.empty((T, H * dv), f32)
        p = K.DeltaPrepArgs()
        p.proj, p.stride = proj.data_ptr(), proj.stride(0)
        p.taps, p.n_taps = self.conv.data_ptr(), self.taps
        p.state, p.state_stride, p.conv_off = state.data_ptr(), state.stride(0), self.conv_off
        p.ba, p.ba_stride, p.a_log, p.dt_bias = ba.data_ptr(), ba.stride(0), self.a_log.data_ptr(), self.dt_bias.data_ptr()
        p.qkv, p.qkv_stride, p.gates, p.gates_stride = qkv.data_ptr(), C, gates.data_ptr(), 2 * H
        p.seq_of, p.q_start, p.slot_of_seq = lay.seq_of.data_ptr(), lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr()
        p.T, p.H, p.G, p.dk, p.dv = T, H, G, dk, dv
        K.delta_prep(p, proj.dtype, ctx.stream)
        a = K.ScanArgs()
        a.q, a.q_stride = qkv.data_ptr(), C
        a.k, a.k_stride = qkv.data_ptr() + G * dk * 4, C
        a.v, a.v_stride = qkv.data_ptr() + 2 * G * dk * 4, C
        a.group, a.gates, a.gates_stride, a.q_scale = H // G, gates.data_ptr(), 2 * H, 1.0
        a.out, a.out_stride = o.data_ptr(), H * dv
        a.state, a.state_stride = state.data_ptr(), state.stride(0)
        a.q_start, a.slot_of_seq = lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr()
        a.B, a.H, a.dk, a.dv = lay.B, H, dk, dv
        a.conv_in, a.conv_stride, a.conv_bf16 = proj.data_ptr(), proj.stride(0), int(proj.dtype == torch.bfloat16)
        a.conv_channels, a.n_taps, a.conv_off = C, self.taps, self.conv_off
        K.recurrent_scan(a, K.SCAN_DELTA, f32, ctx.stream)
        y = ctx.empty((T, H * dv))
        K.head_norm_gate(o, self.norm_w, False, proj[:, C:], y, H, K.GATE_SILU, self.output_scale, self.eps, ctx.stream)
        linear.matmul(y, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("gated_delta", GatedDeltaMixer)
