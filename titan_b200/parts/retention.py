"""Retention as a mixer: linear attention with one fixed decay a head, rotated queries and keys, no softmax and no denominator.

    [q | k | v | g] = h . [W_q ; W_k ; W_v ; W_g]^T                  one product, float32 out
    q, k <- rotary(q, k) by position;  k <- k * scale                 heads x dim (``scale`` defaults to dim^-1/2)
    S_t = decay_h S_{t-1} + k_t v_t^T ;  o_t = S_t^T q_t             per head; S float32 [dim, value_dim], zero at the start
    y = concat_h(o_t,h / rms(o_t,h)) * silu(g) ;  out += y . W_o^T   the heads' norms have no weight

What enters the recurrence is float32 in either dtype: the projection leaves float32 sums, the rotation (angles in float32)
and the key's factor are applied to them in place, and the recurrence kernel of the ``lightning`` mixer reads them as they
stand (``LightningArgs.plain``).  The state is a ``state`` cache group of shape [heads, dim, value_dim] per sequence,
zeroed when a slot is handed out and indexed by slot on the device, so decode steps are captured as graphs; a sequence's
tokens are taken in order whatever the step brings.  Options of the spec: ``value_dim``, ``decay`` (one number a head),
``norm_eps``, ``key_scale``; the rotation is ``MixerSpec.position`` (either pairing, the first ``rotary_dim`` of a head).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, StateGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, POSITIONS, Mixer


class RetentionMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.dk, self.dv = s.num_heads, s.head_dim, int(s.option("value_dim", s.head_dim))
        decay = tuple(float(d) for d in s.option("decay", ()))
        if self.H <= 0 or self.dk <= 0 or self.dv <= 0:
            raise ValueError("retention needs positive heads, dim and value_dim")
        if self.dk > 256:
            raise ValueError(f"{self.dk} key dimensions a head: the recurrence kernel holds up to 256")
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        self.decay_values = decay
        self.eps = float(s.option("norm_eps", 0.0))
        self.key_scale = float(s.option("key_scale", self.dk ** -0.5))
        self.position = POSITIONS.build(s.position)
        if self.position.rotary_dim > self.dk:
            raise ValueError(f"{self.position.rotary_dim} rotated dimensions in a head of {self.dk}")
        self.w_in = self.w_o = self.decay = self.ones = None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", state_shape=(self.H, self.dk, self.dv), state_dtype=torch.float32)

    def _names(self):
        return {role: self.spec.name(role, role) for role in ("q", "k", "v", "g", "o")}

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        W, Nk, Nv = s.hidden_size, self.H * self.dk, self.H * self.dv
        return [WeightSpec(p + n["q"], (Nk, W)), WeightSpec(p + n["k"], (Nk, W)), WeightSpec(p + n["v"], (Nv, W)),
                WeightSpec(p + n["g"], (Nv, W)), WeightSpec(p + n["o"], (W, Nv))]

    def bind(self, get) -> None:
        p, n = self.spec.prefix, self._names()
        self.w_in = torch.cat([get(p + n[role]) for role in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = get(p + n["o"])
        dev = self.w_o.device
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=dev)
        self.ones = torch.ones(self.dv, dtype=torch.float32, device=dev)          # the heads' norms have no weight

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        lay = ctx.layout
        T, H, dk, dv = lay.T, self.H, self.dk, self.dv
        group, index = cache
        if not isinstance(group, StateGroup):
            raise TypeError(f"retention keeps its state in a 'state' cache group, not in {type(group).__name__}")
        proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
        linear.matmul(h, self.w_in, proj, linear.EPI_F32, ctx)
        gate = proj[:, 2 * H * dk + H * dv:]                       # the gate's arguments stay float32 sums
        rope = self.position.kernel_args(ctx.device)
        if rope.inv_freq:
            K.rotary_rows(proj, lay.pos_of, 2 * H, dk, rope, H, self.key_scale, ctx.stream)      # q heads, then k heads (scaled)
        elif self.key_scale != 1.0:
            raise NotImplementedError("retention without a rotation: the key's factor is applied by the rotation kernel")
        o = ctx.empty((T, H * dv), torch.float32)
        a = K.LightningArgs()
        a.proj, a.stride = proj.data_ptr(), proj.stride(0)
        a.out, a.out_stride = o.data_ptr(), o.stride(0)
        a.state, a.decay = group.layer_storage(index).data_ptr(), self.decay.data_ptr()
        a.q_start, a.slot_of_seq = lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr()
        a.B, a.H, a.dk, a.dv, a.max_new, a.plain = lay.B, H, dk, dv, lay.max_new, 1
        K.lightning_scan(a, torch.float32, ctx.stream)
        y = ctx.empty((T, H * dv))
        K.head_norm_gate(o, self.ones, False, gate, y, H, K.GATE_SILU, 1.0, self.eps, ctx.stream)
        linear.matmul(y, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("retention", RetentionMixer)
