"""Attention over a shared latent, as a mixer.

Per token the layer keeps ONE row for all heads: a latent c (``kv_rank`` numbers, RMS-normed) and a rotated key
part k_r (``rot_dim`` numbers).  Head h's key is [U_k,h c | k_r] and its value U_v,h c, with the expansions
U_k [H * dim, kv_rank] and U_v [H * vdim, kv_rank]; they are never formed.  Since q_h . (U_k,h c) = (U_k,h^T q_h) . c
and sum_j p_j U_v,h c_j = U_v,h (sum_j p_j c_j), the mixer moves each head's unrotated query into the latent space,
attends there with the cached row as key AND value (one "kv head" for all query heads), and expands the result:

    [q | c_raw | k_raw] = h . [W_q ; W_dkv]^T                      one product, float32 out
    c = rmsnorm(c_raw) * w_c;  k_r = rot(k_raw);  q_r,h = rot(q_h[dim:])     (latent_prep kernel; appends the row)
    q~_h = q_h[:dim] . U_k,h                                          per head  [T, dim] x [dim, kv_rank]
    s_hij = ([q~_h | q_r,h]_i . [c | k_r]_j) * scale  over keys 0 <= i - j < window;  p = softmax(s)
    o~_h = sum_j p_hij c_j;   o_h = o~_h . U_v,h^T                    per head  [T, kv_rank] x [kv_rank, vdim]
    out += [o_1 .. o_H] . W_o^T

With the option ``q_rank`` the queries go through a latent of their own: c_q = rmsnorm(h . W_dq^T) * w (``q_norm``, a
NormSpec), q = c_q . W_uq^T (tensor roles "dq" and "uq" instead of "q"); the projection then yields [c_q_raw], [c_raw |
k_raw] as two products (query latent; latent and key part), a norm kernel makes c_q, and a third product fills the query
columns of the row that the prep kernel reads.

Rows are padded with zeros to a multiple of 8 elements.  A mixer with ``cache_from`` has no W_dkv: it reads the rows
of the named layer (its own window may be shorter than what that layer keeps).  A step of single tokens appends in
the prep kernel and attends over the cache; a step with longer runs attends over cache + the step's own rows (the
owner leaves them in ``ctx.carried`` for its readers) and appends where that is safe: at once if no row of the step
replaces one that a query of the step still sees (no ring, or every sequence at its start), else after the last
block of the step.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, LatentGroup
from ..weights.loader import WeightSpec
from . import linear
from .attention import decode_split
from .base import MIXERS, NORMS, POSITIONS, Mixer


def _round8(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttentionMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.dn = s.num_heads, s.head_dim
        self.rd, self.dv, self.r = int(s.option("rot_dim", 0)), int(s.option("value_dim", s.head_dim)), int(s.option("kv_rank", 0))
        if self.H <= 0 or self.dn <= 0 or self.dv <= 0 or self.r <= 0 or self.rd < 0:
            raise ValueError("latent attention needs positive heads, dim, value_dim and kv_rank")
        if s.window is not None and s.window <= 0:
            raise ValueError("an attention window must be positive")
        self.dk = _round8(self.r + self.rd)                 # a cached row, and a head's query row
        if self.dk > 1024:
            raise ValueError(f"latent + rotated part of {self.r + self.rd} elements: rows of up to 1024 are supported")
        self.shared = s.cache_from is not None
        self.position = POSITIONS.build(s.position)
        if self.position.rotary_dim > self.rd:
            raise ValueError(f"{self.position.rotary_dim} rotated dimensions of a part of {self.rd}")
        self.latent_norm_spec = s.option("latent_norm")
        self.q_rank, self.q_norm_spec = int(s.option("q_rank", 0) or 0), s.option("q_norm")
        if self.q_rank and self.q_norm_spec is None:
            raise ValueError("queries through a latent need that latent's norm (q_norm)")
        self.w_uq = self.q_norm = self.w_dkv = None
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(self.dn + self.rd)
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.latent_w = None
        self._views = {}

    # -- declaration ------------------------------------------------------ #
    def cache_need(self) -> Optional[CacheNeed]:
        if self.shared:
            return None
        return CacheNeed("latent", 1, self.dk, self.spec.option("cache_window", self.spec.window))

    def _names(self):
        s = self.spec
        return {role: s.name(role, role) for role in ("q", "dq", "uq", "dkv", "uk", "uv", "o")}

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        W = s.hidden_size
        if self.q_rank:
            specs = [WeightSpec(p + n["dq"], (self.q_rank, W)), WeightSpec(p + n["uq"], (self.H * (self.dn + self.rd), self.q_rank))]
            specs += NORMS.build(self.q_norm_spec).weight_specs(p)
        else:
            specs = [WeightSpec(p + n["q"], (self.H * (self.dn + self.rd), W))]
        if not self.shared:
            specs.append(WeightSpec(p + n["dkv"], (self.r + self.rd, W)))
            specs += NORMS.build(self.latent_norm_spec).weight_specs(p)
        specs += [WeightSpec(p + n["uk"], (self.H * self.dn, self.r)), WeightSpec(p + n["uv"], (self.H * self.dv, self.r)),
                  WeightSpec(p + n["o"], (W, self.H * self.dv))]
        return specs

    def bind(self, get) -> None:
        p, n = self.spec.prefix, self._names()
        if self.q_rank:
            q = get(p + n["dq"])
            self.w_uq = get(p + n["uq"])
            self.q_norm = NORMS.build(self.q_norm_spec)
            self.q_norm.bind(lambda name: get(p + name))
        else:
            q = get(p + n["q"])
        if self.shared:
            self.w_in = q
        else:
            # with a query latent the two down-projections stay apart: the key part is written where the prep kernel reads it
            self.w_dkv = get(p + n["dkv"]) if self.q_rank else None
            self.w_in = q if self.q_rank else torch.cat([q, get(p + n["dkv"])], dim=0).contiguous()
            norm = NORMS.build(self.latent_norm_spec)
            norm.bind(lambda name: get(p + name))
            self.latent_w = norm.weight
        # U_k by head, transposed: [H, kv_rank, dim], so that q~_h = q_h . (that)^T; U_v by head as stored: [H, vdim, kv_rank]
        uk, uv = get(p + n["uk"]), get(p + n["uv"])
        self.w_uk_t = uk.view(self.H, self.dn, self.r).transpose(1, 2).contiguous()
        self.w_uv = uv.view(self.H, self.dv, self.r).contiguous()
        # both expansions as one matrix, for prompts that expand keys and values per head (see _expanded_prompt)
        self.w_ukv = torch.cat([uk, uv], dim=0).contiguous() if uk.dtype == torch.bfloat16 else None
        self.w_o = get(p + n["o"])

    # -- one step --------------------------------------------------------- #
    def _view(self, cache) -> K.KvView:
        group, index = cache
        key = (id(group), index)
        if key not in self._views:
            if not isinstance(group, LatentGroup) or group.need.head_dim != self.dk:
                raise TypeError(f"latent attention reads rows of {self.dk} from a 'latent' cache group, not from {type(group).__name__}")
            self._views[key] = K.KvView(group.layer_storage(index).data_ptr(), group.table.data_ptr(), group.table_width,
                                        group.ring_rows, group.page_size, group.num_pages, 1, self.dk)
        return self._views[key]

    def _split_args(self, ctx, q_full, kv, rows, o):
        """Arguments of the tensor-core prompt kernel that scores expanded keys (or None where it does not apply)."""
        s, lay = self.spec, ctx.layout
        if ((self.dn, self.rd, self.dv) not in K.ATTN_SPLIT_SIZES or self.w_ukv is None or not lay.all_fresh or lay.all_single
                or ctx.options.get("attention", "fast") == "plain"
                or ctx.options.get("gemm", "fast") == "plain" or getattr(K, "attn_prefill_split", None) is None):
            return None
        a = K.SplitAttnArgs()
        a.q, a.q_stride = (q_full.data_ptr(), q_full.stride(0)) if q_full is not None else (1 << 12, self.H * (self.dn + self.rd))
        a.kv, a.kv_stride = (kv.data_ptr(), kv.stride(0)) if kv is not None else (1 << 12, self.w_ukv.shape[0])
        a.k_col0, a.v_col0 = 0, self.H * self.dn
        a.tail, a.tail_stride, a.tail_col0 = (rows.data_ptr() if rows is not None else 1 << 12), self.dk, self.r
        a.out, a.out_stride = (o.data_ptr(), o.stride(0)) if o is not None else (1 << 12, self.H * self.dv)
        a.batch = lay.c_struct()
        a.nh, a.dn, a.dt, a.dv = self.H, self.dn, self.rd, self.dv
        a.window, a.scale = s.window or 0, self.scale
        return a if K.attn_prefill_split_accepts(a) else None

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        s, lay = self.spec, ctx.layout
        T, H, dn, rd, dv, r, dk = lay.T, self.H, self.dn, self.rd, self.dv, self.r, self.dk
        view = self._view(cache)
        group, index = cache
        decode = lay.all_single
        if self.q_rank:
            # the query latent and its norm, the queries into the row's first columns, the latent and key part behind them
            cq_raw = ctx.empty((T, self.q_rank), torch.float32)
            linear.matmul(h, self.w_in, cq_raw, linear.EPI_F32, ctx)
            cq = self.q_norm.forward(cq_raw, ctx)
            nq, tail = H * (dn + rd), 0 if self.shared else r + rd
            qcols = -(-nq // 4) * 4                            # the key part starts on a 16-byte border
            proj = ctx.empty((T, qcols + -(-tail // 4) * 4), torch.float32)
            linear.matmul(cq, self.w_uq, proj[:, :nq], linear.EPI_F32, ctx)
            kv_in = None
            if tail:
                kv_in = proj[:, qcols:qcols + tail]
                linear.matmul(h, self.w_dkv, kv_in, linear.EPI_F32, ctx)
        else:
            proj = ctx.empty((T, self.w_in.shape[0]), torch.float32)
            linear.matmul(h, self.w_in, proj, linear.EPI_F32, ctx)
            kv_in = None
        # Whole prompts in bfloat16 with heads of the sizes the tensor-core kernel is built for: keys and values are
        # expanded per head by one product (k_h = U_k,h c, v_h = U_v,h c) and scored as they are; no move into the latent space.
        expanded = self._split_args(ctx, None, None, None, None) is not None
        q_full = ctx.empty((T, H * (dn + rd))) if expanded else None
        q_nope, q_abs = (None, None) if expanded else (ctx.empty((T, H * dn)), ctx.empty((T, H * dk)))
        rows = None
        rows_key = ("latent_rows", id(group), index)
        if not self.shared and not decode:
            rows = ctx.empty((T, dk))
            ctx.carried[rows_key] = rows                   # for the layers of this step that read this cache
        elif self.shared and not decode:
            rows = ctx.carried.get(rows_key)
            if rows is None:
                raise RuntimeError("a layer reads another layer's latents before that layer has run in this step")
        append_now = not self.shared and (decode or view.ring_rows == 0 or lay.all_fresh)
        la = K.LatentArgs()
        la.inp, la.in_stride = proj.data_ptr(), proj.stride(0)
        if kv_in is not None:
            la.kv_in = kv_in.data_ptr()
        if expanded:
            la.q_full, la.qf_stride = q_full.data_ptr(), q_full.stride(0)
        else:
            la.q_nope, la.qn_stride = q_nope.data_ptr(), q_nope.stride(0)
            la.q_abs, la.qa_stride = q_abs.data_ptr(), q_abs.stride(0)
        la.kv_rows, la.kv_stride = (None, 0) if (self.shared or rows is None) else (rows.data_ptr(), rows.stride(0))
        la.latent_w, la.eps = (None if self.shared else self.latent_w.data_ptr()), (0.0 if self.shared else self.latent_norm_spec.eps)
        la.rope = self.position.kernel_args(ctx.device)
        la.H, la.dn, la.rd, la.r, la.dk, la.owner = H, dn, rd, r, dk, int(not self.shared)
        la.pos_of, la.seq_of, la.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        la.kv_len, la.cache, la.append, la.T = lay.kv_len.data_ptr(), view, int(append_now), T
        K.latent_prep(la, ctx.dtype, ctx.stream)
        if not self.shared and not append_now:             # a ring, and sequences that go on: the rows wait until every reader has run
            batch = lay.c_struct()
            ctx.after_blocks.append(lambda: K.latent_append(rows, view, batch, ctx.stream))
        if expanded:
            kv = ctx.empty((T, self.w_ukv.shape[0]))
            linear.matmul(rows[:, :r], self.w_ukv, kv, linear.EPI_STORE, ctx)
            o = ctx.empty((T, H * dv))
            K.attn_prefill_split(self._split_args(ctx, q_full, kv, rows, o), ctx.stream)
            linear.matmul(o, self.w_o, out, linear.EPI_ADD, ctx)
            return
        # the heads' unrotated queries into the latent space
        linear.matmul_heads(q_nope, self.w_uk_t, q_abs, H, dn, dk, ctx)

        lat = ctx.empty((T, H * r))
        aa = K.AttnArgs()
        aa.q, aa.q_stride = q_abs.data_ptr(), q_abs.stride(0)
        aa.out, aa.out_stride = lat.data_ptr(), lat.stride(0)
        aa.cache, aa.batch = view, lay.c_struct()
        aa.nh, aa.nkv, aa.hd, aa.hd_v, aa.v_alias = H, 1, dk, r, 1
        aa.window, aa.scale = s.window or 0, self.scale
        if decode:
            # all heads read one row per key: a block for every few heads (not one for the single "kv head"), and splits
            # of one page, or of half a page while that still leaves SMs without a block (a step of one or two sequences:
            # measured at 16 heads and a window of 1,024, 0.61 -> 0.56 ms a step at batch 1, 0.87 -> 0.88 at batch 8)
            aa.head_blocks = H // 4 if H % 4 == 0 else (H // 2 if H % 2 == 0 else H)          # four heads (a warp each), two, or one a block
            span = min(s.window or lay.max_kv_len, lay.max_kv_len)
            few = lay.B * aa.head_blocks * -(-span // 64) < int(ctx.options.get("sm_count", 148))
            chunk = int(ctx.options.get("latent_chunk", 32 if few else 64))
            chunk, splits = decode_split(lay, 1, dict(ctx.options, attn_chunk=chunk), False)
            need = lay.B * H * splits * (r + 2)
            scratch = ctx.scratch.get("attn_partials")
            if scratch is None or scratch.numel() < need:
                scratch = ctx.scratch["attn_partials"] = torch.empty(need, dtype=torch.float32, device=ctx.device)
            aa.kv_new, aa.kv_stride = None, 0
            aa.chunk, aa.n_splits, aa.scratch = chunk, splits, scratch.data_ptr()
            K.attn_decode(aa, q_abs.dtype, ctx.stream)
        else:
            aa.kv_new, aa.kv_stride = rows.data_ptr(), rows.stride(0)
            K.attn_prefill(aa, q_abs.dtype, ctx.stream)
        # out of the latent space, head by head, and through the output projection
        o = ctx.empty((T, H * dv))
        linear.matmul_heads(lat, self.w_uv, o, H, r, dv, ctx)
        linear.matmul(o, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("latent_attention", LatentAttentionMixer)
