"""Causal grouped-query attention as a mixer.

x -> [Q | K | V] = x . Wqkv^T -> per-head RMSNorm on Q and K (optional) ->
position encoding on Q and K -> keys and values into the cache -> softmax(q.k *
scale) v over the keys the query may see (all earlier ones, or the last
``window``) -> . Wo^T, added into the residual stream.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:300-366 and 440-507;
driver steps forward_driver.rs:1010-1133 (prompt) and 2168-2259 (one token).
Q, K and V are three launches there; here their weights are concatenated at
bind time into one [Q + 2 KV, H] matrix.  Which tensors those are is the spec's
business (``MixerSpec.names``): by default q_proj / k_proj / v_proj / o_proj
``.weight`` under the prefix; a checkpoint that stores one fused tensor names
it under the role "qkv".

A step of single tokens writes K and V into the cache inside the norm/rotary
kernel and attends over the cache.  A step with longer runs of tokens keeps the
step's own K and V beside the cache, attends over both, and appends afterwards,
which is what makes a ring of ``window`` rows safe.

With ``cache_from`` the mixer owns no keys: it projects queries only and reads
the named layer's cache.

Options of the spec (``MixerSpec.extra``) beyond the common fields:

* ``value_dim``: width of a value head where it differs from the key's.  Keys and values are stored at one width, the
  larger of the two rounded up to 16; the narrower one's rows of the projections (and the columns of the output
  projection) are padded with zeros when the tensors are bound, which changes no score and no output.
* ``unit_norm`` = "after_rotation" | "before_rotation" with ``unit_norm_eps``: every Q and K head is divided by its
  root mean square (over the head's own width), without a weight, after or before the rotation.
* ``sink``: name of a tensor with one number per query head that joins the softmax's denominator as exp(sink), with no
  key and no value, once.
* ``value_norm``: an eps; every value head is divided by its root mean square (over the head's own width, without a
  weight) before it goes to the cache, so the cache holds normed values.
* ``keep_first`` (with ``window``): the first ``keep_first`` positions of a sequence stay visible to every later query beside
  the window's keys, at their true positions.  The cache then keeps every key (no ring).
* ``out_gate``: name of a [heads * value_dim, hidden] tensor; the concatenated heads are multiplied by sigmoid(W_g h), h the
  mixer's own input, before the output projection.
* ``output_scale``: a factor on what the mixer adds to the residual stream (a mixer that runs beside another); it is applied to
  the rows that enter the output projection, in float32 before they are rounded.
* Scores shaped before the softmax, and what comes with them in the designs that do so (any of these sends the mixer to the
  mixed-heads kernels, ``csrc/attention_mixed.cu``; no rotation, sink, kept tokens, head norm or blended values beside them):
  ``bias`` = True: the q, k, v and o projections have biases, tensors ``<name>.b``.
  ``whole_norm`` = (q weight name, k weight name, eps): ALL of a token's query elements are divided by one root mean square
  (every head together), times a weight as wide as the projection; likewise the keys.
  ``softcap`` = c: s <- c * tanh(s / c) after the scale.
  ``rel_bias`` = (name, rows, far): a table [rows, heads]; the row for distance n = query position - key position is n itself
  below rows/2, else min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))), added to the
  capped score, unscaled.  The mixer spreads the table by distance once, when the tensors are bound.
  ``head_mix`` = name of a [heads, heads] tensor M: head h's score becomes sum_g M[h, g] * score_g, for every (query, key) pair,
  before the softmax.
  ``head_gate`` = name of a [heads, hidden] tensor: head h's output is multiplied by sigmoid(W h)_h, one number a head.
* ``value_mix`` = (first, name): values are blended across layers.  ``first`` None: this layer's values are what the
  others blend with, and it keeps them for the step; else v <- (1 - l) v + l v_first with l the tensor ``name`` and
  v_first the values of layer ``first`` for the same tokens.  The blended values are what the cache holds.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, KVGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, POSITIONS, Mixer
from .norm import DeferredNorm, rows_of


def decode_split(lay, kv_heads: int, options, fast: bool):
    """(fewest keys per split, most splits) of decode attention; the kernels cut every sequence by its own
    length from these two numbers (``tb_split_keys``).  Neither depends on what the sequences hold or on the
    longest context the engine allows, so a sequence's borders are the same in any cache and beside any
    neighbours, and a captured step and an eager one cut the keys at the same places.

    The any-size kernel takes splits of ``attn_chunk`` keys, as many as the longest sequence needs (an eager
    step) or as the context limit needs (a captured one, whose grid is fixed; the spare ones leave at once):
    the borders are multiples of ``attn_chunk`` either way.  The tensor-core kernel takes the number of splits
    that fills the machine once at this batch size: two of its CTAs fit an SM, and (sequences x kv heads x splits)
    stays within 7/8 of those 2 x SMs places, because the splits of a (sequence, kv head) are a thread-block cluster,
    which is placed as a whole inside one part of the chip: with every place counted, some clusters wait for a
    second round (measured after 2,048-token prompts: 5 sequences 3.28 -> 3.03 ms per step with 6 splits instead
    of 7, 6 sequences 3.36 -> 3.09, 9 sequences 3.54 -> 3.29, 12 sequences 3.80 -> 3.50).  At most 16 splits merge
    inside a cluster (no scratch, no merge kernel), and clusters of more than 8 CTAs only while they fill half of
    the machine (16 / 9 / 8 / 4 / 2 / 1 splits at batch 1 / 2 / 4 / 8 / 16 / 32 with 8 kv heads)."""
    if not fast:
        chunk = int(options.get("attn_chunk", 256))
        cover = int(options.get("max_context", 0)) if options.get("fixed_splits") else 0
        return chunk, max(1, -(-(cover or lay.max_kv_len) // chunk))
    sms = int(options.get("sm_count", 148))
    pairs = lay.B * kv_heads
    splits = max(1, min(16, (2 * sms * 7 // 8) // pairs))
    if splits > 8:
        splits = max(8, min(splits, sms // pairs))
    forced = int(options.get("attn_splits", 0))
    return int(options.get("attn_min_chunk", 128)), forced or splits


def distance_rows(rows: int, far: float) -> List[int]:
    """Row of a distance table of ``rows`` rows for every distance 0 .. ceil(far): the distance itself below rows/2, then
    logarithmic steps that reach the last row at ``far`` (every larger distance reads the last row too)."""
    half = rows // 2
    out = []
    for n in range(int(math.ceil(far)) + 1):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class AttentionMixer(Mixer):
    folds_norm = True           # a decode step's Q|K|V product takes the norm before it in

    def __init__(self, spec):
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"{s.num_heads} query heads are not a multiple of {s.num_kv_heads} kv heads")
        self.key_dim, self.value_dim = s.head_dim, int(s.option("value_dim", s.head_dim))
        self.hd = -(-max(self.key_dim, self.value_dim) // 16) * 16          # the one width heads are computed and stored at
        if self.key_dim <= 0 or self.value_dim <= 0 or self.hd > 256:
            raise ValueError(f"heads of {self.key_dim} (keys) and {self.value_dim} (values) are not supported: at most 256")
        self.padded = (self.key_dim, self.value_dim) != (self.hd, self.hd)
        if self.padded and s.qk_norm is not None:
            raise ValueError("a head norm with a weight needs heads of a multiple of 16, keys and values of one width")
        if s.window is not None and s.window <= 0:
            raise ValueError("an attention window must be positive")
        if s.cache_from is not None and s.window is not None:
            raise ValueError("a mixer that reads another layer's cache cannot have a window")
        self.spec = s
        self.Q, self.KV = s.num_heads * self.hd, s.num_kv_heads * self.hd
        self.shared = s.cache_from is not None
        self.unit_norm = s.option("unit_norm")
        if self.unit_norm not in (None, "after_rotation", "before_rotation") or (self.unit_norm and s.qk_norm is not None):
            raise ValueError("unit_norm is 'after_rotation' or 'before_rotation', and takes the place of a head norm with a weight")
        self.sink_name = s.option("sink")
        self.value_mix = s.option("value_mix")          # None, or (first layer or None, tensor name)
        if self.value_mix is not None and self.shared:
            raise ValueError("a mixer that reads another layer's cache has no values to blend")
        # what the kernels that fold head norm, rotation and append into the attention do not know
        self.extended = bool(self.unit_norm or self.value_mix is not None or self.padded)
        self.value_norm = s.option("value_norm")         # None, or the eps of a unit norm of every value head
        self.keep_first = int(s.option("keep_first", 0) or 0)
        if self.keep_first < 0 or (self.keep_first and self.shared):
            raise ValueError("keep_first is a count of positions, and a mixer that reads another layer's cache takes that layer's keys as they are")
        self.gate_name = s.option("out_gate")
        self.output_scale = float(s.option("output_scale", 1.0))
        self.sink = self.mix_factor = self.w_gate = None
        self.position = POSITIONS.build(s.position)
        adjacent = getattr(s.position, "pairing", "half") != "half" and s.position.kind == "rope"
        self.extended = bool(self.extended or adjacent or self.value_norm is not None)
        self.scale = s.softmax_scale if s.softmax_scale is not None else 1.0 / math.sqrt(s.head_dim)
        if s.position.kind == "rope" and s.position.rotary_dim > self.key_dim:
            raise ValueError(f"{s.position.rotary_dim} rotated dimensions in a head of {self.key_dim}")
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self._views = {}
        # scores shaped before the softmax, biases, norms over the whole projection, one gate a head
        self.has_bias = bool(s.option("bias", False))
        self.whole_norm = s.option("whole_norm")
        self.softcap = float(s.option("softcap", 0.0) or 0.0)
        self.rel_spec = s.option("rel_bias")
        self.mix_name, self.head_gate_name = s.option("head_mix"), s.option("head_gate")
        self.shaped = bool(self.has_bias or self.whole_norm or self.softcap or self.rel_spec or self.mix_name or self.head_gate_name)
        if self.shaped:
            self.folds_norm = False
            if (self.shared or self.sink_name or self.keep_first or self.unit_norm or self.value_mix is not None or self.value_norm is not None
                    or self.gate_name or s.qk_norm is not None or s.position.kind != "none" or self.output_scale != 1.0):
                raise ValueError("shaped scores, biases, whole-projection norms and a gate a head come without rotation, sink, kept tokens, "
                                 "head norms, normed or blended values, an element-wise gate, an output factor or another layer's cache")
            if s.num_heads > 32:
                raise ValueError(f"{s.num_heads} heads whose scores are blended: the kernel takes up to 32")
            if self.softcap < 0:
                raise ValueError("softcap must be positive")
            if self.rel_spec is not None:
                _, rows, far = self.rel_spec
                if rows < 1 or (rows >= 2 and not far > rows // 2):
                    raise ValueError(f"a distance table of {rows} rows that reaches its last row at distance {far}")
        self.bias = self.b_o = self.whole_q_w = self.whole_k_w = self.rel_table = self.head_mix = None

    # -- declaration ------------------------------------------------------ #
    def cache_need(self) -> Optional[CacheNeed]:
        if self.shared:
            return None
        # kept first tokens stay in reach for good: such a window is a mask over a cache that keeps every key, not a ring
        return CacheNeed("kv", self.spec.num_kv_heads, self.hd, None if self.keep_first else self.spec.window)

    def _names(self):
        """Tensor names (relative to the prefix) by role; "qkv" only if the spec names a fused tensor."""
        s = self.spec
        names = {role: s.name(role, role + "_proj.weight") for role in ("q", "k", "v", "o")}
        names["qkv"] = s.name("qkv")
        if names["qkv"] is not None and self.shared:
            raise ValueError("a mixer that reads another layer's cache has queries only: it cannot name a fused q|k|v tensor")
        return names

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        kd, vd = self.key_dim, self.value_dim
        specs = [WeightSpec(p + n["o"], (s.hidden_size, s.num_heads * vd))]
        if n["qkv"] is not None:
            if self.padded:
                raise ValueError("a fused q|k|v tensor needs heads of a multiple of 16, keys and values of one width")
            specs.append(WeightSpec(p + n["qkv"], (self.Q + 2 * self.KV, s.hidden_size)))
        else:
            specs.append(WeightSpec(p + n["q"], (s.num_heads * kd, s.hidden_size)))
            if not self.shared:
                specs += [WeightSpec(p + n["k"], (s.num_kv_heads * kd, s.hidden_size)),
                          WeightSpec(p + n["v"], (s.num_kv_heads * vd, s.hidden_size))]
        if self.sink_name:
            specs.append(WeightSpec(p + self.sink_name, (s.num_heads,), "vector", ("normal", 1.0)))
        if self.gate_name:
            specs.append(WeightSpec(p + self.gate_name, (s.num_heads * vd, s.hidden_size)))
        if self.value_mix is not None and self.value_mix[0] is not None:      # (the layer the others blend with has no use for a factor)
            specs.append(WeightSpec(p + self.value_mix[1], (), "vector", ("normal", 0.3)))
        if s.qk_norm is not None:
            for which in ("q",) if self.shared else ("q", "k"):
                specs.append(WeightSpec(p + s.qk_norm.weight.format(which), (s.head_dim,), "vector", ("one_plus_normal", 0.1)))
        if self.has_bias:
            specs += [WeightSpec(p + n["q"] + ".b", (s.num_heads * kd,), "vector", ("normal", 0.1)),
                      WeightSpec(p + n["k"] + ".b", (s.num_kv_heads * kd,), "vector", ("normal", 0.1)),
                      WeightSpec(p + n["v"] + ".b", (s.num_kv_heads * vd,), "vector", ("normal", 0.1)),
                      WeightSpec(p + n["o"] + ".b", (s.hidden_size,), "vector", ("normal", 0.1))]
        if self.whole_norm:
            specs += [WeightSpec(p + self.whole_norm[0], (s.num_heads * kd,), "vector", ("one_plus_normal", 0.1)),
                      WeightSpec(p + self.whole_norm[1], (s.num_kv_heads * kd,), "vector", ("one_plus_normal", 0.1))]
        if self.rel_spec is not None:
            specs.append(WeightSpec(p + self.rel_spec[0], (int(self.rel_spec[1]), s.num_heads), "vector", ("normal", 0.5)))
        if self.mix_name:
            specs.append(WeightSpec(p + self.mix_name, (s.num_heads, s.num_heads), "vector", ("normal_around", 0.1, 1.0 / s.num_heads)))
        if self.head_gate_name:
            specs.append(WeightSpec(p + self.head_gate_name, (s.num_heads, s.hidden_size)))
        return specs

    def bind(self, get) -> None:
        s, p, n = self.spec, self.spec.prefix, self._names()
        if n["qkv"] is not None:
            self.w_qkv = get(p + n["qkv"])
        else:
            parts = [self._padded_rows(get(p + n["q"]), s.num_heads, self.key_dim)]
            if not self.shared:
                parts += [self._padded_rows(get(p + n["k"]), s.num_kv_heads, self.key_dim),
                          self._padded_rows(get(p + n["v"]), s.num_kv_heads, self.value_dim)]
            self.w_qkv = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else parts[0]
        self.w_o = get(p + n["o"])
        if self.value_dim != self.hd:                 # zero columns where the heads' outputs are padded
            w = self.w_o.reshape(s.hidden_size, s.num_heads, self.value_dim)
            self.w_o = torch.nn.functional.pad(w, (0, self.hd - self.value_dim)).reshape(s.hidden_size, self.Q).contiguous()
        if self.sink_name:
            self.sink = get(p + self.sink_name)
        if self.gate_name:
            self.w_gate = self._padded_rows(get(p + self.gate_name), s.num_heads, self.value_dim)
        if self.value_mix is not None and self.value_mix[0] is not None:
            self.mix_factor = get(p + self.value_mix[1]).reshape(1)
        if s.qk_norm is not None:
            self.q_norm = get(p + s.qk_norm.weight.format("q"))
            self.k_norm = None if self.shared else get(p + s.qk_norm.weight.format("k"))
        if self.shaped:
            dev = self.w_o.device
            if self.has_bias:
                self.bias = torch.cat([self._padded_vec(get(p + n["q"] + ".b"), s.num_heads, self.key_dim),
                                       self._padded_vec(get(p + n["k"] + ".b"), s.num_kv_heads, self.key_dim),
                                       self._padded_vec(get(p + n["v"] + ".b"), s.num_kv_heads, self.value_dim)]).float().contiguous()
                self.b_o = get(p + n["o"] + ".b").float().contiguous()
            if self.whole_norm:
                self.whole_q_w = self._padded_vec(get(p + self.whole_norm[0]), s.num_heads, self.key_dim).float().contiguous()
                self.whole_k_w = self._padded_vec(get(p + self.whole_norm[1]), s.num_kv_heads, self.key_dim).float().contiguous()
            if self.rel_spec is not None:              # the table spread by distance: row n for distance n, the last row for every larger one
                name, rows, far = self.rel_spec
                index = torch.tensor(distance_rows(int(rows), float(far)), dtype=torch.long, device=dev)
                self.rel_table = get(p + name).float().index_select(0, index).contiguous()
            if self.mix_name:
                self.head_mix = get(p + self.mix_name).float().contiguous()
            if self.head_gate_name:                    # one more block of the fused projection: the heads' gate logits, padded to whole 32 bytes
                g = get(p + self.head_gate_name)
                pad = -(-s.num_heads // 8) * 8 - s.num_heads
                self.w_qkv = torch.cat([self.w_qkv, g, g.new_zeros((pad, g.shape[1]))], dim=0).contiguous()

    def _padded_vec(self, v: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
        """A vector over heads of ``dim`` elements as one over heads of ``self.hd``, the new elements zero."""
        if dim == self.hd:
            return v
        return torch.nn.functional.pad(v.reshape(heads, dim), (0, self.hd - dim)).reshape(heads * self.hd).contiguous()

    def _padded_rows(self, w: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
        """A projection whose heads are ``dim`` wide as one whose heads are ``self.hd`` wide, the new rows zero."""
        if dim == self.hd:
            return w
        w = w.reshape(heads, dim, w.shape[1])
        return torch.nn.functional.pad(w, (0, 0, 0, self.hd - dim)).reshape(heads * self.hd, -1).contiguous()

    # -- one step --------------------------------------------------------- #
    def _view(self, cache) -> K.KvView:
        group, index = cache
        key = (id(group), index)
        if key not in self._views:
            if not isinstance(group, KVGroup):
                raise TypeError(f"attention reads keys and values from a 'kv' cache group, not from {type(group).__name__}")
            self._views[key] = K.KvView(group.layer_storage(index).data_ptr(), group.table.data_ptr(), group.table_width,
                                        group.ring_rows, group.page_size, group.num_pages, group.need.num_kv_heads,
                                        group.need.head_dim)
        return self._views[key]

    def _qk_args(self, qkv, width, q_buf, q_stride, view, lay, rope, T, hd, append: bool, zero_in: bool) -> K.QkArgs:
        s = self.spec
        qa = K.QkArgs()
        qa.inp, qa.in_stride = (None if qkv is None else qkv.data_ptr()), width
        qa.q_out, qa.q_stride = q_buf.data_ptr(), q_stride
        qa.k_out, qa.k_stride = None, 0
        qa.q_w = None if self.q_norm is None else self.q_norm.data_ptr()
        qa.k_w = None if self.k_norm is None else self.k_norm.data_ptr()
        qa.rope = rope                              # the position encoding's block, passed on as it is
        qa.eps = s.qk_norm.eps if s.qk_norm is not None else float(s.option("unit_norm_eps", 0.0))
        if self.unit_norm:
            qa.norm_dims, qa.norm_after = self.key_dim, int(self.unit_norm == "after_rotation")
        if self.value_norm is not None and not self.shared:
            qa.v_norm_dims, qa.v_eps = self.value_dim, float(self.value_norm)
        qa.nh, qa.nkv, qa.hd = s.num_heads, (0 if self.shared else s.num_kv_heads), hd
        qa.pos_of, qa.seq_of, qa.slot_of_seq = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr()
        qa.cache, qa.append, qa.T = view, int(append), T
        qa.zero_in = int(zero_in)
        qa.kv_len = lay.kv_len.data_ptr()
        return qa

    def _forward_shaped(self, h, ctx, cache, out: torch.Tensor) -> None:
        """Biases, norms over the whole projection, shaped and blended scores, one gate a head: one float32 product
        (Q | K | V | gate logits), the kernel that adds biases, norms, rounds and appends, the mixed-heads attention, the
        output projection."""
        s, lay = self.spec, ctx.layout
        T, Q, KV, hd = lay.T, self.Q, self.KV, self.hd
        view = self._view(cache)
        decode = lay.all_single
        width = self.w_qkv.shape[0]
        proj = ctx.empty((T, width), torch.float32)
        linear.matmul(rows_of(h), self.w_qkv, proj, linear.EPI_F32, ctx)
        q_buf = ctx.empty((T, Q))
        kv_rows = None if decode else ctx.empty((T, 2 * KV))
        append_now = decode or view.ring_rows == 0 or lay.all_fresh
        wa = K.WholeNormArgs()
        wa.inp, wa.in_stride = proj.data_ptr(), width
        wa.bias = None if self.bias is None else self.bias.data_ptr()
        if self.whole_norm:
            wa.q_w, wa.k_w, wa.eps = self.whole_q_w.data_ptr(), self.whole_k_w.data_ptr(), float(self.whole_norm[2])
            wa.q_count, wa.k_count = s.num_heads * self.key_dim, s.num_kv_heads * self.key_dim
        wa.q_out, wa.q_stride = q_buf.data_ptr(), Q
        wa.kv_out, wa.kv_stride = (None, 0) if kv_rows is None else (kv_rows.data_ptr(), 2 * KV)
        wa.nh, wa.nkv, wa.hd = s.num_heads, s.num_kv_heads, hd
        wa.pos_of, wa.seq_of, wa.slot_of_seq, wa.kv_len = lay.pos_of.data_ptr(), lay.seq_of.data_ptr(), lay.slot_of_seq.data_ptr(), lay.kv_len.data_ptr()
        wa.cache, wa.append, wa.T = view, int(append_now), T
        if self.b_o is not None:
            wa.o_bias, wa.o_out, wa.o_stride, wa.o_width = self.b_o.data_ptr(), out.data_ptr(), out.stride(0), s.hidden_size
        K.qkv_whole_norm(wa, q_buf.dtype, ctx.stream)

        attn = ctx.empty((T, Q))
        aa = K.AttnArgs()
        aa.q, aa.q_stride = q_buf.data_ptr(), Q
        aa.out, aa.out_stride = attn.data_ptr(), Q
        aa.cache, aa.batch = view, lay.c_struct()
        aa.nh, aa.nkv, aa.hd = s.num_heads, view.kv_heads, hd
        aa.window, aa.scale = s.window or 0, self.scale
        aa.softcap = self.softcap
        if self.rel_table is not None:
            aa.rel_bias, aa.rel_far = self.rel_table.data_ptr(), self.rel_table.shape[0] - 1
        aa.head_mix = None if self.head_mix is None else self.head_mix.data_ptr()
        if self.head_gate_name:
            aa.head_gate, aa.head_gate_stride = proj.data_ptr() + (Q + 2 * KV) * 4, width
        if decode:
            # a block takes all heads of one split of one sequence: splits of 32 keys (one round) while the sequences are few,
            # longer ones as they grow in number; by the batch size alone, so that eager and captured steps cut alike
            chunk = int(ctx.options.get("mixed_chunk", 32 if lay.B <= 4 else (64 if lay.B <= 16 else (128 if lay.B <= 64 else 256))))
            chunk, splits = decode_split(lay, view.kv_heads, dict(ctx.options, attn_chunk=chunk), False)
            need = lay.B * s.num_heads * splits * (hd + 2)
            scratch = ctx.scratch.get("attn_partials")
            if scratch is None or scratch.numel() < need:
                scratch = ctx.scratch["attn_partials"] = torch.empty(need, dtype=torch.float32, device=ctx.device)
            aa.kv_new, aa.kv_stride = None, 0
            aa.chunk, aa.n_splits, aa.scratch = chunk, splits, scratch.data_ptr()
            K.attn_mixed_decode(aa, q_buf.dtype, ctx.stream)
        else:
            aa.kv_new, aa.kv_stride = kv_rows.data_ptr(), 2 * KV
            K.attn_mixed_prefill(aa, q_buf.dtype, ctx.stream)
            if not append_now:
                K.kv_append(kv_rows, view, lay.c_struct(), ctx.stream)
        linear.matmul(attn, self.w_o, out, linear.EPI_ADD, ctx)

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        if self.shaped:
            return self._forward_shaped(h, ctx, cache, out)
        s, lay = self.spec, ctx.layout
        T, Q, KV, hd = lay.T, self.Q, self.KV, self.hd
        width = Q if self.shared else Q + 2 * KV
        view = self._view(cache)
        decode = lay.all_single
        rope = self.position.kernel_args(ctx.device)
        # A decode step in bfloat16 sums Q | K | V in float32 (K slices of the product add into a zeroed
        # buffer), and the norm/rotary kernel rounds once, into the query buffer and the cache.
        wide_sum = decode and not self.shared and h.dtype == torch.bfloat16 and ctx.options.get("gemm", "fast") != "plain"
        row_sums = None
        if wide_sum:
            key = f"acc_qkv_{T}x{width}"            # zeroed once; the norm/rotary kernel leaves it zeroed again (Engine.reset_accumulators after a failed step)
            qkv = ctx.scratch.get(key)
            if qkv is None:
                qkv = ctx.scratch[key] = torch.zeros((T, width), dtype=torch.float32, device=ctx.device)
            # The norm before the projection, if it was handed over unevaluated, goes into the product: the kernel
            # adds the products of the unscaled rows into the sums and leaves the rows' sums of squares, one part per
            # K slice, at a place of this step's own; the head norm/rotary kernel adds the parts and scales the rows first.
            if isinstance(h, DeferredNorm) and T <= 32:
                row_sums = ctx.row_sums()
                if row_sums is not None and K.gemm_tc_normed_accepts(h.x, h.weight, self.w_qkv, qkv, linear.EPI_ADD, row_sums):
                    K.gemm_tc_normed(h.x, h.weight, h.eps, self.w_qkv, qkv, linear.EPI_ADD, ctx.stream, sumsq=row_sums,
                                     ordered=bool(ctx.options.get("reproducible", False)))
                else:
                    row_sums = None
            if row_sums is None:
                linear.matmul(rows_of(h), self.w_qkv, qkv, linear.EPI_ADD, ctx)
            q_buf, q_stride = ctx.empty((T, Q)), Q
        else:
            qkv = ctx.empty((T, width))
            linear.matmul(rows_of(h), self.w_qkv, qkv, linear.EPI_STORE, ctx)
            q_buf, q_stride = qkv, width
        # K and V go into the cache in this kernel when nothing of this step still has to read the rows
        # they replace: always for single tokens and for caches that keep everything; in a ring only if
        # every sequence starts at position 0 (attention then reads the step's own rows alone).
        append_now = not self.shared and (decode or view.ring_rows == 0 or lay.all_fresh)
        qa = self._qk_args(qkv, width, q_buf, q_stride, view, lay, rope, T, hd, append=append_now, zero_in=wide_sum)
        if not (self.shared or wide_sum):
            qa.k_out, qa.k_stride = qkv.data_ptr() + Q * qkv.element_size(), width
        if row_sums is not None:
            qa.row_sumsq = row_sums.data_ptr()
            qa.row_parts = K.gemm_tc_normed_slices(self.w_qkv, linear.EPI_ADD, T, bool(ctx.options.get("reproducible", False)))
            qa.row_width, qa.row_eps = s.hidden_size, h.eps
        # A decode step whose Q | K | V are float32 sums may leave head norm, rotation and append to the attention
        # kernel itself (one kernel less between the projection and the attention); decided below, where the
        # attention's arguments are known.  Everything else runs the kernel now.
        if self.value_mix is not None:
            first, _ = self.value_mix
            if first is None:                                  # the values that later layers blend theirs with, kept for the step
                kept = ctx.empty((T, KV))
                qa.v_keep, qa.v_keep_stride = kept.data_ptr(), KV
                ctx.carried[("values_of", s.option("layer_index"))] = kept
            else:
                kept = ctx.carried.get(("values_of", first))
                if kept is None or kept.shape[0] != T or kept.shape[1] % s.num_kv_heads:
                    raise RuntimeError(f"the values of layer {first} that this layer blends with were not kept in this step")
                # (that layer may pad its heads to another width: the kernel reads a head's first elements from either)
                qa.v_first, qa.v_first_stride, qa.v_mix = kept.data_ptr(), kept.shape[1], self.mix_factor.data_ptr()
                qa.v_first_head = kept.shape[1] // s.num_kv_heads
                if not wide_sum:                               # the step's own V columns are what a prompt's attention reads
                    qa.v_keep, qa.v_keep_stride = qkv.data_ptr() + (Q + KV) * qkv.element_size(), width
        if self.value_norm is not None and not self.shared and not wide_sum and not qa.v_keep:
            # the normed values are what a prompt's attention reads: written back over the step's own V columns
            qa.v_keep, qa.v_keep_stride = qkv.data_ptr() + (Q + KV) * qkv.element_size(), width
        folds_head_norm = wide_sum and ctx.options.get("fold_head_norm", True) and not self.extended
        if not folds_head_norm:
            K.qk_norm_rope(qa, qkv.dtype, q_buf.dtype, ctx.stream)

        attn = ctx.empty((T, Q))
        aa = K.AttnArgs()
        aa.q, aa.q_stride = q_buf.data_ptr(), q_stride
        aa.out, aa.out_stride = attn.data_ptr(), Q
        aa.cache, aa.batch = view, lay.c_struct()
        aa.nh, aa.nkv, aa.hd = s.num_heads, view.kv_heads, hd
        aa.window, aa.scale = s.window or 0, self.scale
        aa.sink = None if self.sink is None else self.sink.data_ptr()
        aa.keep_first = self.keep_first if s.window else 0
        if decode:
            fast = ctx.options.get("attention", "fast") != "plain" and q_buf.dtype == torch.bfloat16 and hd in (64, 128)
            chunk, splits = decode_split(lay, view.kv_heads, ctx.options, fast)
            need = lay.B * s.num_heads * splits * (hd + 2)
            scratch = ctx.scratch.get("attn_partials")
            if scratch is None or scratch.numel() < need:
                scratch = ctx.scratch["attn_partials"] = torch.empty(need, dtype=torch.float32, device=ctx.device)
            aa.kv_new, aa.kv_stride = None, 0
            aa.chunk, aa.n_splits, aa.scratch = chunk, splits, scratch.data_ptr()
            if ctx.options.get("early_pages", True):       # lengths the kernel may read before its predecessors end
                if lay.lengths_by_copy:
                    aa.early_len, aa.early_mode = lay.kv_len.data_ptr(), 1
                elif lay.committed_len is not None:
                    aa.early_len, aa.early_mode = lay.committed_len.data_ptr(), 2
            if folds_head_norm:
                aa.fused_qk = ctypes.pointer(qa)
                if not (fast and K.attn_decode_mma_accepts(aa, q_buf.dtype)):      # the kernel cannot take it in: as a kernel of its own, then
                    aa.fused_qk = None
                    K.qk_norm_rope(qa, qkv.dtype, q_buf.dtype, ctx.stream)
            if fast and K.attn_decode_mma_accepts(aa, q_buf.dtype):
                K.attn_decode_mma(aa, ctx.stream)
            else:
                K.attn_decode(aa, q_buf.dtype, ctx.stream)
        else:
            if self.shared:
                aa.kv_new, aa.kv_stride = None, 0
            else:
                aa.kv_new, aa.kv_stride = qkv.data_ptr() + Q * qkv.element_size(), width
            mode = ctx.options.get("attention", "fast")   # "fast" | "mma" | "plain"
            # The tensor-core kernels read keys and values from the step's own rows when every sequence starts at
            # position 0, and else from the cache's pages, if the step's keys lie there already (a cache that keeps
            # everything; a reader of another layer's cache finds them there in any case).
            if lay.all_fresh and not self.shared:
                source = K.KV_FROM_STEP
            elif view.ring_rows == 0 and (self.shared or append_now):
                source = K.KV_FROM_CACHE
            else:
                source = K.KV_NOWHERE
            if hd not in (64, 128):                       # what the tensor-core kernels are built for: nothing else asks for (and compiles) them
                source = K.KV_NOWHERE
            if mode == "fast" and source and K.attn_prefill_tc_accepts(aa, q_buf.dtype, source):
                K.attn_prefill_tc(aa, source, ctx.stream)
            elif mode in ("fast", "mma") and source and K.attn_prefill_mma_accepts(aa, q_buf.dtype, source):
                K.attn_prefill_mma(aa, source, ctx.stream)
            else:
                K.attn_prefill(aa, q_buf.dtype, ctx.stream)
            if not self.shared and not append_now:
                K.kv_append(qkv[:, Q:], view, lay.c_struct(), ctx.stream)
        if self.w_gate is not None:                  # the heads times sigmoid(W_g h) (and the mixer's factor), in place
            gate = ctx.empty((T, Q))
            linear.matmul(rows_of(h), self.w_gate, gate, linear.EPI_STORE, ctx)
            K.gate_rows(attn, gate, attn, K.GATE_SIGMOID, self.output_scale, ctx.stream)
        elif self.output_scale != 1.0:
            raise NotImplementedError("an output scale is applied with the output gate; a mixer without a gate has none")
        linear.matmul(attn, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("attention", AttentionMixer)
