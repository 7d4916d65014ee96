"""Typed configuration of the Vuvosun design, from its config.json.

A Vuvosun model keeps several copies of the residual stream ("hyper-connections": every sublayer reads one learned blend
of them through an RMS norm, and its result is written into each while the streams are mixed among themselves; the block
arrangement ``hyper``).  The embedded rows pass an RMS norm first; the logits come from the embedding table.  Mixers:

* ``parallel``: two mixers on the same input, their results added with one factor each.  ``left``: softmax attention with
  grouped queries, neighbouring dimensions rotated in pairs, values divided by their root mean square per head before they are
  cached, a sliding window that also keeps a sequence's first tokens, a learned sink in the softmax's denominator and a
  sigmoid gate on the concatenated heads.  ``right``: the gated delta rule behind short causal convolutions.
* ``mlstm``: the matrix memory of xLSTM with capped gates.

Feed-forward: ``dense``, down(polynorm(up(x))), or none.  The keys read here:

    architecture "Vuvosun";  vocab, width, streams;  norm.eps
    layers[i].type "parallel": mixer {left {heads, kv_heads, dim, vdim, rot {base, dims}, scale, mask {size, keep_first}},
                                      right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale}
    layers[i].type "mlstm":    mixer {heads, dim, vdim, gate_cap}
    layers[i].mlp  null | {kind "dense", ff}

Tensor names: embed, embed.norm, l<i>.norm1|norm2, l<i>.hc1|hc2.in|out|mix, l<i>.mix.*, l<i>.mlp.up|down|act, final.norm.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict

from .spec import ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tefezen import _get

# No position limit is part of the design; positions are exact in float32 up to here.
MAX_POSITIONS = 1 << 24
MAX_STREAMS = 8


def _count(d, path, where):
    """A key that holds a count (0 allowed), or is absent (0)."""
    v = _get(d, path, default=0)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != int(v) or v < 0:
        raise ConfigError(f"{where}: {path} {v!r} must be a count")
    return int(v)


@dataclass(frozen=True)
class VuvosunConfig:
    raw: Any                       # the config.json dict, checked
    architecture: str = "Vuvosun"

    def __hash__(self):
        return id(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VuvosunConfig":
        d = copy.deepcopy(d)
        _get(d, "vocab", int), _get(d, "width", int)
        if not _get(d, "norm.eps", float) > 0:
            raise ConfigError("norm.eps must be positive")
        if _get(d, "streams", int) > MAX_STREAMS:
            raise ConfigError(f"{d['streams']} residual streams (at most {MAX_STREAMS})")
        layers = _get(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind, m = _get(layer, "type"), _get(layer, "mixer")
            if kind == "parallel":
                a, r = _get(m, "left"), _get(m, "right")
                heads, kv, dim = _get(a, "heads", int), _get(a, "kv_heads", int), _get(a, "dim", int)
                _get(a, "vdim", int)
                if heads % kv:
                    raise ConfigError(f"{where}: {heads} query heads are not a multiple of {kv} key/value heads")
                dims, base = _get(a, "rot.dims", int), _get(a, "rot.base", float)
                if dims % 2 or dims > dim or not base > 0:
                    raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {dim}, rot.base positive")
                _get(a, "scale", float)
                if a.get("mask") is not None:
                    _get(a, "mask.size", int)
                    _count(a, "mask.keep_first", where)
                heads, kv = _get(r, "heads", int), _get(r, "kv_heads", int)
                _get(r, "dim", int), _get(r, "vdim", int)
                if heads % kv:
                    raise ConfigError(f"{where}: {heads} value heads are not a multiple of {kv} key heads")
                if _get(r, "conv", int) > 64:
                    raise ConfigError(f"{where}: a convolution of {r['conv']} taps (at most 64)")
                _get(m, "left_scale", float), _get(m, "right_scale", float)
            elif kind == "mlstm":
                _get(m, "heads", int), _get(m, "dim", int), _get(m, "vdim", int)
                if not _get(m, "gate_cap", float) > 0:
                    raise ConfigError(f"{where}: gate_cap must be positive")
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not known (parallel, mlstm)")
            f = layer.get("mlp")
            if f is None:
                continue
            if f.get("kind") != "dense":
                raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not known (dense)")
            _get(f, "ff", int)
        return cls(raw=d, architecture=d.get("architecture") or (d.get("architectures") or ["Vuvosun"])[0])

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    # ------------------------------------------------------------------ #
    def to_model_spec(self) -> ModelSpec:
        d = self.raw
        W, V, S, eps = d["width"], d["vocab"], d["streams"], float(d["norm"]["eps"])
        norm = lambda name: NormSpec("rmsnorm", W, eps, name)
        layers, unused = [], []
        for i, layer in enumerate(d["layers"]):
            m = layer["mixer"]
            if layer["type"] == "parallel":
                a, r = m["left"], m["right"]
                mask = a.get("mask") or {}
                keep = int(mask.get("keep_first") or 0) if mask.get("size") else 0
                left = MixerSpec(
                    kind="attention", hidden_size=W, num_heads=a["heads"], num_kv_heads=a["kv_heads"], head_dim=a["dim"],
                    window=mask.get("size"), softmax_scale=float(a["scale"]), prefix="left.",
                    position=PositionSpec("rope", rotary_dim=a["rot"]["dims"], theta=float(a["rot"]["base"]), pairing="adjacent"),
                    names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")),
                    extra=(("value_dim", a["vdim"]), ("value_norm", eps), ("keep_first", keep), ("sink", "sink"), ("out_gate", "g"),
                           ("output_scale", float(m["left_scale"]))))
                right = MixerSpec(
                    kind="gated_delta", hidden_size=W, num_heads=r["heads"], num_kv_heads=r["kv_heads"], head_dim=r["dim"], prefix="right.",
                    extra=(("value_dim", r["vdim"]), ("taps", r["conv"]), ("norm_eps", eps), ("output_scale", float(m["right_scale"]))))
                mixer = MixerSpec(kind="parallel", hidden_size=W, prefix="mix.", extra=(("branches", (left, right)),))
            else:
                mixer = MixerSpec(kind="mlstm", hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], prefix="mix.",
                                  extra=(("value_dim", m["vdim"]), ("gate_cap", float(m["gate_cap"])), ("norm_eps", eps)))
            f = layer.get("mlp")
            ffn = None
            if f is not None:
                ffn = FeedForwardSpec(kind="mlp", hidden_size=W, intermediate_size=f["ff"], activation="polynorm", prefix="mlp.",
                                      extra=(("act_eps", eps),))
            else:                  # a file may carry the second sublayer's small tensors of a layer that has none
                unused += [f"l{i}.norm2"] + [f"l{i}.hc2.{s}" for s in ("in", "out", "mix")]
            layers.append(LayerSpec(index=i, arrangement="hyper", mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
                                    feed_forward_norm=None if ffn is None else norm("norm2"), prefix=f"l{i}.",
                                    extra=(("connections", ("hc1",) if ffn is None else ("hc1", "hc2")), ("streams", S))))
        spec = ModelSpec(architecture=self.architecture, hidden_size=W, vocab_size=V, layers=tuple(layers), order=tuple(range(len(layers))),
                         final_norm=norm("final.norm"), embedding="embed", lm_head=None, max_positions=MAX_POSITIONS,
                         embedding_norm=norm("embed.norm"), streams=S, ignorable_tensors=tuple(unused))
        spec.validate()
        return spec
