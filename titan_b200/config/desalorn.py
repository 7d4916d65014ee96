"""Typed configuration of the Desalorn design, from its config.json.

A Desalorn model is a list of layers in which ONE norm feeds both sublayers: with h = norm1(x), x += m * (mixer(h) + ff(h)),
m one number for the whole model (the block arrangement ``parallel``).  The norm is an RMS norm in groups: the row is cut into
equal runs and each is divided by its own root mean square.  The embedded rows are multiplied by a constant.  Mixers:

* ``attention``: grouped queries with biases on every projection, one norm over all of a token's queries and one over all of
  its keys, no rotation; scores are capped by a tanh, get a learned bias by distance (a table whose rows are reached by the
  distance itself at first and by its logarithm further out) and are blended across heads by a matrix before the causal
  softmax; one sigmoid gate a head on the output.
* ``retention``: linear attention with a fixed decay a head, rotated (halves paired) queries and keys, no softmax and no
  denominator; unit norm a head, a silu gate.
* ``latent_attention``: attention over one shared latent a token with a rotated (neighbours paired) key part, queries through
  a latent of their own, a sliding window.

Feed-forward: a mixture of experts (sigmoid scores, choice by score + correction among the groups whose two best add up
highest, weights not renormalised, a shared expert without a gate), or none.  The keys read here:

    architecture "Desalorn";  vocab, width;  embedding.scale;  norm {eps, groups};  residual_mult
    layers[i].type "attention":        mixer {heads, kv_heads, dim, vdim, scale, softcap, bias_max}  (+ bias_rows, if no tensor gives it)
    layers[i].type "retention":        mixer {heads, dim, vdim, decay [heads], rot {base, dims}}
    layers[i].type "latent_attention": mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}, mask {size}}
    layers[i].mlp  null | {kind "moe", expert {ff}, router {experts, top, groups {count, keep}}, shared {ff} (optional)}

The number of rows of an attention layer's distance table is the shape of its tensor ``l<i>.mix.rel``; a description without a
model folder gives it as ``bias_rows``.

Tensor names: embed, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tefezen import _get

# No position limit is part of the design; positions are exact in float32 up to here.
MAX_POSITIONS = 1 << 24


def _rotation(m, limit, where):
    dims, base = _get(m, "rot.dims", int), _get(m, "rot.base", float)
    if dims % 2 or dims > limit or not base > 0:
        raise ConfigError(f"{where}: rot.dims {dims} must be even and at most {limit}, rot.base positive")


@dataclass(frozen=True)
class DesalornConfig:
    raw: Any                       # the config.json dict, checked, with every attention layer's bias_rows filled in
    architecture: str = "Desalorn"
    reads_tensor_shapes = True     # ``from_dict`` takes the shapes of the folder's tensors (name -> shape) where there is a folder

    def __hash__(self):
        return id(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], shapes: Optional[Dict[str, tuple]] = None) -> "DesalornConfig":
        d = copy.deepcopy(d)
        W = _get(d, "width", int)
        _get(d, "vocab", int)
        if not _get(d, "norm.eps", float) > 0:
            raise ConfigError("norm.eps must be positive")
        groups = _get(d, "norm.groups", int, 1)
        if W % groups:
            raise ConfigError(f"norm.groups {groups} does not divide the width {W}")
        _get(d, "residual_mult", float, 1.0)
        _get(d, "embedding.scale", float, 1.0)
        layers = _get(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind, m = _get(layer, "type"), _get(layer, "mixer")
            heads, dim = _get(m, "heads", int), _get(m, "dim", int)
            _get(m, "vdim", int)
            if kind == "attention":
                kv = _get(m, "kv_heads", int)
                if heads % kv:
                    raise ConfigError(f"{where}: {heads} query heads are not a multiple of {kv} key/value heads")
                _get(m, "scale", float)
                if m.get("softcap") is not None and not _get(m, "softcap", float) > 0:
                    raise ConfigError(f"{where}: softcap must be positive")
                if m.get("bias_rows") is None:
                    shape = (shapes or {}).get(f"l{i}.mix.rel")
                    if shape is None or len(shape) != 2:
                        raise ConfigError(f"{where}: the distance table's rows are neither in the description ('bias_rows') nor given by a tensor l{i}.mix.rel")
                    m["bias_rows"] = int(shape[0])
                rows, far = _get(m, "bias_rows", int), _get(m, "bias_max", float)
                if rows >= 2 and not far > rows // 2:
                    raise ConfigError(f"{where}: bias_max {far} must lie beyond half of the table's {rows} rows")
            elif kind == "retention":
                decay = _get(m, "decay")
                if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(x, (int, float)) and 0 <= x <= 1 for x in decay):
                    raise ConfigError(f"{where}: 'decay' must list one number in [0, 1] for each of the {heads} heads")
                _rotation(m, dim, where)
            elif kind == "latent_attention":
                rd = _get(m, "rot_dim", int)
                _get(m, "kv_rank", int), _get(m, "q_rank", int), _get(m, "mask.size", int), _get(m, "scale", float)
                _rotation(m, rd, where)
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not known (attention, retention, latent_attention)")
            f = layer.get("mlp")
            if f is None:
                continue
            if f.get("kind") != "moe":
                raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not known (moe)")
            E, top = _get(f, "router.experts", int), _get(f, "router.top", int)
            g = f["router"].get("groups")
            count, keep = (1, 1) if g is None else (_get(g, "count", int), _get(g, "keep", int))
            if keep > count or E % count or top > keep * (E // count):
                raise ConfigError(f"{where}: {top} of {E} experts in {count} groups of which {keep} are open")
            _get(f, "expert.ff", int)
            if f.get("shared") is not None:
                _get(f, "shared.ff", int)
        return cls(raw=d, architecture=d.get("architecture") or (d.get("architectures") or ["Desalorn"])[0])

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    # ------------------------------------------------------------------ #
    def to_model_spec(self) -> ModelSpec:
        d = self.raw
        W, V, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        groups = int(d["norm"].get("groups") or 1)
        mult = float(_get(d, "residual_mult", float, 1.0))
        norm = lambda name: NormSpec("rmsnorm", W, eps, name, groups=groups)
        plain = lambda name, size: NormSpec("rmsnorm", size, eps, name)
        layers = []
        for i, layer in enumerate(d["layers"]):
            m = layer["mixer"]
            if layer["type"] == "attention":
                extra = [("value_dim", m["vdim"]), ("bias", True), ("whole_norm", ("q.norm", "k.norm", eps)),
                         ("rel_bias", ("rel", int(m["bias_rows"]), float(m["bias_max"]))), ("head_mix", "talk"), ("head_gate", "g")]
                if m.get("softcap") is not None:
                    extra.append(("softcap", float(m["softcap"])))
                mixer = MixerSpec(kind="attention", hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                  softmax_scale=float(m["scale"]), prefix="mix.", position=PositionSpec("none"),
                                  names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")), extra=tuple(extra))
            elif layer["type"] == "retention":
                mixer = MixerSpec(kind="retention", hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], prefix="mix.",
                                  position=PositionSpec("rope", rotary_dim=m["rot"]["dims"], theta=float(m["rot"]["base"]), pairing="half"),
                                  extra=(("value_dim", m["vdim"]), ("decay", tuple(float(x) for x in m["decay"])), ("norm_eps", eps)))
            else:
                mixer = MixerSpec(
                    kind="latent_attention", hidden_size=W, num_heads=m["heads"], num_kv_heads=1, head_dim=m["dim"],
                    window=int(m["mask"]["size"]), softmax_scale=float(m["scale"]), prefix="mix.",
                    position=PositionSpec("rope", rotary_dim=m["rot"]["dims"], theta=float(m["rot"]["base"]), pairing="adjacent"),
                    extra=(("rot_dim", m["rot_dim"]), ("value_dim", m["vdim"]), ("kv_rank", m["kv_rank"]),
                           ("latent_norm", plain("dkv.norm", m["kv_rank"])), ("q_rank", m["q_rank"]), ("q_norm", plain("dq.norm", m["q_rank"]))))
            f = layer.get("mlp")
            ffn = None
            if f is not None:
                r = f["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                shared = f.get("shared")
                ffn = FeedForwardSpec(kind="moe", hidden_size=W, intermediate_size=f["expert"]["ff"], activation="silu", prefix="mlp.",
                                      extra=(("experts", r["experts"]), ("top", r["top"]), ("routing", "sigmoid_all"),
                                             ("groups", g["count"]), ("keep", g["keep"]), ("group_best", 2), ("renormalize", False),
                                             ("shared_size", 0 if shared is None else shared["ff"]), ("shared_gate", False)))
            layers.append(LayerSpec(index=i, arrangement="parallel", mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
                                    feed_forward_norm=None, prefix=f"l{i}.", extra=(("residual_mult", mult),)))
        scale = float(_get(d, "embedding.scale", float, 1.0))
        spec = ModelSpec(architecture=self.architecture, hidden_size=W, vocab_size=V, layers=tuple(layers), order=tuple(range(len(layers))),
                         final_norm=norm("final.norm"), embedding="embed", lm_head="head", max_positions=MAX_POSITIONS,
                         embedding_scale=None if scale == 1.0 else scale)
        spec.validate()
        return spec
