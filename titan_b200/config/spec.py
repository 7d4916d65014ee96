"""Architecture-neutral description of a decoder: what every part is built from.

An architecture's typed configuration (for instance ``Qwen3Config``) turns its
own ``config.json`` keys into a ``ModelSpec``.  Parts are built from the specs
below and never see the architecture's configuration, so no part knows which
model it is in.  A spec carries a ``kind`` string that names the part's class in
the part registries (``titan_b200.parts``), its sizes and its constants.

berniehans/titan keeps the same numbers in one flat ``ModelConfig``
(engine/engine-io/src/config.rs:36-72) and hard-codes the arrangement in
``ForwardDriver`` (engine/engine-core/src/forward_driver.rs:988-1207); here the
arrangement is data.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value that is not supported."""


@dataclass(frozen=True)
class NormSpec:
    kind: str                 # "rmsnorm"
    size: int
    eps: float
    weight: str               # tensor name relative to the owner's prefix
    weight_offset: float = 0.0  # the rows are multiplied by (weight_offset + stored weight): 1.0 for weights stored around zero
    groups: int = 1           # the row is cut into this many equal runs, each divided by its own root mean square (1: the whole row by one)


@dataclass(frozen=True)
class PositionSpec:
    kind: str                 # "rope" | "none"
    rotary_dim: int = 0       # leading dims of a head that are rotated
    theta: float = 10000.0
    pairing: str = "half"     # "half": (k, k + rotary_dim/2) turn together; "adjacent": (2k, 2k + 1)


def _lookup(pairs, key, default):
    for k, v in pairs:
        if k == key:
            return v
    return default


@dataclass(frozen=True)
class MixerSpec:
    kind: str                 # "attention" | "latent_attention" | "lightning" | "retention" | "wkv" | "gated_delta" | "mlstm" | "parallel"
    hidden_size: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None          # None: all keys; n: keys p-n < t <= p
    qk_norm: Optional[NormSpec] = None    # per-head norm on Q and K before the rotation
    position: PositionSpec = PositionSpec("none")
    softmax_scale: Optional[float] = None  # None: 1/sqrt(head_dim)
    cache_from: Optional[int] = None      # read (and do not write) this layer's cache
    prefix: str = "self_attn."
    # Tensor names by role, relative to ``prefix``; roles a part knows and that are not listed keep the
    # part's default.  Attention: "q", "k", "v", "o" (defaults q_proj.weight ...), or "qkv" for a checkpoint
    # that stores the three projections as one [Q + 2 KV, H] tensor.
    names: Tuple[Tuple[str, str], ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = ()   # for mixers defined outside the package

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)

    def name(self, role: str, default: Optional[str] = None) -> Optional[str]:
        return _lookup(self.names, role, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                 # "gated_mlp" | "mlp" | "moe" | "token_table"
    hidden_size: int
    intermediate_size: int = 0
    activation: str = "silu"
    prefix: str = "mlp."
    # Tensor names by role: "gate", "up", "down" (defaults gate_proj.weight ...), or "gate_up" for a
    # checkpoint that stores gate and up as one [2 F, H] tensor (gate rows first).
    names: Tuple[Tuple[str, str], ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)

    def name(self, role: str, default: Optional[str] = None) -> Optional[str]:
        return _lookup(self.names, role, default)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which mixer, which feed-forward, which norms, how arranged.  The arrangement gives the
    fields their meaning: ``pre_norm`` needs all four parts; another arrangement may do without a
    feed-forward (None), or take more norms than two from ``norms`` (a norm after each part as well as
    before it, say) and its own constants from ``extra``."""
    index: int
    arrangement: str          # "pre_norm" | "pre_norm_scaled" | "output_norm" | "hyper" | "parallel"
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: Optional[NormSpec]
    feed_forward_norm: Optional[NormSpec]
    prefix: str               # "model.layers.3."
    norms: Tuple[NormSpec, ...] = ()          # further norms, in the order the arrangement defines
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[int, ...]                # indices into ``layers`` in running order
    final_norm: NormSpec
    embedding: str = "model.embed_tokens.weight"
    lm_head: Optional[str] = "lm_head.weight"   # None: tied to the embedding
    max_positions: int = 4096
    stop_token_ids: Tuple[int, ...] = ()
    embedding_scale: Optional[float] = None   # the embedded rows are multiplied by this (None: as stored)
    logit_scale: Optional[float] = None       # the logits are multiplied by this (None: as computed)
    embedding_norm: Optional[NormSpec] = None  # a norm on the embedded rows, before the first layer (None: none)
    streams: int = 1                          # copies of the residual stream that the blocks keep (the "hyper" arrangement); their sum leaves the last block
    # Tensors that no single layer owns (a table that every layer reads a slice of): (name, shape) pairs.  The model
    # loads each once and hands the dict to every part that has ``bind_shared``.
    shared_tensors: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()
    # Tensors that a file of this model may hold although the model, as described, uses none of them (the factor of a
    # mechanism that a layer's description switches off): present or absent, they are not an error and are not loaded.
    ignorable_tensors: Tuple[str, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ConfigError(f"layer order names layer {i}, but there are {len(self.layers)} layers")
        if self.streams < 1 or (self.streams > 1 and any(l.arrangement != "hyper" for l in self.layers)):
            raise ConfigError(f"{self.streams} residual streams need every block to be of the 'hyper' arrangement")
        for layer in self.layers:
            src = layer.mixer.cache_from
            if src is None:
                continue
            me = layer.mixer
            if not 0 <= src < len(self.layers) or self.layers[src].mixer.cache_from is not None:
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src}, which owns none")
            if layer.index not in self.order:
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src} but never runs (it is not in the order)")
            if src not in self.order or self.order.index(src) > self.order.index(layer.index):
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src} before it is written")
            owner = self.layers[src].mixer
            if owner.kind != me.kind:
                raise ConfigError(f"layer {layer.index} ({me.kind}) reads the cache of layer {src}, whose mixer is of another kind ({owner.kind})")
            why = _SHARING_RULES.get(me.kind, lambda *a: None)(layer.index, me, src, owner)
            if why:
                raise ConfigError(why)


def _share_kv(index, me, src, owner):
    """Grouped-query attention reading another layer's keys and values."""
    if owner.window != me.window:
        return (f"layer {index} reads the cache of layer {src}, which keeps a window of {owner.window} keys, "
                f"with a window of {me.window}: a reader must see exactly what the owner keeps")
    if owner.head_dim != me.head_dim:
        return f"layer {index} has heads of {me.head_dim}, the cache of layer {src} holds heads of {owner.head_dim}"
    if owner.num_kv_heads <= 0 or me.num_heads % owner.num_kv_heads:
        return (f"layer {index} has {me.num_heads} query heads, not a multiple of the {owner.num_kv_heads} "
                f"kv heads in the cache of layer {src}")
    return None


def _share_latent(index, me, src, owner):
    """Latent attention reading another layer's latents: the cached row must mean the same to both (latent size,
    rotated size, rotation), and the owner must keep at least the keys the reader's window reaches."""
    for key in ("kv_rank", "rot_dim"):
        if owner.option(key) != me.option(key):
            return f"layer {index} has {key} {me.option(key)}, the cache of layer {src} holds {key} {owner.option(key)}"
    if owner.position != me.position:
        return f"layer {index} rotates its keys otherwise than layer {src}, whose cache it reads"
    kept = owner.option("cache_window", owner.window)
    if kept is not None and (me.window is None or me.window > kept):
        return f"layer {index} looks {me.window} keys back, the cache of layer {src} keeps {kept}"
    return None


_SHARING_RULES = {"attention": _share_kv, "latent_attention": _share_latent}
