"""Small Desalorn configurations for the tests, each unlike the others in every size, option and layer order, and random
weights that a bfloat16 file holds exactly.  The list of a model's tensors is ``plain.desalorn_plain.tensor_shapes``."""
import copy

import torch

from plain import desalorn_plain as P


def attention(heads, kv_heads, dim, vdim, scale, softcap, rows, far):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "bias_max": far, "bias_rows": rows}


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": rot_dims}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, size, scale, base=10000.0):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": size},
            "scale": scale, "rot": {"base": base, "dims": rot_dim}}


def moe(experts, top, ff, count, keep, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}},
            "shared": None if shared is None else {"ff": shared}}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(layers, width, vocab, eps, groups, mult, embed_scale):
    return {"architecture": "Desalorn", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "residual_mult": mult,
            "embedding": {"scale": embed_scale}, "layers": layers}


CASES = {
    # attention / retention / latent without feed-forward; three norm groups; part of a retention head rotated; a table of eight
    # rows; groups of experts of which half are open
    "mix": lambda: model([layer("attention", attention(4, 2, 16, 16, 0.3, 5.0, 8, 40), moe(8, 2, 24, 4, 2, shared=40)),
                          layer("retention", retention(3, 8, 12, (0.9, 0.97, 0.995), 4, base=300.0), moe(8, 2, 24, 4, 2, shared=40)),
                          layer("latent_attention", latent(2, 16, 8, 12, 20, 12, 20, 0.2, base=50.0))],
                         width=48, vocab=97, eps=1e-5, groups=3, mult=0.5, embed_scale=3.0),
    # latent first; one norm group; widths that are no multiples of 8; keys and values of unequal width; a table with an odd number
    # of rows; one kv head, and as many kv heads as heads; a window of seven (a ring that turns many times); all groups open, one
    # group, three experts a token, no shared expert; a retention head rotated whole; a residual factor of one
    "odd": lambda: model([layer("latent_attention", latent(3, 12, 4, 20, 28, 9, 7, 0.25, base=500.0), moe(6, 3, 20, 1, 1)),
                          layer("attention", attention(3, 1, 12, 20, 0.3, 30.0, 5, 17.0), moe(6, 3, 20, 3, 3, shared=33)),
                          layer("retention", retention(1, 40, 20, (0.9990234375,), 40, base=77.0)),
                          layer("attention", attention(6, 6, 8, 8, 0.5, 2.0, 12, 300), moe(9, 1, 16, 3, 1)),
                          layer("retention", retention(5, 4, 36, (0.5, 0.8, 0.9, 0.99, 1.0), 2), moe(4, 4, 8, 2, 2, shared=8))],
                         width=56, vocab=131, eps=3e-6, groups=1, mult=1.0, embed_scale=1.0),
    # heads of 64 and 128; latent attention at the sizes whose whole prompts run on tensor cores in bfloat16, with a window of a
    # page; eight heads whose scores are blended; two norm groups; one expert a token out of the one open group
    "wide": lambda: model([layer("retention", retention(2, 64, 128, (0.96, 0.999), 32), moe(4, 1, 64, 2, 1, shared=128)),
                           layer("attention", attention(8, 2, 64, 64, 0.125, 50.0, 32, 128), moe(16, 4, 32, 8, 3)),
                           layer("latent_attention", latent(2, 128, 64, 128, 64, 48, 64, 0.07), moe(4, 2, 64, 1, 1, shared=64)),
                           layer("attention", attention(2, 1, 128, 64, 0.09, 20.0, 16, 1000))],
                          width=128, vocab=211, eps=1e-6, groups=2, mult=0.3, embed_scale=8.0),
}


def make_config(name):
    return copy.deepcopy(CASES[name]())


def rel_rows(cfg):
    """Rows of the distance tables (one number for the model's attention layers, as ``tensor_shapes`` wants it; None if they differ)."""
    rows = {l["mixer"]["bias_rows"] for l in cfg["layers"] if l["type"] == "attention"}
    return rows.pop() if len(rows) == 1 else None


def shapes_of(cfg):
    """name -> shape, with every attention layer's own number of table rows."""
    out = P.tensor_shapes(cfg, 0)
    for i, l in enumerate(cfg["layers"]):
        if l["type"] == "attention":
            out[f"l{i}.mix.rel"] = (l["mixer"]["bias_rows"], l["mixer"]["heads"])
    return out


def random_weights(cfg, seed):
    """float32 torch tensors that bfloat16 holds exactly.  Matrices ~ N(0, 1/fan_in) (the embedding N(0, 1)); the small tensors are
    spread so that every mechanism matters: biases and distance tables that move scores by about one, blending matrices well
    away from the identity, router outputs of a few units and corrections that change the choice."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes_of(cfg).items():
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = n()
        elif "norm" in last:
            t = n(0.2, 1.0)
        elif last == "b":
            t = n(0.3)
        elif last == "rel":
            t = n(1.0)
        elif last == "talk":
            t = torch.eye(shape[0]) + torch.randn(shape, generator=g) * 0.3
        elif last == "correction":
            t = n(0.3)
        elif last == "router":
            t = n(3.0 / shape[-1] ** 0.5)
        elif name.endswith("mix.g") and len(shape) == 2 and shape[0] < 64:
            t = n(2.0 / shape[-1] ** 0.5)
        else:
            t = n(1.0 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16).float()
    return out


def as_numpy(weights):
    return {k: v.double().numpy() for k, v in weights.items()}
