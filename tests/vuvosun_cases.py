"""Small Vuvosun configurations for the tests, each unlike the others in every size, option and layer order; the list of a
model's tensors written out by hand; and random weights that a bfloat16 file holds exactly."""
import copy

import numpy as np
import torch


def left(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=0.25, size=None, keep_first=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims}, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep_first}
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(l, r, left_scale=1.0, right_scale=1.0, ff=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm(heads, dim, vdim, cap, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(layers, width, vocab, eps, streams):
    return {"architecture": "Vuvosun", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps}, "layers": layers}


CASES = {
    # parallel / mlstm without feed-forward / parallel; two streams; a window of 20 that keeps three first tokens; part of the
    # head rotated; value heads of another width than the keys in the recurrence
    "mix": lambda: model([parallel(left(4, 2, 16, 16, 8, base=300.0, scale=0.3, size=20, keep_first=3), right(4, 2, 8, 12, 3), 0.8, 1.3, ff=40),
                          mlstm(3, 8, 12, 10.0),
                          parallel(left(2, 1, 24, 8, 24, base=50.0, scale=0.2, size=33, keep_first=1), right(2, 2, 12, 4, 4), 1.1, 0.6, ff=24)],
                         width=48, vocab=97, eps=1e-5, streams=2),
    # mlstm first; three streams; widths that are no multiples of 8; one kv head; a window without kept tokens (a ring in the
    # cache) and one wider than every prompt; a convolution of two taps and one of five; a layer without feed-forward; as many
    # kv heads as heads; an odd feed-forward width
    "odd": lambda: model([mlstm(1, 40, 20, 15.0, ff=33),
                          parallel(left(3, 1, 12, 20, 4, base=500.0, scale=0.3, size=7, keep_first=0), right(2, 2, 20, 8, 2), 1.5, 0.5),
                          parallel(left(6, 6, 8, 8, 8, base=77.0, scale=0.6, size=300, keep_first=2), right(3, 1, 4, 36, 5), 0.7, 1.0, ff=50),
                          mlstm(2, 20, 24, 6.0, ff=18)],
                         width=56, vocab=131, eps=3e-6, streams=3),
    # one stream; heads of 64 and of 128 (in bfloat16 the tensor-core kernels where the mask lets them); no mask at all; a
    # window over a ring at a page's width; kept tokens beyond a page; one tap (no convolution state)
    "wide": lambda: model([parallel(left(4, 2, 64, 64, 16, base=30000.0, scale=0.14, size=64, keep_first=0), right(4, 2, 64, 64, 4), 1.0, 1.0, ff=192),
                           parallel(left(2, 1, 128, 128, 64, scale=0.09), right(2, 1, 32, 64, 1), 0.9, 1.2, ff=128),
                           mlstm(2, 64, 128, 12.0, ff=64),
                           parallel(left(4, 4, 64, 32, 64, scale=0.11, size=40, keep_first=70), right(8, 4, 16, 16, 3), 1.0, 0.4)],
                          width=128, vocab=211, eps=1e-6, streams=1),
}


def make_config(name):
    return copy.deepcopy(CASES[name]())


def tensor_shapes(cfg):
    """name -> shape of every tensor of a model, written from the design's description."""
    W, V, S = cfg["width"], cfg["vocab"], cfg["streams"]
    out = {"embed": (V, W), "embed.norm": (W,), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = ["1"] if layer["mlp"] is None else ["1", "2"]
        for q in subs:
            out[p + "norm" + q] = (W,)
            out[p + f"hc{q}.in"], out[p + f"hc{q}.out"], out[p + f"hc{q}.mix"] = (S,), (S,), (S, S)
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            out[q + "q"], out[q + "k"], out[q + "v"] = (a["heads"] * a["dim"], W), (a["kv_heads"] * a["dim"], W), (a["kv_heads"] * a["vdim"], W)
            out[q + "sink"], out[q + "g"], out[q + "o"] = (a["heads"],), (a["heads"] * a["vdim"], W), (W, a["heads"] * a["vdim"])
            q = p + "mix.right."
            nk, nv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"] = (nk, W), (nk, W), (nv, W)
            out[q + "q.conv"], out[q + "k.conv"], out[q + "v.conv"] = (nk, r["conv"]), (nk, r["conv"]), (nv, r["conv"])
            out[q + "b"], out[q + "a"], out[q + "A_log"], out[q + "dt_bias"] = (r["heads"], W), (r["heads"], W), (r["heads"],), (r["heads"],)
            out[q + "norm"], out[q + "g"], out[q + "o"] = (r["vdim"],), (nv, W), (W, nv)
        else:
            q = p + "mix."
            nk, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "g"], out[q + "o"] = (nk, W), (nk, W), (nv, W), (nv, W), (W, nv)
            out[q + "norm"] = (nv,)
            out[q + "i"], out[q + "f"], out[q + "i.b"], out[q + "f.b"] = (m["heads"], W), (m["heads"], W), (m["heads"],), (m["heads"],)
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            out[p + "mlp.up"], out[p + "mlp.down"], out[p + "mlp.act"] = (F, W), (W, F), (4,)
    return out


def random_weights(cfg, seed):
    """float32 torch tensors that bfloat16 holds exactly.  Matrices ~ N(0, 1/fan_in) (the embedding N(0, 1)); the small tensors are
    spread so that every mechanism matters: sinks that weigh as much as a key, decays from nearly 1 to well below, gates on both
    sides of their caps, streams that mix with weights of either sign."""
    g = torch.Generator().manual_seed(seed)
    S = cfg["streams"]
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = n()
        elif "norm" in last:
            t = n(0.2, 1.0)
        elif last == "conv":
            t = n(0.4, 0.3)
        elif last == "sink":
            t = n(1.5, 0.5)
        elif last == "A_log":
            t = n(1.0, -1.0)
        elif last == "dt_bias":
            t = n(1.0)
        elif name.endswith("i.b"):
            t = n(2.0)
        elif name.endswith("f.b"):
            t = n(2.0, 3.0)
        elif last == "act":
            t = n(0.5, 0.5)
        elif last == "in" and ".hc" in name:
            t = n(0.3, 1.0 / S)
        elif last == "out" and ".hc" in name:
            t = n(0.3, 1.0)
        elif last == "mix" and ".hc" in name:
            t = torch.eye(S) + torch.randn(shape, generator=g) * 0.2
        elif last in ("i", "f"):
            t = n(3.0 / shape[-1] ** 0.5)                   # gate pre-activations of a few units: into the cap's curve
        else:
            t = n(1.0 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16).float()
    return out


def as_numpy(weights):
    return {k: v.double().numpy() for k, v in weights.items()}
