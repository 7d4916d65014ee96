"""The Desalorn design in the engine against the plain implementation (tests/plain/desalorn_plain.py): every mechanism alone,
then whole models under every way of cutting the work.  Needs a B200; float32 (true 32-bit) and bfloat16."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from desalorn_cases import as_numpy, attention, latent, layer, make_config, model, moe, random_weights, retention
from helpers import TOL, random_tokens, rel_l2, rows_close, write_folder
from plain import desalorn_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = ["float32", "bfloat16"]
WIDTH = 40


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def make_ctx(entries, starts, dtype, options=None):
    from titan_b200 import kernels as K
    from titan_b200.engine.batch import StepContext, StepLayout
    lay = StepLayout(entries, starts, "cuda")
    return StepContext(lay, K.current_stream(), dtype, torch.device("cuda"), dict(options or {}), {})


def ctx_of(T, dtype, options=None):
    from titan_b200.engine.batch import StepEntry
    return make_ctx([StepEntry(0, [0] * T, [])], [0], DT[dtype], options)


def bind(part, weights, dtype, prefix=""):
    from titan_b200.weights import held_dtype
    specs = {w.name: w for w in part.weight_specs(prefix)}
    part.bind(lambda rel: weights[prefix + rel].to("cuda", held_dtype(specs[prefix + rel].role, dtype)).contiguous())


def weights_for(part, seed, prefix=""):
    """bfloat16-representable random tensors for a part's declaration: matrices ~ N(0, 1/fan_in), vectors around their means."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for w in part.weight_specs(prefix):
        t = torch.randn(w.shape, generator=g)
        if w.role == "vector":
            mean = 1.0 if w.init[0] == "one_plus_normal" else (w.init[2] if w.init[0] == "normal_around" else 0.0)
            t = t * 0.3 + mean
        else:
            t = t / (w.shape[-1] ** 0.5)
        out[w.name] = t.to(torch.bfloat16).float()
    return out


def plain_weights(w, prefix):
    return {k[len(prefix):]: v.double().numpy() for k, v in w.items() if k.startswith(prefix)}


def inputs(lens, seed, width=WIDTH):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lens]


def drive(run_step, cache, xs, dtype, first_sizes):
    """Feed the sequences ``xs`` (rows of inputs) through ``run_step(h, ctx) -> out``, each on a slot of its own: first in
    portions of the given sizes (one list per step, a size per sequence), then token by token.  Returns each sequence's rows."""
    from titan_b200.engine.batch import StepEntry
    lens = [x.shape[0] for x in xs]
    slots = [cache.alloc_slot() for _ in xs]
    at, got = [0] * len(xs), [[] for _ in xs]
    plan = [list(s) for s in first_sizes]
    while any(a < n for a, n in zip(at, lens)):
        sizes = plan.pop(0) if plan else [1] * len(xs)
        live = [i for i in range(len(xs)) if at[i] < lens[i] and sizes[i] > 0]
        take = {i: min(sizes[i], lens[i] - at[i]) for i in live}
        cache.reserve({slots[i]: at[i] + take[i] for i in live})
        ctx = make_ctx([StepEntry(slots[i], [0] * take[i], []) for i in live], [at[i] for i in live], DT[dtype])
        h = torch.cat([xs[i][at[i]:at[i] + take[i]] for i in live]).to(DT[dtype]).cuda()
        out = run_step(h, ctx)
        for late in ctx.after_blocks:
            late()
        o = 0
        for i in live:
            got[i].append(out[o:o + take[i]].float().cpu())
            o += take[i]
            at[i] += take[i]
            cache.commit(slots[i], at[i])
    for s in slots:
        cache.free_slot(s)
    return [torch.cat(g) for g in got]


def mixer_step(mixer, cache):
    def step(h, ctx):
        out = torch.zeros(h.shape[0], WIDTH, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        return out
    return step


def t64(a):
    return torch.from_numpy(np.asarray(a)).float()


# --------------------------------------------------------------------------- #
# mechanisms alone
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("H,groups,T", [(48, 3, 9), (40, 1, 5), (192, 6, 70), (56, 7, 3), (1000, 4, 4), (2048, 8, 300), (36, 36, 2)])
def test_norm_in_groups_alone_and_behind_the_residual_sum(H, groups, T):
    """Every run of a row by its own root mean square, one weight over the row; the same behind x += m * y, with the sum's
    buffer left zeroed; and the row gather of the final norm."""
    from titan_b200 import kernels as K
    g = torch.Generator().manual_seed(H + groups)
    x, y, w = torch.randn(T, H, generator=g) * 3, torch.randn(T, H, generator=g), torch.randn(H, generator=g)
    x[:, : H // groups] *= 20                                     # one loud run: a norm over the whole row would flatten the others
    want = t64(P.group_norm(x.double().numpy(), w.double().numpy(), groups, 1e-5))
    assert groups == 1 or rel_l2(t64(P.group_norm(x.double().numpy(), w.double().numpy(), 1, 1e-5)), want) > 0.3
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    for dtype in BOTH:
        h = torch.empty(T, H, dtype=DT[dtype], device="cuda")
        K.group_rmsnorm(x.cuda(), w.cuda(), h, groups, 1e-5, K.current_stream())
        rows_close(h, want, dtype, "norm in groups")
        picked = torch.empty(2, H, dtype=DT[dtype], device="cuda")
        K.group_rmsnorm(x.cuda(), w.cuda(), picked, groups, 1e-5, K.current_stream(), rows)
        rows_close(picked, want[[T - 1, 0]], dtype, "gathered rows")
        x_d, y_d = x.cuda().clone(), y.cuda().clone()
        K.residual_group_norm(y_d, 0.3, x_d, K.current_stream(), norm_w=w.cuda(), groups=groups, eps=1e-5, h=h)
        new = x.double() + 0.3 * y.double()
        rows_close(x_d, new.float(), "float32", "residual sum")
        rows_close(h, t64(P.group_norm(new.numpy(), w.double().numpy(), groups, 1e-5)), dtype, "norm of the new rows")
        assert float(y_d.abs().max()) == 0.0
    x_d, y_d = x.cuda().clone(), y.cuda().clone()
    K.residual_group_norm(y_d, -1.5, x_d, K.current_stream())
    rows_close(x_d, (x.double() - 1.5 * y.double()).float(), "float32", "the sum alone")
    assert float(y_d.abs().max()) == 0.0


def attention_spec(H, G, dim, vdim, scale, cap, rows, far, eps=1e-5, window=None):
    from titan_b200.config import MixerSpec, PositionSpec
    extra = [("value_dim", vdim), ("bias", True), ("whole_norm", ("q.norm", "k.norm", eps)), ("rel_bias", ("rel", rows, float(far))),
             ("head_mix", "talk"), ("head_gate", "g")]
    if cap is not None:
        extra.append(("softcap", cap))
    return MixerSpec("attention", WIDTH, H, G, dim, window=window, softmax_scale=scale, prefix="a.", position=PositionSpec("none"),
                     names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")), extra=tuple(extra))


def attention_weights(mixer, seed, H):
    w = weights_for(mixer, seed)
    g = torch.Generator().manual_seed(seed + 1)
    w["a.talk"] = (torch.eye(H) + torch.randn(H, H, generator=g) * 0.4).to(torch.bfloat16).float()      # a blend well away from the identity
    w["a.rel"] = (torch.randn(w["a.rel"].shape, generator=g) * 1.5).to(torch.bfloat16).float()
    w["a.g"] = w["a.g"] * 3
    return w


ATTENTION_SIZES = [
    (4, 2, 16, 16, 5.0, 8, 40),             # a cap that bends the scores; a table of eight rows
    (3, 1, 12, 20, 30.0, 5, 17.0),          # unequal widths, no multiples of 8, an odd number of rows
    (6, 6, 8, 8, 2.0, 12, 300),             # as many kv heads as heads; a table that reaches further than the prompts
    (1, 1, 32, 32, None, 2, 3),             # one head (the blend is one number); no cap; a table of two rows
    (8, 2, 64, 64, 50.0, 32, 128),          # heads of 64
    (2, 1, 128, 64, 20.0, 16, 1000),        # keys of 128, values of 64
    (32, 4, 8, 16, 10.0, 6, 50),            # as many heads as the kernel's block has warps
]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dim,vdim,cap,rows,far", ATTENTION_SIZES)
def test_attention_alone(dtype, H, G, dim, vdim, cap, rows, far):
    """Biases, the norms over all queries and all keys, the cap, the bias by distance, the blend of the heads' scores, the gate
    a head: whole prompts of two unequal sequences, portions, portions of two tokens, then single tokens across a page's
    border; then the slots again (freed pages overwritten)."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(attention_spec(H, G, dim, vdim, 0.4, cap, rows, far))
    w = attention_weights(mixer, 3, H)
    bind(mixer, w, DT[dtype])
    m = attention(H, G, dim, vdim, 0.4, cap, rows, far)
    lens = [150, 71]
    xs = inputs(lens, 5)
    want = [t64(P.softmax_attention(x.numpy(), plain_weights(w, "a."), "", m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([lens], [[60, 33], [50, 2], [2, 2], [2, 30]], [[1, 1]]):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dim,vdim,cap,rows,far", [ATTENTION_SIZES[0], ATTENTION_SIZES[1], ATTENTION_SIZES[4], ATTENTION_SIZES[5]])
def test_attention_on_the_one_query_prompt_kernel(dtype, H, G, dim, vdim, cap, rows, far):
    """The prompt kernel that every size falls back to (a block a query, rows read from the cache and the step as they lie),
    against the plain result: whole prompts and portions."""
    from titan_b200 import kernels as K
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(attention_spec(H, G, dim, vdim, 0.4, cap, rows, far))
    w = attention_weights(mixer, 3, H)
    bind(mixer, w, DT[dtype])
    m = attention(H, G, dim, vdim, 0.4, cap, rows, far)
    lens = [150, 71]
    xs = inputs(lens, 5)
    want = [t64(P.softmax_attention(x.numpy(), plain_weights(w, "a."), "", m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    K.set_attn_mixed_tile(False)
    try:
        for sizes in ([lens], [[60, 33], [50, 2], [2, 2]]):
            got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
            for i in range(2):
                rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)
    finally:
        K.set_attn_mixed_tile(True)


LAST = 229


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim", [16, 64])
@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 127, 128, 191, 192, LAST - 1])
def test_one_far_key_decides_across_page_borders(dtype, dim, far):
    """The key matrix is minus the query matrix and the last token's input row is minus that of position ``far``: that one key,
    among hundreds, takes nearly all the softmax's weight of both heads.  Losing it (a page's last row, the next page's first,
    the sequence's first tokens) changes the output altogether.  Through a whole prompt, as a single token, in portions, and
    decoded from the key on."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H = G = 2
    mixer = MIXERS.build(attention_spec(H, G, dim, dim, 40.0 / dim, 1000.0, 8, 40))     # the key's own score is 40, the others' spread 40 / sqrt(dim)
    w = weights_for(mixer, 7)
    w["a.k"] = -w["a.q"]
    for name in ("a.q.b", "a.k.b", "a.v.b", "a.o.b"):
        w[name] = w[name] * 0.0
    w["a.q.norm"], w["a.k.norm"] = torch.ones_like(w["a.q.norm"]), torch.ones_like(w["a.k.norm"])
    w["a.talk"] = torch.tensor([[1.0, 0.25], [0.25, 1.0]])
    w["a.g"] = w["a.g"] * 0.0                                      # a gate of one half everywhere
    bind(mixer, w, DT[dtype])
    m = attention(H, G, dim, dim, 40.0 / dim, 1000.0, 8, 40)
    n = LAST + 1
    x = inputs([n], 8)[0]
    x[-1] = -x[far]
    W = plain_weights(w, "a.")
    want = t64(P.softmax_attention(x.numpy(), W, "", m, 1e-5))
    only_far = t64(0.5 * (x[far].numpy() @ W["v"].T) @ W["o"].T)              # what the heads return if that key has all the weight
    assert rel_l2(only_far, want[-1]) < 0.2, "the test's weights do not single the key out"
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    step = mixer_step(mixer, cache)
    whole = drive(step, cache, [x], dtype, [[n]])[0]
    rows_close(whole[-1:], want[-1:], dtype, "in a prompt", row_factor=6.0)
    decoded = drive(step, cache, [x], dtype, [[n - 1]])[0]
    rows_close(decoded[-1:], want[-1:], dtype, "decoded alone", row_factor=6.0)
    pieces = drive(step, cache, [x], dtype, [[far + 1], [max(1, n - far - 3)], [2]])[0]
    rows_close(pieces[-1:], want[-1:], dtype, "in portions", row_factor=6.0)
    long_tail = drive(step, cache, [x], dtype, [[max(1, far)]])[0]
    rows_close(long_tail[-1:], want[-1:], dtype, "decoded from the key on", row_factor=6.0)


@pytest.mark.parametrize("rows,far", [(8, 40), (5, 17.0), (12, 100)])
def test_one_row_of_the_distance_table_decides(rows, far):
    """Queries and keys are zero, so every score is its bias by distance; one row of the table is far above the others, so the
    last query returns the mean value over exactly the keys whose distance falls into that row.  A table read one distance
    off at a row's first or last distance moves a key in or out of that mean.  Every row in turn, the last one (all distances
    from ``far`` on) included; in a prompt and decoded (float32)."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H = 2
    mixer = MIXERS.build(attention_spec(H, 1, 16, 16, 1.0, 10.0, rows, far))
    w = weights_for(mixer, 11)
    for name in ("a.q", "a.k", "a.q.b", "a.k.b", "a.g", "a.o.b"):
        w[name] = w[name] * 0.0
    w["a.talk"] = torch.eye(H)
    n = int(2.5 * far)
    x = inputs([n], 12)[0]
    m = attention(H, 1, 16, 16, 1.0, 10.0, rows, far)
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, torch.float32, "cuda", mark_freed=True)      # one cache for the mixer's life: it keeps its view of it
    for loud in range(rows):
        w["a.rel"] = torch.zeros(rows, H)
        w["a.rel"][loud] = 40.0
        bind(mixer, w, torch.float32)
        W = plain_weights(w, "a.")
        want = t64(P.softmax_attention(x.numpy(), W, "", m, 1e-5))
        inside = [j for j in range(n) if P.distance_bucket(n - 1 - j, rows, far) == loud]
        assert inside, "no key of the prompt reads this row"
        mean_v = 0.5 * (x[inside].numpy() @ W["v"].T + W["v.b"]).mean(axis=0)
        assert rel_l2(t64(np.tile(mean_v, H) @ W["o"].T), want[-1]) < 1e-3
        for sizes in ([[n]], [[n - 3]]):
            got = drive(mixer_step(mixer, cache), cache, [x], "float32", sizes)[0]
            rows_close(got, want, "float32", f"row {loud}, portions {sizes}", row_factor=6.0)


def retention_spec(H, dk, dv, decay, rot, base=10000.0, eps=1e-5):
    from titan_b200.config import MixerSpec, PositionSpec
    return MixerSpec("retention", WIDTH, H, head_dim=dk, prefix="r.", position=PositionSpec("rope", rot, base, "half"),
                     extra=(("value_dim", dv), ("decay", tuple(decay)), ("norm_eps", eps)))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dk,dv,rot", [(3, 8, 12, 4), (1, 40, 20, 40), (2, 64, 128, 32), (5, 4, 36, 2), (1, 130, 8, 64), (4, 128, 128, 128), (1, 256, 64, 16),
                                          (2, 64, 64, 64), (6, 16, 16, 8)])
def test_retention_alone(dtype, H, dk, dv, rot):
    """Decays from one half to nearly one (and one itself): whole prompts, portions down to two tokens, single tokens, then
    the slots given back and used again: outputs, and a state that starts from zero."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    decay = [(0.5, 0.9, 0.97, 0.9990234375, 1.0, 0.75)[i % 6] for i in range(H)]
    mixer = MIXERS.build(retention_spec(H, dk, dv, decay, rot, base=300.0))
    w = weights_for(mixer, 9)
    bind(mixer, w, DT[dtype])
    m = retention(H, dk, dv, decay, rot, base=300.0)
    lens = [90, 37]
    xs = inputs(lens, 11)
    want = [t64(P.retention(x.numpy(), plain_weights(w, "r."), "", m, 1e-5)[0]) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([[90, 37]], [[40, 20], [2, 2], [17, 1], [2, 0], [1, 2]], []):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


def test_retention_remembers_a_value_far_back():
    """A decay of nearly one and a loud token early on: 300 tokens later a query that matches its key (without rotation to
    speak of) reads its value out of the state and blends it with the last token's own; a state that lost the early write
    gives another direction.  float32; whole, decoded after the write, and in portions."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H, dk, dv = 1, 16, 16
    mixer = MIXERS.build(retention_spec(H, dk, dv, [0.9990234375], 2, base=1e6))
    w = weights_for(mixer, 21)
    half = WIDTH // 2
    w["r.q"][:, half:] = 0.0                                        # queries and keys read one half of the input row, values the other
    w["r.k"] = w["r.q"].clone()
    w["r.v"][:, :half] = 0.0
    bind(mixer, w, torch.float32)
    n = 300
    x = inputs([n], 22)[0] * 0.05
    x[3] = inputs([1], 23)[0][0] * 4
    x[-1, :half] = x[3, :half]                                      # the early token's key at the end, with a value of its own: the result blends both values
    x[-1, half:] = x[-1, half:] * 60
    m = retention(H, dk, dv, [0.9990234375], 2, base=1e6)
    W = plain_weights(w, "r.")
    want = t64(P.retention(x.numpy(), W, "", m, 1e-5)[0])
    quiet = x.clone()
    quiet[3] = quiet[4]
    assert rel_l2(t64(P.retention(quiet.numpy(), W, "", m, 1e-5)[0])[-1], want[-1]) > 0.3, "the early token does not reach the last position"
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, torch.float32, "cuda", mark_freed=True)
    for sizes in ([[n]], [[5]], [[64], [64], [2]]):
        got = drive(mixer_step(mixer, cache), cache, [x], "float32", sizes)[0]
        rows_close(got, want, "float32", f"portions {sizes}", row_factor=6.0)


def latent_spec(H, dn, rd, dv, r, qr, size, scale, base=10000.0, eps=1e-5):
    from titan_b200.config import MixerSpec, NormSpec, PositionSpec
    return MixerSpec("latent_attention", WIDTH, H, 1, dn, window=size, softmax_scale=scale, prefix="m.",
                     position=PositionSpec("rope", rd, base, "adjacent"),
                     extra=(("rot_dim", rd), ("value_dim", dv), ("kv_rank", r), ("latent_norm", NormSpec("rmsnorm", r, eps, "dkv.norm")),
                            ("q_rank", qr), ("q_norm", NormSpec("rmsnorm", qr, eps, "dq.norm"))))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dn,rd,dv,r,qr,size", [(2, 16, 8, 12, 20, 12, 20), (3, 12, 4, 20, 28, 9, 7), (2, 128, 64, 128, 64, 48, 64), (4, 32, 16, 32, 40, 24, 65),
                                                   (1, 8, 2, 8, 6, 5, 300)])
def test_latent_attention_with_queries_through_a_latent(dtype, H, dn, rd, dv, r, qr, size):
    """The query latent with its norm before the heads' queries; windows of a few keys, of a page, of a page and a row, and
    wider than the prompts: whole prompts, portions, single tokens over a ring that turns, slots used again."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(latent_spec(H, dn, rd, dv, r, qr, size, 0.3, base=500.0))
    w = weights_for(mixer, 31)
    bind(mixer, w, DT[dtype])
    m = latent(H, dn, rd, dv, r, qr, size, 0.3, base=500.0)
    lens = [150, 71]
    xs = inputs(lens, 32)
    want = [t64(P.latent_attention(x.numpy(), plain_weights(w, "m."), "", m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([lens], [[60, 33], [50, 2], [2, 2], [2, 30]], [[1, 1]]):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


SIZE = 72 + 9


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("far,seen", [(LAST - SIZE, False), (LAST - SIZE + 1, True), (LAST - SIZE + 2, True), (191, True), (192, True), (LAST - 1, True), (100, False)])
def test_a_loud_key_just_inside_and_just_outside_the_window(dtype, far, seen):
    """The input row at one position is replaced by another: if the position is the window's oldest key or a later one, the last
    query's plain result moves; one position further back it does not move at all.  The engine follows the plain result for
    both prompts (float32 is the sharp one of the two: an edge key carries about a hundredth of the weight), in a prompt, decoded
    alone, and decoded from the key on."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H, dn, rd, dv, r, qr = 2, 16, 8, 16, 24, 16
    mixer = MIXERS.build(latent_spec(H, dn, rd, dv, r, qr, SIZE, 0.3, base=1e6))
    w = weights_for(mixer, 41)
    bind(mixer, w, DT[dtype])
    m = latent(H, dn, rd, dv, r, qr, SIZE, 0.3, base=1e6)
    n = LAST + 1
    x = inputs([n], 42)[0]
    W = plain_weights(w, "m.")
    want = t64(P.latent_attention(x.numpy(), W, "", m, 1e-5))
    moved = x.clone()
    moved[far] = inputs([1], 43)[0][0]
    changed = rel_l2(torch.from_numpy(P.latent_attention(moved.numpy(), W, "", m, 1e-5))[-1], torch.from_numpy(P.latent_attention(x.numpy(), W, "", m, 1e-5))[-1]) > 1e-9
    assert changed == seen, "the plain result does not depend on the key as the window says"
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    step = mixer_step(mixer, cache)
    for xx in (x, moved):
        ref = t64(P.latent_attention(xx.numpy(), W, "", m, 1e-5))
        rows_close(drive(step, cache, [xx], dtype, [[n]])[0][-1:], ref[-1:], dtype, "in a prompt", row_factor=6.0)
        rows_close(drive(step, cache, [xx], dtype, [[n - 1]])[0][-1:], ref[-1:], dtype, "decoded alone", row_factor=6.0)
        rows_close(drive(step, cache, [xx], dtype, [[max(1, far)]])[0][-1:], ref[-1:], dtype, "decoded from the key on", row_factor=6.0)


def test_router_on_hand_made_and_random_outputs():
    """The device's choice against the plain one: the two best of a group decide which groups are open, negative choice scores
    in an open group beat every closed one, the weights are the sigmoids themselves; then random rows at several shapes."""
    from titan_b200 import kernels as K
    logit = lambda p: math.log(p / (1 - p))
    cases = [([0.9, 0.1, 0.1, 0.6, 0.6, 0.2], [0.0] * 6, 2, 2, 1), ([0.9, 0.1, 0.1, 0.6, 0.6, 0.2], [0, 0, 0, -2.0, -2.0, -2.0], 2, 2, 1),
             ([0.9, 0.1, 0.1, 0.6, 0.6, 0.2], [-5.0, -5.0, -5.0, -2.0, -2.0, -2.0], 3, 2, 1)]
    for s, corr, top, groups, keep in cases:
        z = torch.tensor([[logit(p) for p in s]], dtype=torch.float32)
        ids, wts = torch.empty(1, top, dtype=torch.int32, device="cuda"), torch.empty(1, top, device="cuda")
        K.moe_route_scored(z.cuda(), top, torch.tensor(corr, dtype=torch.float32).cuda(), groups, keep, ids, wts, K.current_stream(), sigmoid=True, group_best=2, renorm=False)
        pi, pw = P.route(z.double().numpy(), np.array(corr), top, groups, keep)
        assert sorted(ids[0].tolist()) == sorted(pi[0].tolist())
        assert np.allclose(sorted(wts[0].tolist()), sorted(pw[0]), atol=1e-6)
    g = torch.Generator().manual_seed(5)
    for E, top, groups, keep, T in ((8, 2, 4, 2, 50), (6, 3, 1, 1, 20), (16, 4, 8, 3, 64), (9, 1, 3, 1, 33), (64, 6, 8, 4, 40), (4, 4, 2, 2, 7), (12, 2, 12, 5, 30)):
        z = torch.randn(T, E, generator=g) * 2
        corr = torch.randn(E, generator=g) * 0.5
        ids, wts = torch.empty(T, top, dtype=torch.int32, device="cuda"), torch.empty(T, top, device="cuda")
        K.moe_route_scored(z.cuda(), top, corr.cuda(), groups, keep, ids, wts, K.current_stream(), sigmoid=True, group_best=2, renorm=False)
        pi, pw = P.route(z.double().numpy(), corr.double().numpy(), top, groups, keep)
        ids, wts = ids.cpu().numpy(), wts.cpu().numpy()
        for t in range(T):
            assert sorted(ids[t].tolist()) == sorted(pi[t].tolist()), f"{E} experts, row {t}"
            assert np.allclose(sorted(wts[t]), sorted(pw[t]), atol=1e-6)


def moe_spec(E, top, F, groups, keep, shared):
    from titan_b200.config import FeedForwardSpec
    return FeedForwardSpec("moe", WIDTH, F, "silu", prefix="f.", extra=(("experts", E), ("top", top), ("routing", "sigmoid_all"), ("groups", groups),
                                                                         ("keep", keep), ("group_best", 2), ("renormalize", False), ("shared_size", shared),
                                                                         ("shared_gate", False)))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top,F,groups,keep,shared,T", [(8, 2, 24, 4, 2, 40, 5), (6, 3, 20, 1, 1, 0, 3), (8, 2, 32, 2, 1, 64, 300), (16, 4, 16, 8, 3, 16, 40),
                                                           (4, 1, 64, 2, 1, 128, 700)])
def test_mixture_on_every_product_path(dtype, E, top, F, groups, keep, shared, T):
    """A few pairs (a warp an output), many pairs on CUDA cores, and a bfloat16 prompt on tensor cores; with and without the
    shared expert, which carries no gate.  The router reads the rows as the engine's dtype holds them."""
    from titan_b200.parts import FEED_FORWARDS
    ff = FEED_FORWARDS.build(moe_spec(E, top, F, groups, keep, shared))
    w = weights_for(ff, 51)
    w["f.router"] = w["f.router"] * 4
    bind(ff, w, DT[dtype])
    x = inputs([T], 52)[0]
    out = torch.zeros(T, WIDTH, device="cuda")
    ff.forward(x.to(DT[dtype]).cuda(), ctx_of(T, dtype), out)
    f = moe(E, top, F, groups, keep, shared or None)
    want = t64(P.mixture(x.numpy(), plain_weights(w, "f."), "", f))
    rows_close(out, want, dtype, "mixture", row_factor=6.0)


# --------------------------------------------------------------------------- #
# whole models
# --------------------------------------------------------------------------- #
def close(got, want, dtype, what="", slack=1.0):
    """float32: the whole tensor and every row.  bfloat16: a near-tie in a router sends the rounded row to another expert than
    the float64 evaluation takes, which moves that row by more than rounding does; so the rows' median is held to the bound,
    and nine rows in ten to six times it."""
    if dtype == "float32":
        return rows_close(got, want, dtype, what, row_factor=6.0, slack=slack)
    g, w = got.double().reshape(-1, got.shape[-1]).cpu(), want.double().reshape(-1, want.shape[-1])
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} instead of {tuple(w.shape)}"
    rows = (g - w).norm(dim=1) / w.norm(dim=1).clamp_min(1e-30)
    bound = slack * TOL[dtype]
    assert float(rows.median()) < bound, f"{what}: median row error {float(rows.median()):.3e} over {bound:.0e}"
    off = float((rows > 6 * bound).double().mean())
    assert off <= 0.1 and float(rows.max()) < 1.0, f"{what}: {off:.2f} of the rows beyond {6 * bound:.2f}, the worst {float(rows.max()):.2f}"


class World:
    """One small model: weights, plain logits of its requests, engines by dtype and options."""

    def __init__(self, name, seed, lengths):
        self.cfg = make_config(name)
        self.weights = random_weights(self.cfg, seed)
        self.numpy = as_numpy(self.weights)
        self.requests = [random_tokens(n, self.cfg["vocab"], 50 + i) for i, n in enumerate(lengths)]
        self._plain, self._engines = {}, {}

    def plain(self, tokens, layers=False):
        key = tuple(tokens)
        if key not in self._plain:
            after = []
            logits = P.forward(self.cfg, self.numpy, list(tokens), after_layer=lambda i, x: after.append(x.copy()))
            self._plain[key] = (t64(logits), t64(np.stack(after)))
        return self._plain[key][1 if layers else 0]

    def engine(self, dtype, **kw):
        from titan_b200 import Engine
        from titan_b200.config import config_from_dict
        key = (dtype, tuple(sorted(kw.items())))
        if key not in self._engines:
            opts = {"max_tokens": 1536, "max_slots": 6, "mark_freed_pages": True} | kw
            self._engines[key] = Engine.from_tensors(config_from_dict(self.cfg), self.weights, dtype=dtype, **opts)
        return self._engines[key]


LENGTHS = {"mix": [150, 9, 66, 1], "odd": [140, 64, 3, 129], "wide": [70, 200, 17, 2]}
_worlds = {}


def world(name):
    if name not in _worlds:
        _worlds[name] = World(name, {"mix": 1, "odd": 2, "wide": 3}[name], LENGTHS[name])
    return _worlds[name]


MODELS = [(n, d) for n in ("mix", "odd", "wide") for d in BOTH]


def run_in_pieces(e, tokens, pieces):
    """Feed ``tokens`` to one fresh slot in steps of the given sizes (the rest one by one); logits at every position."""
    from titan_b200 import StepEntry
    s, at, got = e.alloc_slot(), 0, []
    sizes = list(pieces)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        got.append(e.step([StepEntry(s, tokens[at:at + n], list(range(n)))]))
        at += n
    e.free_slot(s)
    return torch.cat(got).float().cpu()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_whole_prompts_alone(name, dtype):
    wd = world(name)
    e = wd.engine(dtype)
    got = [run_in_pieces(e, toks, [len(toks)]) for toks in wd.requests]
    want = [wd.plain(toks) for toks in wd.requests]
    if dtype == "float32":
        for toks, g, w in zip(wd.requests, got, want):
            close(g, w, dtype, f"{name}: prompt of {len(toks)}")
    close(torch.cat(got), torch.cat(want), dtype, f"{name}: all prompts")
    e.check_kernels()
    e.cache.check()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_the_residual_stream_after_every_layer(name, dtype):
    """Layer by layer on the longest request: the first layer that differs is named."""
    from titan_b200 import StepEntry
    wd = world(name)
    e = wd.engine(dtype)
    toks = max(wd.requests, key=len)
    seen = []
    e.layer_observer = lambda run, x: seen.append(x.clone())
    try:
        s = e.alloc_slot()
        e.step([StepEntry(s, toks, [0])])
        e.free_slot(s)
    finally:
        e.layer_observer = None
    want = wd.plain(toks, layers=True)
    assert len(seen) == len(want)
    for i, got in enumerate(seen):
        close(got, want[i], dtype, f"{name}: after layer {i}")


@pytest.mark.parametrize("name,dtype", MODELS)
def test_prompt_then_token_by_token_and_portions_down_to_two(name, dtype):
    wd = world(name)
    e = wd.engine(dtype)
    toks = wd.requests[0]
    want = wd.plain(toks)
    close(run_in_pieces(e, toks, [len(toks) - 40]), want, dtype, f"{name}: prompt then 40 single tokens")
    close(run_in_pieces(e, toks, [1]), want, dtype, f"{name}: token by token from the first")
    close(run_in_pieces(e, toks, [64, 2, 2, 31, 1, 2, 40]), want, dtype, f"{name}: portions")
    close(run_in_pieces(e, toks, [2] * (len(toks) // 2)), want, dtype, f"{name}: portions of two")
    close(run_in_pieces(e, toks, [3, 61, 64, 1, 1, 9]), want, dtype, f"{name}: portions that end at a page's border")
    e.check_kernels()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_a_batch_of_unequal_requests_against_each_alone_and_slots_used_again(name, dtype):
    """All requests as one batch of prompts, decoded together while the shorter ones leave; then the same again in the
    freed slots and pages (which were overwritten when they were freed), in the other order."""
    from titan_b200 import StepEntry
    wd = world(name)
    e = wd.engine(dtype)
    reqs = wd.requests
    tail = 6
    alone = [run_in_pieces(e, r, [max(1, len(r) - tail)]) for r in reqs]
    for turn in range(2):
        order = list(range(len(reqs))) if turn == 0 else list(reversed(range(len(reqs))))
        heads = {i: max(1, len(reqs[i]) - tail) for i in order}
        slots = {i: e.alloc_slot() for i in order}
        got = {i: [] for i in order}
        out = e.step([StepEntry(slots[i], reqs[i][:heads[i]], list(range(heads[i]))) for i in order])
        o = 0
        for i in order:
            got[i].append(out[o:o + heads[i]].float().cpu())
            o += heads[i]
        at = dict(heads)
        for i in order:
            if at[i] == len(reqs[i]):
                e.free_slot(slots[i])
        while any(at[i] < len(reqs[i]) for i in order):
            live = [i for i in order if at[i] < len(reqs[i])]
            out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1].float().cpu())
                at[i] += 1
                if at[i] == len(reqs[i]):
                    e.free_slot(slots[i])
        for i in order:
            if dtype == "float32":
                close(torch.cat(got[i]), wd.plain(reqs[i]), dtype, f"{name}: request {i} in a batch, turn {turn}")
                close(torch.cat(got[i]), alone[i], dtype, f"{name}: request {i} in a batch against itself alone, turn {turn}")
        close(torch.cat([torch.cat(got[i]) for i in order]), torch.cat([alone[i] for i in order]), dtype, f"{name}: a batch against each alone, turn {turn}")
        close(torch.cat([torch.cat(got[i]) for i in order]), torch.cat([wd.plain(reqs[i]) for i in order]), dtype, f"{name}: all requests of a batch, turn {turn}")
        e.cache.check()
    e.check_kernels()


@pytest.mark.parametrize("dtype", BOTH)
def test_a_loud_first_token_reaches_far_through_the_state_and_the_first_key(dtype):
    """The first token's embedding row is unlike the others': every later position feels it, through the retention's state and
    the attention's first key, in a prompt and when decoded token by token."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg = make_config("mix")
    w = random_weights(cfg, 5)
    toks = random_tokens(200, cfg["vocab"], 77)
    toks[0] = 3
    assert 3 not in toks[1:]
    want = t64(P.forward(cfg, as_numpy(w), toks))
    other = list(toks)
    other[0] = 4
    assert rel_l2(t64(P.forward(cfg, as_numpy(w), other))[-1], want[-1]) > 20 * TOL["float32"], "the first token does not reach the last position"
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=1024, max_slots=2)
    close(run_in_pieces(e, toks, [len(toks)]), want, dtype, "whole")
    close(run_in_pieces(e, toks, [100]), want, dtype, "decoded from 100")
    close(run_in_pieces(e, toks, [1, 2]), want, dtype, "decoded from the first tokens on")


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding(dtype):
    """A short prompt, then 400 single tokens over several pages and many turns of the window's ring."""
    wd = world("odd")
    toks = random_tokens(420, wd.cfg["vocab"], 123)
    e = wd.engine(dtype)
    close(run_in_pieces(e, toks, [20]), wd.plain(toks), dtype, "long decoding")
    e.check_kernels()


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_greedy_generation_through_the_scheduler(name):
    """Engine.generate (scheduler, sampler, captured decode steps) against greedy decoding with the plain implementation,
    in float32, where the argmax is decided."""
    wd = world(name)
    e = wd.engine("float32", max_batch=3)
    prompts = [r[:12] for r in wd.requests if len(r) >= 12] + [wd.requests[-1]]
    steps = 10
    from titan_b200.sampling import SamplerParams
    results = e.generate(prompts, max_tokens=steps, params=SamplerParams.greedy(), stop_tokens=())
    for p, r in zip(prompts, results):
        seq = list(p)
        for _ in range(steps):
            logits = t64(P.forward(wd.cfg, wd.numpy, seq)[-1])
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break                                           # a near tie: float32 and float64 may differ from here
            seq.append(int(logits.argmax()))
        n = len(seq) - len(p)
        assert n > 0 and list(r.tokens)[:n] == seq[len(p):], f"{name}: generation differs"
    e.cache.check()


def test_captured_decode_steps_give_the_eager_steps_logits():
    """bfloat16, as served: a batch decoded through advance() (eager first, then replayed graphs) against step()."""
    from titan_b200 import StepEntry
    from titan_b200.sampling import SamplerParams
    wd = world("wide")
    e = wd.engine("bfloat16")
    prompts = [wd.requests[0][:40], wd.requests[1][:90]]
    slots, toks = e.start(prompts, [SamplerParams.greedy()] * 2, [1, 2])
    seqs = [list(p) + [t] for p, t in zip(prompts, toks)]
    for _ in range(6):
        toks = e.advance(slots, [s[-1] for s in seqs])
        for s, t in zip(seqs, toks):
            s.append(t)
    captured = e.last_logits.float().cpu()
    for s in slots:
        e.finish(s)
    assert e.graph_launches > 0, "no decode step was replayed from a graph"
    fresh = [e.alloc_slot(), e.alloc_slot()]
    out = e.step([StepEntry(fresh[i], seqs[i][:-1], [len(seqs[i]) - 2]) for i in range(2)]).float().cpu()
    for s in fresh:
        e.free_slot(s)
    close(captured, out, "bfloat16", "captured against whole prompts")
    e.check_kernels()


def test_trace_runner_as_a_subprocess(tmp_path):
    """bin/trace_run on a model folder whose description leaves the tables' rows to the tensors: a batch of two prompts, single
    tokens after them while one request leaves, then many short requests at once, in slots and pages that were used before."""
    cfg = make_config("odd")
    weights = random_weights(cfg, 9)
    stripped = json.loads(json.dumps(cfg))
    for l in stripped["layers"]:
        l["mixer"].pop("bias_rows", None)
    folder = write_folder(str(tmp_path / "model"), stripped, {k: v.to(torch.bfloat16) for k, v in weights.items()})
    a, b = random_tokens(70, cfg["vocab"], 1), random_tokens(21, cfg["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:20], "want": [19]}], "end": []}]
    for i in range(10):
        es = [{"id": "a", "tokens": [a[60 + i]], "want": [0]}]
        if i == 0:
            es.append({"id": "b", "tokens": [b[20]], "want": [0]})
        steps.append({"step": i + 1, "entries": es, "end": ["b"] if i == 0 else (["a"] if i == 9 else [])})
    many = [random_tokens(3, cfg["vocab"], 30 + i) for i in range(20)]
    steps.append({"step": 11, "entries": [{"id": f"m{i}", "tokens": m[:2], "want": []} for i, m in enumerate(many)], "end": []})
    steps.append({"step": 12, "entries": [{"id": f"m{i}", "tokens": m[2:], "want": [0]} for i, m in enumerate(many)], "end": [f"m{i}" for i in range(20)]})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "192"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(13)]
    W = as_numpy(weights)
    pa, pb = t64(P.forward(cfg, W, a)), t64(P.forward(cfg, W, b))
    V = cfg["vocab"]
    read = lambda name: torch.from_numpy(np.fromfile(out / name, dtype="<f4").reshape(-1, V))
    rows_close(read("0.f32"), torch.stack([pa[0], pa[59], pb[19]]), "float32", "step 0")
    rows_close(read("1.f32"), torch.stack([pa[60], pb[20]]), "float32", "step 1")
    rows_close(read("10.f32"), pa[69:70], "float32", "step 10")
    rows_close(read("12.f32"), torch.stack([t64(P.forward(cfg, W, m))[2] for m in many]), "float32", "twenty short requests")


def test_command_line_with_random_weights(tmp_path):
    """bin/titan_b200 run --random: the design through the command line, the scheduler and the sampler, from a description alone."""
    path = tmp_path / "config.json"
    path.write_text(json.dumps(make_config("mix")))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "titan_b200"), "run", "--random", str(path), "--weights-seed", "3", "--prompt-ids", "5,6,7,8",
                        "--prompt-ids", "9,10", "--max-tokens", "12", "--temp", "0", "--dtype", "bfloat16", "--kv-capacity", "512"],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.strip(), "nothing was generated"


def drawn_config(seed):
    """A configuration drawn at random: sizes, head counts, layer order, windows, groups, constants; odd sizes and ones included."""
    import random
    r = random.Random(seed)
    groups = r.choice([1, 2, 3, 4, 8])
    width = groups * r.choice([8, 12, 17, 24, 34])
    layers = []
    for i in range(r.randint(2, 5)):
        kind = r.choice(["attention", "retention", "latent_attention"])
        if kind == "attention":
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 4])
            dim = r.choice([6, 8, 12, 16, 20, 32, 40, 64])
            rows = r.choice([1, 2, 3, 8, 9, 16, 32])
            far = r.choice([rows // 2 + 1, rows // 2 + 0.5, 20, 120, 1000.0])
            m = attention(heads, kv, dim, r.choice([dim, dim, 8, 24, 16]), r.choice([0.1, 0.3, dim ** -0.5]), r.choice([None, 1.0, 8.0, 50.0]), rows, far)
            if m["softcap"] is None:
                m.pop("softcap")
        elif kind == "retention":
            heads, dim = r.choice([1, 2, 3, 5]), r.choice([4, 8, 12, 24, 48, 72])
            m = retention(heads, dim, r.choice([4, 8, 20, 33, 64]), [r.choice([0.5, 0.9, 0.97, 0.9990234375, 1.0]) for _ in range(heads)],
                          r.choice([d for d in (2, 4, 8, 12, 24, 48) if d <= dim]), base=r.choice([100.0, 1e4, 1e6]))
        else:
            rd = r.choice([2, 4, 8, 16])
            m = latent(r.choice([1, 2, 3, 4]), r.choice([4, 8, 12, 16, 32]), rd, r.choice([4, 8, 20, 32]), r.choice([6, 16, 28, 40]), r.choice([5, 8, 24]),
                       r.choice([1, 2, 5, 31, 64, 65, 100, 500]), r.choice([0.1, 0.3]), base=r.choice([100.0, 1e4, 5e5]))
        f = None
        if r.random() < 0.75:
            count = r.choice([1, 2, 3, 4])
            per = r.choice([1, 2, 3, 4])
            keep = r.randint(1, count)
            f = moe(count * per, r.randint(1, keep * per), r.choice([8, 16, 33, 64]), count, keep, shared=r.choice([None, 8, 40]))
        layers.append(layer(kind, m, f))
    return model(layers, width=width, vocab=r.choice([50, 97, 300]), eps=r.choice([1e-6, 1e-5, 1e-4]), groups=groups,
                 mult=r.choice([0.2, 0.5, 1.0]), embed_scale=r.choice([1.0, 2.0, 12.0]))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("seed", range(int(os.environ.get("DESALORN_DRAWN", "12"))))
def test_configurations_drawn_at_random(seed, dtype):
    """A prompt whole, then a second request as a prompt with single tokens after it, in a batch with a third.  float32 is the
    sharp test (a wrong branch costs tens of percent, summation order 1e-6); bfloat16 by the rows' median and nine in ten."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg = drawn_config(seed)
    w = random_weights(cfg, 100 + seed)
    W = as_numpy(w)
    a, b, c = (random_tokens(n, cfg["vocab"], 7 * seed + n) for n in (75, 130, 9))
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=1024, max_slots=4, mark_freed_pages=True)
    whole = run_in_pieces(e, a, [len(a)])
    sb, sc = e.alloc_slot(), e.alloc_slot()
    got_b = [e.step([StepEntry(sb, b[:66], list(range(66))), StepEntry(sc, c[:8], [])])[:66]]
    got_b.append(e.step([StepEntry(sb, [b[66]], [0]), StepEntry(sc, [c[8]], [])])[:1])
    e.free_slot(sc)
    for t in b[67:]:
        got_b.append(e.step([StepEntry(sb, [t], [0])]))
    e.free_slot(sb)
    e.check_kernels()
    e.cache.check()
    slack = 1.0 if dtype == "float32" else 2.0
    close(whole, t64(P.forward(cfg, W, a)), dtype, f"seed {seed}: whole", slack=slack)
    close(torch.cat(got_b).float().cpu(), t64(P.forward(cfg, W, b)), dtype, f"seed {seed}: prompt in a batch, then single tokens", slack=slack)
