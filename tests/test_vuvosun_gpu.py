"""The Vuvosun design in the engine against the plain implementation (tests/plain/vuvosun_plain.py): every mechanism alone,
then whole models under every way of cutting the work.  Needs a B200; float32 (true 32-bit) and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL, random_tokens, rel_l2, rows_close, write_folder
from plain import vuvosun_plain as P
from vuvosun_cases import as_numpy, left, make_config, mlstm, model, parallel, random_weights, right

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


def ctx_of(T, dtype):
    from titan_b200.engine.batch import StepEntry
    return make_ctx([StepEntry(0, [0] * T, [])], [0], DT[dtype])


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
    """The tensors under ``prefix`` as float64 numpy arrays, by their names below it."""
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
@pytest.mark.parametrize("S,W,T", [(2, 48, 9), (1, 40, 5), (3, 100, 70), (8, 24, 3), (4, 1000, 4)])
def test_streams_are_written_mixed_and_read(S, W, T):
    """The kernel between two sublayers: the write of a result into every stream with the mix among them, the normed blend for
    the next sublayer in either dtype, the plain sum that leaves the last layer, and the result's buffer left zeroed."""
    from titan_b200 import kernels as K
    g = torch.Generator().manual_seed(S * 100 + W)
    xs, y = torch.randn(T, S, W, generator=g) * 3, torch.randn(T, W, generator=g)
    mix, out_w, in_w, norm_w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(W, generator=g)
    new = torch.einsum("sr,tsw->trw", mix.double(), xs.double()) + out_w.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("r,trw->tw", in_w.double(), new)
    normed = t64(P.rms_div(u.numpy(), 1e-5)) * norm_w
    for dtype in BOTH:
        x_d, y_d = xs.reshape(T, S * W).cuda().clone(), y.cuda().clone()
        h = torch.empty(T, W, dtype=DT[dtype], device="cuda")
        K.hyper(x_d, S, K.current_stream(), y=y_d, mix=mix.cuda(), out_w=out_w.cuda(), in_w=in_w.cuda(), norm_w=norm_w.cuda(), eps=1e-5, h=h)
        rows_close(x_d.reshape(T, S, W), new.float(), "float32", "streams")
        rows_close(h, normed, dtype, "normed blend")
        assert float(y_d.abs().max()) == 0.0
    x_d = xs.reshape(T, S * W).cuda().clone()
    total = torch.empty(T, W, device="cuda")
    K.hyper(x_d, S, K.current_stream(), in_w=torch.ones(S, device="cuda"), h=total)
    rows_close(total, xs.double().sum(1).float(), "float32", "sum of the streams")
    assert torch.equal(x_d.cpu(), xs.reshape(T, S * W))                 # a read alone changes nothing
    h = torch.empty(T, W, device="cuda")
    K.hyper(x_d, S, K.current_stream(), in_w=in_w.cuda(), norm_w=norm_w.cuda(), eps=1e-5, h=h)
    rows_close(h, t64(P.rms_div(torch.einsum("r,trw->tw", in_w.double(), xs.double()).numpy(), 1e-5)) * norm_w, "float32", "read alone")


@pytest.mark.parametrize("dtype", BOTH)
def test_feed_forward_with_the_polynorm_activation(dtype):
    from titan_b200.config import FeedForwardSpec
    from titan_b200.parts import FEED_FORWARDS
    for F, T, coef in ((33, 5, (0.7, -0.4, 0.25, 0.1)), (192, 300, (0.0, 1.0, 0.0, -0.5)), (520, 3, (1.0, 0.5, 2.0, 0.0))):
        ff = FEED_FORWARDS.build(FeedForwardSpec("mlp", WIDTH, F, "polynorm", prefix="mlp.", extra=(("act_eps", 1e-5),)))
        w = weights_for(ff, 12)
        w["mlp.act"] = torch.tensor(coef).to(torch.bfloat16).float()
        w["mlp.up"] = w["mlp.up"] * 2
        bind(ff, w, DT[dtype])
        x = inputs([T], 13)[0]
        out = torch.zeros(T, WIDTH, device="cuda")
        ff.forward(x.to(DT[dtype]).cuda(), ctx_of(T, dtype), out)
        rows_close(out, t64(P.polynorm_ff(x.numpy(), plain_weights(w, "mlp."), 1e-5)), dtype, f"ff {F}", row_factor=6.0)


def attention_spec(H, G, dim, vdim, rot, base, scale, size, keep, eps=1e-5, out_scale=1.0):
    from titan_b200.config import MixerSpec, PositionSpec
    return MixerSpec("attention", WIDTH, H, G, dim, window=size, softmax_scale=scale, prefix="a.", position=PositionSpec("rope", rot, base, "adjacent"),
                     names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")),
                     extra=(("value_dim", vdim), ("value_norm", eps), ("keep_first", keep), ("sink", "sink"), ("out_gate", "g"), ("output_scale", out_scale)))


def attention_description(H, G, dim, vdim, rot, base, scale, size, keep):
    return left(H, G, dim, vdim, rot, base, scale, size, keep)


ATTENTION_SIZES = [
    (4, 2, 16, 16, 8, 300.0, 20, 3),          # a part of the head rotated; a window that keeps three tokens
    (3, 1, 12, 20, 4, 50.0, 7, 0),            # unequal widths, no multiples of 8; a window alone: a ring in the cache
    (6, 6, 24, 8, 24, 1e4, 65, 1),            # as many kv heads as heads; the whole head rotated; a window of a page and a row
    (2, 1, 32, 32, 32, 1e4, 5, 70),           # more kept tokens than a page holds, a window of five
    (4, 2, 64, 64, 48, 3e4, None, 0),         # no mask at all; bfloat16: the mma.sync kernels
    (4, 2, 64, 64, 64, 1e4, 64, 0),           # a ring of exactly a page; bfloat16: the mma.sync kernels where they take a ring
    (2, 1, 128, 128, 64, 1e4, None, 0),       # bfloat16: the tcgen05 prompt kernel
    (4, 2, 64, 64, 32, 1e4, 20, 3),           # bfloat16: the mma.sync kernels with kept tokens whose tile the window has left behind
    (2, 1, 128, 128, 64, 1e4, 40, 70),        # bfloat16: the tcgen05 prompt kernel with two tiles of kept tokens, then the window's
]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dim,vdim,rot,base,size,keep", ATTENTION_SIZES)
def test_attention_alone(dtype, H, G, dim, vdim, rot, base, size, keep):
    """Rotation of neighbours, normed values, window with kept first tokens, sink, gate and the mixer's factor: whole prompts of
    two unequal sequences, portions, portions of two tokens, then single tokens across a page's border; then the slots again."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(attention_spec(H, G, dim, vdim, rot, base, 0.4, size, keep, out_scale=0.75))
    w = weights_for(mixer, 3)
    w["a.sink"] = w["a.sink"] * 5 + 1.0                          # sinks that weigh as much as a key or more
    bind(mixer, w, DT[dtype])
    m = attention_description(H, G, dim, vdim, rot, base, 0.4, size, keep)
    lens = [330 if keep and dim >= 64 else 150, 71]      # long enough for a block of queries that skips tiles between the kept keys and its window
    xs = inputs(lens, 5)
    want = [0.75 * t64(P.windowed_sink_attention(x.numpy(), plain_weights(w, "a."), m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([lens], [[60, 33], [lens[0] - 100, 2], [2, 2], [2, 30]], [[1, 1]]):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


SIZE, KEEP, LAST = 72 + 9, 5, 229         # a window and a count of kept tokens for the test below; the last position


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim", [32, 64, 128])
@pytest.mark.parametrize("far,seen", [(0, True), (KEEP - 1, True), (KEEP, False), (63, False), (64, False), (LAST - SIZE, False), (LAST - SIZE + 1, True),
                                      (LAST - SIZE + 2, True), (191, True), (192, True), (LAST - 1, True)])
def test_one_key_decides_at_the_edges_of_the_window_and_of_the_kept_tokens(dtype, dim, far, seen):
    """The key matrix is minus the query matrix and the last token's input row is minus that of position ``far``: that one key,
    among hundreds, takes nearly all the softmax's weight if the last query sees it (a kept first token, the window's oldest
    key, a page's last row or the next page's first), and none if it lies one position outside.  Losing it, or seeing it when
    it is outside, changes the output altogether.  Through a whole prompt, as a single token, and in portions."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H = G = 2
    scale = 24.0 / dim
    mixer = MIXERS.build(attention_spec(H, G, dim, dim, 2, 1e6, scale, SIZE, KEEP))     # one rotated pair: the angle between far positions costs little
    w = weights_for(mixer, 7)
    w["a.k"] = -w["a.q"]
    w["a.g"] = w["a.g"] * 0.0                                      # a gate of one half everywhere
    w["a.sink"] = torch.tensor([0.5, -1.0])
    bind(mixer, w, DT[dtype])
    m = attention_description(H, G, dim, dim, 2, 1e6, scale, SIZE, KEEP)
    n = LAST + 1
    x = inputs([n], 8)[0]
    x[far] = x[far] * 1.5                                       # a loud key: its score with its own query grows with the square
    x[-1] = -x[far]
    assert P.sees(LAST, far, SIZE, KEEP) == seen
    W = plain_weights(w, "a.")
    want = t64(P.windowed_sink_attention(x.numpy(), W, m, 1e-5))
    v = (x[far].numpy() @ W["v"].T).reshape(G, dim)
    only_far = t64(0.5 * P.rms_div(v, 1e-5).reshape(-1) @ W["o"].T)            # what the heads return if that key has all the weight
    if seen:
        assert rel_l2(only_far, want[-1]) < 0.2, "the test's weights do not single the key out"
    else:
        assert rel_l2(only_far, want[-1]) > 0.7, "the key outside the window still decides the plain result"
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    step = mixer_step(mixer, cache)
    whole = drive(step, cache, [x], dtype, [[n]])[0]
    rows_close(whole[-1:], want[-1:], dtype, "in a prompt", row_factor=6.0)
    decoded = drive(step, cache, [x], dtype, [[n - 1]])[0]
    rows_close(decoded[-1:], want[-1:], dtype, "decoded alone", row_factor=6.0)
    pieces = drive(step, cache, [x], dtype, [[far + 1], [max(1, n - far - 3)], [2]])[0]       # a portion that ends on the key, and one of two tokens
    rows_close(pieces, want, dtype, "every row, in portions", row_factor=6.0)
    long_tail = drive(step, cache, [x], dtype, [[max(1, far)]])[0]            # everything after the key decoded token by token
    rows_close(long_tail, want, dtype, "every row, decoded from the key on", row_factor=6.0)


def delta_spec(H, G, dk, dv, taps, out_scale=1.0, eps=1e-5):
    from titan_b200.config import MixerSpec
    return MixerSpec("gated_delta", WIDTH, H, G, dk, prefix="r.", extra=(("value_dim", dv), ("taps", taps), ("norm_eps", eps), ("output_scale", out_scale)))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 8, 12, 3), (1, 1, 40, 20, 4), (2, 2, 64, 64, 2), (6, 2, 20, 36, 5), (1, 1, 130, 8, 1), (3, 1, 4, 70, 4),
                                             (8, 4, 128, 128, 4), (2, 1, 256, 32, 3)])
def test_delta_rule_alone(dtype, H, G, dk, dv, taps):
    """Two sequences through whole prompts, portions down to two tokens (shorter than the convolution) and single tokens, then
    the slots given back and used again: outputs, and a state (memory and convolution window) that starts from zero."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(delta_spec(H, G, dk, dv, taps, out_scale=1.25))
    w = weights_for(mixer, 9)
    g = torch.Generator().manual_seed(10)
    w["r.A_log"] = (torch.randn(H, generator=g) - 1.0).to(torch.bfloat16).float()          # decays from nearly 1 to well below
    w["r.dt_bias"] = torch.randn(H, generator=g).to(torch.bfloat16).float()
    w["r.a"], w["r.b"] = w["r.a"] * 3, w["r.b"] * 3
    bind(mixer, w, DT[dtype])
    m = right(H, G, dk, dv, taps)
    lens = [90, 37]
    xs = inputs(lens, 11)
    want = [1.25 * t64(P.gated_delta(x.numpy(), plain_weights(w, "r."), m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([[90, 37]], [[40, 20], [2, 2], [17, 1], [2, 0], [1, 2]], []):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


def test_delta_rule_remembers_a_value_far_back():
    """A decay of nearly one and a key that no later key resembles: 300 tokens on, a query that equals that key reads its
    value out of the state.  Keys and queries read one half of the input row and values the other, and the last token has
    the early token's key half but a value half of its own: what it returns is a blend of its own value and the early
    one, so a state that lost the early write gives another direction (float32; whole, and decoded token by token after the
    write)."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H, dk, dv = 1, 16, 16
    half = WIDTH // 2
    mixer = MIXERS.build(delta_spec(H, H, dk, dv, 1))
    w = weights_for(mixer, 21)
    w["r.A_log"], w["r.dt_bias"] = torch.tensor([-12.0]), torch.tensor([-6.0])      # g = exp(-e^-12 softplus(.)): no forgetting to speak of
    w["r.a"], w["r.b"] = w["r.a"] * 0.0, w["r.b"] * 0.0                                # beta = 1/2 everywhere
    w["r.q"][:, half:] = 0.0
    w["r.k"] = w["r.q"].clone()
    w["r.v"][:, :half] = 0.0
    w["r.q.conv"], w["r.k.conv"], w["r.v.conv"] = torch.ones(dk, 1), torch.ones(dk, 1), torch.ones(dv, 1)
    bind(mixer, w, torch.float32)
    n = 300
    x = inputs([n], 22)[0] * 0.05
    x[3] = inputs([1], 23)[0][0] * 4                                # a loud token early on
    x[-1, :half] = x[3, :half]                                      # and its key, with another value, at the end
    m = right(H, H, dk, dv, 1)
    W = plain_weights(w, "r.")
    want = t64(P.gated_delta(x.numpy(), W, m, 1e-5))
    quiet = x.clone()
    quiet[3] = quiet[4]
    assert rel_l2(t64(P.gated_delta(quiet.numpy(), W, m, 1e-5))[-1], want[-1]) > 0.3, "the early token does not reach the last position"
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, torch.float32, "cuda", mark_freed=True)
    for sizes in ([[n]], [[5]], [[64], [64], [2]]):
        got = drive(mixer_step(mixer, cache), cache, [x], "float32", sizes)[0]
        rows_close(got, want, "float32", f"portions {sizes}", row_factor=6.0)


def mlstm_spec(H, dk, dv, cap, eps=1e-5):
    from titan_b200.config import MixerSpec
    return MixerSpec("mlstm", WIDTH, H, head_dim=dk, prefix="m.", extra=(("value_dim", dv), ("gate_cap", cap), ("norm_eps", eps)))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dk,dv,cap", [(3, 8, 12, 10.0), (1, 40, 20, 15.0), (2, 64, 128, 12.0), (2, 20, 24, 3.0), (1, 130, 8, 8.0), (5, 4, 70, 20.0),
                                          (4, 128, 128, 12.0), (1, 256, 64, 6.0)])
def test_mlstm_alone(dtype, H, dk, dv, cap):
    """Gates on both sides of their caps and of the running maximum's start (input gates below and above zero): whole prompts,
    portions, single tokens, and slots used again."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(mlstm_spec(H, dk, dv, cap))
    w = weights_for(mixer, 15)
    g = torch.Generator().manual_seed(16)
    w["m.i"], w["m.f"] = w["m.i"] * 6, w["m.f"] * 6
    w["m.i.b"] = (torch.randn(H, generator=g) * 2).to(torch.bfloat16).float()
    w["m.f.b"] = (torch.randn(H, generator=g) * 2 + 2).to(torch.bfloat16).float()
    bind(mixer, w, DT[dtype])
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    lens = [90, 37]
    xs = inputs(lens, 17)
    want = [t64(P.mlstm(x.numpy(), plain_weights(w, "m."), m, 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([[90, 37]], [[40, 20], [2, 2], [17, 1], [2, 0]], []):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
def test_two_mixers_side_by_side_with_their_factors(dtype):
    """The parallel mixer: both branches on the same rows, each with its own cache view and factor."""
    from titan_b200.cache import SequenceCache
    from titan_b200.config import MixerSpec
    from titan_b200.parts import MIXERS
    a = attention_spec(4, 2, 16, 8, 8, 300.0, 0.3, 20, 3, out_scale=0.6)
    r = delta_spec(4, 2, 8, 12, 3, out_scale=1.7)
    mixer = MIXERS.build(MixerSpec("parallel", WIDTH, prefix="p.", extra=(("branches", (a, r)),)))
    w = weights_for(mixer, 19)
    bind(mixer, w, DT[dtype])
    lens = [100, 30]
    xs = inputs(lens, 20)
    want = [0.6 * t64(P.windowed_sink_attention(x.numpy(), plain_weights(w, "p.a."), attention_description(4, 2, 16, 8, 8, 300.0, 0.3, 20, 3), 1e-5))
            + 1.7 * t64(P.gated_delta(x.numpy(), plain_weights(w, "p.r."), right(4, 2, 8, 12, 3), 1e-5)) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, DT[dtype], "cuda", mark_freed=True)
    for sizes in ([[100, 30]], [[70, 2], [2, 20]]):
        got = drive(mixer_step(mixer, cache), cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


# --------------------------------------------------------------------------- #
# whole models
# --------------------------------------------------------------------------- #
def close(got, want, dtype, what="", slack=1.0):
    return rows_close(got, want, dtype, what, row_factor=6.0, slack=slack)


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
            logits, after = P.forward(self.cfg, self.numpy, list(tokens))
            self._plain[key] = (t64(logits), t64(after))
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
    """In float32 every request is held to the bound by itself.  In bfloat16 the requests' rows are judged together, and each
    row by the row bound: a prompt of two or three tokens has no later tokens over which the rounding of a 40-wide head's
    q . k sums (about 1e-2 each in 8 bits of mantissa) would average out."""
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
def test_the_sum_of_the_streams_after_every_layer(name, dtype):
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
    freed slots and pages (which were overwritten when they were freed), in the other order.  In float32 every request is
    held to the plain result by itself; in bfloat16 the requests' rows are judged together against it (a prompt of three tokens
    has too few rows for its rounding to average out), and each request against the same request run alone."""
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
                    e.free_slot(slots[i])                      # a shorter request leaves; its slot may be taken in the next turn
        for i in order:
            if dtype == "float32":
                close(torch.cat(got[i]), wd.plain(reqs[i]), dtype, f"{name}: request {i} in a batch, turn {turn}")
            close(torch.cat(got[i]), alone[i], dtype, f"{name}: request {i} in a batch against itself alone, turn {turn}")
        close(torch.cat([torch.cat(got[i]) for i in order]), torch.cat([wd.plain(reqs[i]) for i in order]), dtype, f"{name}: all requests of a batch, turn {turn}")
        e.cache.check()
    e.check_kernels()


@pytest.mark.parametrize("dtype", BOTH)
def test_a_loud_first_token_reaches_far_through_states_and_kept_keys(dtype):
    """The first token's embedding row is unlike the others': every later position feels it, through the recurrences' states and
    through the attention's kept first key, in a prompt and when decoded token by token."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg = make_config("mix")
    w = random_weights(cfg, 5)
    toks = random_tokens(200, cfg["vocab"], 77)
    toks[0] = 3
    assert 3 not in toks[1:]
    want = t64(P.forward(cfg, as_numpy(w), toks)[0])
    other = list(toks)
    other[0] = 4
    assert rel_l2(t64(P.forward(cfg, as_numpy(w), other)[0])[-1], want[-1]) > 20 * TOL["float32"], "the first token does not reach the last position"
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=1024, max_slots=2)
    close(run_in_pieces(e, toks, [len(toks)]), want, dtype, "whole")
    close(run_in_pieces(e, toks, [100]), want, dtype, "decoded from 100")
    close(run_in_pieces(e, toks, [1, 2]), want, dtype, "decoded from the first tokens on")


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding(dtype):
    """A short prompt, then 400 single tokens over several pages and several turns of every window (captured steps where the
    engine captures them)."""
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
            logits = t64(P.forward(wd.cfg, wd.numpy, seq)[0][-1])
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
    rows_close(captured, out, "bfloat16", "captured against whole prompts")
    e.check_kernels()


def test_trace_runner_as_a_subprocess(tmp_path):
    """bin/trace_run on a model folder: a batch of two prompts, single tokens after them while one request leaves, then many
    short requests at once, in slots and pages that were used before."""
    cfg = make_config("odd")
    weights = random_weights(cfg, 9)
    folder = write_folder(str(tmp_path / "model"), cfg, {k: v.to(torch.bfloat16) for k, v in weights.items()})
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
    pa, pb = t64(P.forward(cfg, W, a)[0]), t64(P.forward(cfg, W, b)[0])
    V = cfg["vocab"]
    read = lambda name: torch.from_numpy(np.fromfile(out / name, dtype="<f4").reshape(-1, V))
    rows_close(read("0.f32"), torch.stack([pa[0], pa[59], pb[19]]), "float32", "step 0")
    rows_close(read("1.f32"), torch.stack([pa[60], pb[20]]), "float32", "step 1")
    rows_close(read("10.f32"), pa[69:70], "float32", "step 10")
    rows_close(read("12.f32"), torch.stack([t64(P.forward(cfg, W, m)[0])[2] for m in many]), "float32", "twenty short requests")


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
    """A configuration drawn at random: sizes, head counts, layer order, windows, constants, odd sizes and ones included."""
    import random
    r = random.Random(seed)
    width = r.choice([24, 40, 56, 72, 100, 136])
    layers = []
    for i in range(r.randint(2, 5)):
        ff = r.choice([None, 16, 33, 64, 100])
        if r.random() < 0.6:
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 4])
            dim = r.choice([6, 8, 12, 16, 20, 32, 40, 64])
            vdim = r.choice([dim, dim, 8, 24, 16])
            rot = r.choice([d for d in (2, 4, 6, 8, 16, 32, 64) if d <= dim])
            size = r.choice([None, 1, 2, 5, 31, 64, 65, 100, 500])
            keep = r.choice([0, 0, 1, 2, 7, 66])
            a = left(heads, kv, dim, vdim, rot, base=r.choice([100.0, 1e4, 5e5]), scale=r.choice([0.1, 0.3, dim ** -0.5]), size=size, keep_first=keep)
            g = r.choice([1, 2, 3])
            b = right(g * r.choice([1, 2, 3]), g, r.choice([4, 8, 12, 24, 48, 72]), r.choice([4, 8, 20, 33, 64]), r.choice([1, 2, 3, 4, 6]))
            layers.append(parallel(a, b, r.choice([0.5, 1.0, 1.4]), r.choice([0.3, 1.0, 2.0]), ff=ff))
        else:
            layers.append(mlstm(r.choice([1, 2, 3, 5]), r.choice([4, 8, 12, 24, 48, 72]), r.choice([4, 8, 20, 33, 64]), r.choice([1.0, 5.0, 15.0, 30.0]), ff=ff))
    return model(layers, width=width, vocab=r.choice([50, 97, 300]), eps=r.choice([1e-6, 1e-5, 1e-4]), streams=r.choice([1, 2, 3, 4, 5]))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("seed", range(int(os.environ.get("VUVOSUN_DRAWN", "12"))))
def test_configurations_drawn_at_random(seed, dtype):
    """A prompt whole, then a second request as a prompt with single tokens after it, in a batch with a third.  float32 is
    the sharp test here (a wrong branch costs tens of percent, summation order 1e-6).  For bfloat16 the bound follows the
    model: the drawn models have heads of four dimensions and feed-forwards of sixteen values whose cubes pass a norm, and
    where the mLSTM read-out's denominator |n . q| comes near zero or near its floor a row amplifies whatever rounding
    reaches it, and the states carry that on.  How much a model amplifies rounding shows in the float32 engine's own error
    against the float64 result; bfloat16 rounds 2^15 times as coarsely (its error is measured at 0.4 to 0.6 of that multiple), so
    the whole tensor is held to 2^16 times the float32 error, at least twice the usual bound and never more than 0.15; and
    since the row that comes near a zero of its denominator is another one in each rounding, rows are counted: one in twenty
    may be off by more than six times the usual bound, none by as much as its own size."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg = drawn_config(seed)
    w = random_weights(cfg, 100 + seed)
    W = as_numpy(w)
    a, b, c = (random_tokens(n, cfg["vocab"], 7 * seed + n) for n in (75, 130, 9))

    def run(dt):
        e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dt, max_tokens=1024, max_slots=4, mark_freed_pages=True)
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
        return whole, torch.cat(got_b).float().cpu()

    want = t64(P.forward(cfg, W, a)[0]), t64(P.forward(cfg, W, b)[0])
    got = run(dtype)
    names = (f"seed {seed}: whole", f"seed {seed}: prompt in a batch, then single tokens")
    if dtype == "float32":
        for g, x, name in zip(got, want, names):
            close(g, x, dtype, name)
        return
    exact = run("float32")
    for g, g32, x, name in zip(got, exact, want, names):
        err, bound = rel_l2(g, x), min(max(2 * TOL[dtype], 2.0 ** 16 * rel_l2(g32, x)), 0.15)
        assert err < bound, f"{name}: relative error {err:.3e} over the bound {bound:.1e}"
        rows = (g.double() - x.double()).norm(dim=1) / x.double().norm(dim=1)
        assert float((rows > 6 * TOL[dtype]).double().mean()) <= 0.05 and float(rows.max()) < 1.0, \
            f"{name}: {int((rows > 6 * TOL[dtype]).sum())} of {len(rows)} rows are off by more than {6 * TOL[dtype]:.2f}, the worst by {float(rows.max()):.2f}"
