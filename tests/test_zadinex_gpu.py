"""The Zadinex design in the engine against the plain implementation (tests/plain/zadinex_plain.py): every mechanism
alone, then whole models under every way of cutting the work.  Needs a B200; float32 (true 32-bit) and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL, random_tokens, rel_l2, rows_close, write_folder
from plain import zadinex_plain as P
from zadinex_cases import make_config

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
    """The context of a step that brings one prompt of T tokens."""
    from titan_b200.engine.batch import StepEntry
    return make_ctx([StepEntry(0, [0] * T, [])], [0], DT[dtype])


def bind(part, weights, dtype, prefix=""):
    from titan_b200.weights import held_dtype
    specs = {w.name: w for w in part.weight_specs(prefix)}
    part.bind(lambda rel: weights[prefix + rel].to("cuda", held_dtype(specs[prefix + rel].role, dtype)).contiguous())


def weights_for(part, seed, prefix=""):
    """bfloat16-representable random tensors for a part's declaration: matrices ~ N(0, 1/fan_in), vectors around one or zero."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for w in part.weight_specs(prefix):
        t = torch.randn(w.shape, generator=g)
        if w.role == "vector":
            t = t * 0.3 + (1.0 if w.init[0] == "one_plus_normal" else 0.0)
        else:
            t = t / (w.shape[-1] ** 0.5)
        out[w.name] = t.to(torch.bfloat16).float()
    return out


def close(got, want, dtype, what=""):
    """float32: the tensor and every row within the bound.  bfloat16: a token whose router scores nearly tie may take another
    expert than the plain implementation, which moves that row (and, through state and cache, some after it) by more than
    rounding does; so the typical row must be within the bound and five in six within four times the bound."""
    if dtype == "float32":
        return rows_close(got, want, dtype, what)
    g, w = got.double().cpu().reshape(-1, got.shape[-1]), want.double().reshape(-1, want.shape[-1])
    assert g.shape == w.shape, what
    per_row = (g - w).norm(dim=1) / w.norm(dim=1).clamp_min(1e-30)
    assert float(per_row.median()) < TOL[dtype], f"{what}: median row error {float(per_row.median()):.3e}"
    if len(per_row) >= 6:
        assert float((per_row < 4 * TOL[dtype]).double().mean()) >= 5 / 6, f"{what}: too many rows over four times the bound"


def inputs(lens, seed, width=WIDTH):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, width, generator=g).to(torch.bfloat16).double() for n in lens]


def drive(run_step, cache, xs, dtype, first_sizes, width=WIDTH):
    """Feed the sequences ``xs`` (rows of inputs) through ``run_step(h, ctx) -> out`` on two slots: first in portions of the
    given sizes (one list per step, a size per sequence), then token by token.  Returns each sequence's output rows."""
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


# --------------------------------------------------------------------------- #
# mechanisms alone
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("dtype", BOTH)
def test_norm_without_statistics_and_the_scaled_sum(dtype):
    """tanh(alpha x) w + b alone, on picked rows, and inside the kernel that adds a scaled sublayer output to the stream."""
    from titan_b200 import kernels as K
    from titan_b200.config import NormSpec
    from titan_b200.parts import NORMS
    norm = NORMS.build(NormSpec("dyt", 52, 1e-5, "n"))
    w = weights_for(norm, 1)
    w["n.alpha"] = torch.tensor(0.37)
    bind(norm, w, DT[dtype])
    W = {k: v.double() for k, v in w.items()}
    x = torch.randn(9, 52, generator=torch.Generator().manual_seed(2)) * 3
    ctx = ctx_of(9, dtype)
    rows_close(norm.forward(x.cuda(), ctx), P.tanh_norm(x.double(), W, "n"), dtype, "norm")
    pick = torch.tensor([7, 0, 3], dtype=torch.int32)
    rows_close(norm.forward(x.cuda(), ctx, pick.cuda()), P.tanh_norm(x.double()[pick.long()], W, "n"), dtype, "picked rows")
    y, s = torch.randn(9, 52, generator=torch.Generator().manual_seed(3)), torch.rand(52, generator=torch.Generator().manual_seed(4)) * 2 - 0.5
    xg, yg, h = x.cuda().clone(), y.cuda().clone(), torch.empty(9, 52, dtype=DT[dtype], device="cuda")
    K.scale_add(yg, s.cuda(), xg, K.current_stream(), zero_y=True, norm=norm.triple(), h=h)
    want = x.double() + s.double() * y.double()
    rows_close(xg, want, "float32", "stream")
    rows_close(h, P.tanh_norm(want, W, "n"), dtype, "next norm")
    assert float(yg.abs().max()) == 0.0


def attention_spec(H, G, dim, vdim, rot, base, scale, value_mix=None, layer=0, eps=1e-5):
    from titan_b200.config import MixerSpec, PositionSpec
    extra = [("value_dim", vdim), ("unit_norm", "after_rotation"), ("unit_norm_eps", eps), ("sink", "sink"), ("layer_index", layer)]
    if value_mix is not None:
        extra.append(("value_mix", value_mix))
    return MixerSpec("attention", WIDTH, H, G, dim, softmax_scale=scale, prefix="mix.", position=PositionSpec("rope", rot, base, "half"),
                     names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")), extra=tuple(extra))


ATTENTION_SIZES = [
    (4, 2, 16, 16, 8, 300.0),          # a part of the head rotated
    (3, 1, 12, 20, 4, 50.0),           # keys and values of unequal widths, no multiples of 8: padded in the cache
    (6, 6, 24, 8, 24, 1e4),            # as many kv heads as heads; the whole head rotated; values narrower than keys
    (4, 2, 64, 64, 48, 3e4),           # bfloat16: the mma.sync kernels
    (2, 1, 128, 128, 64, 1e4),         # bfloat16: the tcgen05 prompt kernel
]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,dim,vdim,rot,base", ATTENTION_SIZES)
def test_attention_alone_with_blended_values(dtype, H, G, dim, vdim, rot, base):
    """Two attention mixers in one step, the second blending its values with the first one's: whole prompts of two unequal
    sequences, a further portion, portions of two tokens, then single tokens across a page's border."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot}, "scale": 0.4, "v_mix": True}
    first = MIXERS.build(attention_spec(H, G, dim, vdim, rot, base, 0.4, (None, "vmix"), 0))
    second = MIXERS.build(attention_spec(H, G, dim, vdim, rot, base, 0.4, (0, "vmix"), 1))
    w1, w2 = weights_for(first, 3), weights_for(second, 4)
    w2["mix.vmix"] = torch.tensor(0.3125)
    w1["mix.sink"], w2["mix.sink"] = w1["mix.sink"] * 3, w2["mix.sink"] * 3 + 1.0       # sinks that weigh as much as a key or more
    bind(first, w1, DT[dtype]); bind(second, w2, DT[dtype])
    lens = [150, 71]
    xs, zs = inputs(lens, 5), inputs(lens, 6)           # the two layers' input rows
    W1, W2 = {k: v.double() for k, v in w1.items()}, {k: v.double() for k, v in w2.items()}
    want1, want2 = [], []
    for x, z in zip(xs, zs):
        pos = torch.arange(x.shape[0])
        v1 = P.attention_values(x, m, W1, "mix.", None)
        want1.append(P.attention(x, m, W1, "mix.", 1e-5, pos, v1).float())
        want2.append(P.attention(z, m, W2, "mix.", 1e-5, pos, P.attention_values(z, m, W2, "mix.", v1)).float())
    cache = SequenceCache([first.cache_need(), second.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    both = [torch.cat([x, z], dim=1) for x, z in zip(xs, zs)]

    def step(h, ctx):
        out = torch.zeros(h.shape[0], 2 * WIDTH, device="cuda")
        a, b = torch.zeros(h.shape[0], WIDTH, device="cuda"), torch.zeros(h.shape[0], WIDTH, device="cuda")
        first.forward(h[:, :WIDTH].contiguous(), ctx, cache.view_for_layer(0), a)
        second.forward(h[:, WIDTH:].contiguous(), ctx, cache.view_for_layer(1), b)
        out[:, :WIDTH], out[:, WIDTH:] = a, b
        return out

    got = drive(step, cache, both, dtype, [[60, 33], [50, 2], [2, 2], [2, 30]], width=2 * WIDTH)
    for i in range(2):
        rows_close(got[i][:, :WIDTH], want1[i], dtype, f"first layer, sequence {i}", row_factor=6.0)
        rows_close(got[i][:, WIDTH:], want2[i], dtype, f"blending layer, sequence {i}", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim,far", [(32, 0), (32, 1), (32, 63), (32, 64), (32, 65), (32, 127), (32, 128), (64, 0), (64, 63), (64, 64), (64, 191), (64, 192)])
def test_one_far_key_decides(dtype, dim, far):
    """The key matrix is minus the query matrix and the last token's input row is minus that of position ``far`` (the first
    tokens, a page's last row, the next page's first): with unit heads and a sharp softmax that one key takes nearly all
    the weight (the last token's own key is the opposite of its query), so losing it or its value, among hundreds of
    others, changes the output altogether.  Through a whole prompt, as a single token, and in a portion of two."""
    from titan_b200.cache import SequenceCache
    from titan_b200.parts import MIXERS
    H = G = 2
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "rot": {"base": 1e6, "dims": 2}, "scale": 24.0 / dim, "v_mix": False}
    mixer = MIXERS.build(attention_spec(H, G, dim, dim, 2, 1e6, 24.0 / dim))      # one rotated pair: the angle between far positions costs little of the score
    w = weights_for(mixer, 7)
    w["mix.k"] = -w["mix.q"]
    w["mix.sink"] = torch.tensor([0.5, -1.0])
    bind(mixer, w, DT[dtype])
    W = {k: v.double() for k, v in w.items()}
    n = 230
    x = inputs([n], 8)[0]
    x[-1] = -x[far]                                    # the last query looks for position ``far``
    pos = torch.arange(n)
    want = P.attention(x, m, W, "mix.", 1e-5, pos, P.attention_values(x, m, W, "mix.", None)).float()
    just_values = torch.nn.functional.linear(x[far].float(), w["mix.v"])              # what the heads return if that key has all the weight
    assert rel_l2(torch.nn.functional.linear(just_values, w["mix.o"]), want[-1]) < 0.2, "the test's weights do not single the key out"
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)

    def step(h, ctx):
        out = torch.zeros(h.shape[0], WIDTH, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        return out

    whole = drive(step, cache, [x], dtype, [[n]])[0]
    rows_close(whole[-1:], want[-1:], dtype, "in a prompt", row_factor=6.0)
    decoded = drive(step, cache, [x], dtype, [[n - 1]])[0]
    rows_close(decoded[-1:], want[-1:], dtype, "decoded alone", row_factor=6.0)
    pieces = drive(step, cache, [x], dtype, [[far + 1], [n - far - 3], [2]])[0]          # a portion that ends on the key, and one of two tokens
    rows_close(pieces[-1:], want[-1:], dtype, "in portions", row_factor=6.0)
    rows_close(pieces, want, dtype, "every row, in portions", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dk,rank", [(3, 8, 5), (1, 40, 3), (2, 64, 16), (2, 20, 9), (1, 130, 7), (4, 32, 32), (2, 96, 8),
                                          (80, 8, 4), (40, 64, 6), (20, 128, 5)])      # the last three: heads enough for the kernel of four lanes a column
def test_wkv_alone(dtype, H, dk, rank):
    """Two sequences through whole prompts, portions of two tokens and single tokens, then the slots given back and used
    again: outputs, and a state that starts from zero for the next owner."""
    from titan_b200.cache import SequenceCache
    from titan_b200.config import MixerSpec
    from titan_b200.parts import MIXERS
    mixer = MIXERS.build(MixerSpec("wkv", WIDTH, H, head_dim=dk, prefix="mix.", extra=(("rank", rank), ("norm_eps", 1e-5))))
    w = weights_for(mixer, 9)
    g = torch.Generator().manual_seed(10)
    for s in "rkvgw":
        w["mix.mu." + s] = torch.rand(WIDTH, generator=g).to(torch.bfloat16).float()
    w["mix.w0"] = (torch.randn(H * dk, generator=g) - 1.5).to(torch.bfloat16).float()      # decays from nearly 1 to nearly 0
    bind(mixer, w, DT[dtype])
    m = {"heads": H, "dim": dk}
    lens = [90, 37]
    xs = inputs(lens, 11)
    W = {k: v.double() for k, v in w.items()}
    want = [P.wkv(x, m, W, "mix.", 1e-5)[0].float() for x in xs]
    cache = SequenceCache([mixer.cache_need()], 1024, 2, 512, DT[dtype], "cuda", mark_freed=True)

    def step(h, ctx):
        out = torch.zeros(h.shape[0], WIDTH, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        return out

    for sizes in ([[90, 37]], [[40, 20], [2, 2], [17, 1], [2, 0]], []):      # whole; portions; token by token (in slots used before)
        got = drive(step, cache, xs, dtype, sizes)
        for i in range(2):
            rows_close(got[i], want[i], dtype, f"sequence {i}, portions {sizes}", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
def test_dense_feed_forward_with_the_gelu_gate(dtype):
    from titan_b200.config import FeedForwardSpec
    from titan_b200.parts import FEED_FORWARDS
    for F, T in ((33, 5), (192, 300)):
        ff = FEED_FORWARDS.build(FeedForwardSpec("gated_mlp", WIDTH, F, "gelu_tanh", prefix="mlp.", names=(("gate", "gate"), ("up", "up"), ("down", "down"))))
        w = weights_for(ff, 12)
        w["mlp.gate"] = w["mlp.gate"] * 3              # into the curved part of the gate
        bind(ff, w, DT[dtype])
        x = inputs([T], 13)[0]
        out = torch.zeros(T, WIDTH, device="cuda")
        ff.forward(x.to(DT[dtype]).cuda(), ctx_of(T, dtype), out)
        rows_close(out, P.dense_ff(x, {k: v.double() for k, v in w.items()}, "mlp.").float(), dtype, f"ff {F}", row_factor=6.0)


def moe_spec(E, top, F, limit, identity, groups, keep):
    from titan_b200.config import FeedForwardSpec
    return FeedForwardSpec("moe", WIDTH, F, "swish_clamped", prefix="mlp.",
                           extra=(("experts", E), ("top", top), ("identity", identity), ("routing", "softmax_all"), ("groups", groups), ("keep", keep), ("limit", limit)))


@pytest.mark.parametrize("E,top,identity,groups,keep", [(6, 2, 2, 4, 2), (5, 1, 0, 1, 1), (3, 2, 3, 3, 1), (8, 3, 0, 4, 3), (4, 4, 4, 2, 2), (30, 4, 2, 8, 3)])
def test_router_choice_and_weights(E, top, identity, groups, keep):
    """The choice alone, on logits made by hand: scores over all outputs, corrections that turn choices around and push every
    choice score below zero, groups that shut better experts out, ties left aside."""
    from titan_b200 import kernels as K
    n_all, T = E + identity, 64
    g = torch.Generator().manual_seed(E * 100 + top)
    z = (torch.randn(T, n_all, generator=g) * 2).float()
    corr = torch.randn(n_all, generator=g).float() * 0.3 - 1.0       # every choice score negative: a closed group must count as minus infinity, not 0
    f = {"router": {"experts": E, "top": top, "identity": identity, "groups": {"count": groups, "keep": keep}}}
    W = {"r.router": torch.eye(n_all, dtype=torch.float64), "r.correction": corr.double()}
    idx, wts = P.routed_choice(z.double(), f, W, "r.")
    ids, got = torch.empty(T, top, dtype=torch.int32, device="cuda"), torch.empty(T, top, device="cuda")
    K.moe_route_all(z.cuda(), top, corr.cuda(), groups, keep, ids, got, K.current_stream())
    order = ids.cpu().long().argsort(dim=1)
    want_order = idx.argsort(dim=1)
    assert torch.equal(ids.cpu().long().gather(1, order), idx.gather(1, want_order))
    assert torch.allclose(got.cpu().double().gather(1, order), wts.gather(1, want_order), atol=1e-6)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top,F,limit,identity,groups,keep,T", [
    (6, 2, 24, 1.5, 2, 4, 2, 7),        # a few pairs: a warp per output
    (5, 1, 18, 0.7, 0, 1, 1, 150),      # one expert a token; a limit that clamps often
    (3, 2, 10, 2.5, 3, 3, 1, 90),       # as many pass-through experts as real ones
    (10, 2, 72, 1.0, 2, 3, 1, 700),     # bfloat16: rows gathered by expert, tensor-core products
])
def test_mixture_of_experts_alone(dtype, E, top, F, limit, identity, groups, keep, T):
    from titan_b200.parts import FEED_FORWARDS
    ff = FEED_FORWARDS.build(moe_spec(E, top, F, limit, identity, groups, keep))
    w = weights_for(ff, 14)
    w["mlp.router"] = w["mlp.router"] * 6              # decided choices: the two dtypes route alike
    for e in range(E):
        w[f"mlp.e{e}.gate"], w[f"mlp.e{e}.up"] = w[f"mlp.e{e}.gate"] * 2, w[f"mlp.e{e}.up"] * 2      # sums beyond the limit on both sides
    bind(ff, w, DT[dtype])
    x = inputs([T], 15)[0]
    out = torch.zeros(T, WIDTH, device="cuda")
    ff.forward(x.to(DT[dtype]).cuda(), ctx_of(T, dtype), out)
    f = {"expert": {"ff": F, "limit": limit}, "router": {"experts": E, "top": top, "identity": identity, "groups": {"count": groups, "keep": keep}}}
    close(out, P.mixture_of_experts(x, f, {k: v.double() for k, v in w.items()}, "mlp.").float(), dtype, "mixture")


# --------------------------------------------------------------------------- #
# whole models
# --------------------------------------------------------------------------- #
class World:
    """One small model: weights, plain logits of its requests, engines by dtype and options."""

    def __init__(self, name, seed, lengths):
        self.cfg = make_config(name)
        self.weights = P.random_weights(self.cfg, seed)
        self.requests = [random_tokens(n, self.cfg["vocab"], 50 + i) for i, n in enumerate(lengths)]
        self._plain, self._engines = {}, {}

    def plain(self, tokens):
        key = tuple(tokens)
        if key not in self._plain:
            self._plain[key] = P.forward(self.cfg, self.weights, list(tokens)).float()
        return self._plain[key]

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
    for toks in wd.requests:
        close(run_in_pieces(e, toks, [len(toks)]), wd.plain(toks), dtype, f"{name}: prompt of {len(toks)}")
    e.check_kernels()
    e.cache.check()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_the_residual_stream_after_every_layer(name, dtype):
    """Layer by layer in float32 terms: the first layer that differs is named."""
    from titan_b200 import StepEntry
    wd = world(name)
    e = wd.engine(dtype)
    toks = wd.requests[2]
    trace = []
    P.forward(wd.cfg, wd.weights, toks, trace=trace)
    seen = []
    originals = [b.forward for b in e.model.blocks]
    try:
        for b, orig in zip(e.model.blocks, originals):
            b.forward = (lambda x, ctx, cache, orig=orig: (orig(x, ctx, cache), seen.append(x.clone()))[0])
        s = e.alloc_slot()
        e.step([StepEntry(s, toks, [0])])
        e.free_slot(s)
    finally:
        for b, orig in zip(e.model.blocks, originals):
            b.forward = orig
    assert len(seen) == len(trace)
    for i, (got, want) in enumerate(zip(seen, trace)):
        close(got, want.float(), dtype, f"{name}: after layer {i}")


@pytest.mark.parametrize("name,dtype", MODELS)
def test_prompt_then_token_by_token_and_portions_down_to_two(name, dtype):
    wd = world(name)
    e = wd.engine(dtype)
    toks = wd.requests[0]
    want = wd.plain(toks)
    close(run_in_pieces(e, toks, [len(toks) - 40]), want, dtype, f"{name}: prompt then 40 single tokens")
    close(run_in_pieces(e, toks, [1]), want[: len(toks)], dtype, f"{name}: token by token from the first")
    close(run_in_pieces(e, toks, [64, 2, 2, 31, 1, 2, 40]), want, dtype, f"{name}: portions")
    close(run_in_pieces(e, toks, [2] * (len(toks) // 2)), want, dtype, f"{name}: portions of two")
    e.check_kernels()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_a_batch_of_unequal_requests_against_each_alone_and_slots_used_again(name, dtype):
    """All requests as one batch of prompts, decoded together while the shorter ones leave; then the same again in the
    freed slots and pages (which were overwritten when they were freed)."""
    from titan_b200 import StepEntry
    wd = world(name)
    e = wd.engine(dtype)
    reqs = wd.requests
    tail = 6
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
        while any(at[i] < len(reqs[i]) for i in order):
            live = [i for i in order if at[i] < len(reqs[i])]
            out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
            for k, i in enumerate(live):
                got[i].append(out[k:k + 1].float().cpu())
                at[i] += 1
                if at[i] == len(reqs[i]):
                    e.free_slot(slots[i])                      # a shorter request leaves; its slot may be taken in the next turn
        for i in order:
            close(torch.cat(got[i]), wd.plain(reqs[i]), dtype, f"{name}: request {i} in a batch, turn {turn}")
        e.cache.check()
    e.check_kernels()


@pytest.mark.parametrize("dtype", BOTH)
def test_a_loud_first_token_reaches_far_through_state_and_cache(dtype):
    """The first token's embedding is made loud: every later position feels it, through the recurrence's state and through
    the attention's first key, in a prompt and when decoded token by token."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg = make_config("mix")
    w = P.random_weights(cfg, 5)
    toks = random_tokens(200, cfg["vocab"], 77)
    toks[0] = 3
    assert 3 not in toks[1:]
    w["embed"][3] *= 6.0
    want = P.forward(cfg, w, toks).float()
    quiet = dict(w, embed=w["embed"].clone())
    quiet["embed"][3] /= 6.0
    # (the float32 run is the one that can tell: what the first token adds at the last position is below bfloat16's rounding)
    assert rel_l2(P.forward(cfg, quiet, toks).float()[-1], want[-1]) > 20 * TOL["float32"], "the first token does not reach the last position"
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=1024, max_slots=2)
    close(run_in_pieces(e, toks, [len(toks)]), want, dtype, "whole")
    close(run_in_pieces(e, toks, [100]), want, dtype, "decoded from 100")


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding(dtype):
    """A short prompt, then 400 single tokens over several pages (captured steps where the engine captures them)."""
    wd = world("mix")
    toks = random_tokens(420, wd.cfg["vocab"], 123)
    e = wd.engine(dtype)
    got = run_in_pieces(e, toks, [20])
    close(got, wd.plain(toks), dtype, "long decoding")
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
            logits = P.forward(wd.cfg, wd.weights, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break                                           # a near tie: float32 and float64 may differ from here
            seq.append(int(logits.argmax()))
        n = len(seq) - len(p)
        assert list(r.tokens)[:n] == seq[len(p):], f"{name}: generation differs"
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
    """bin/trace_run on a model folder whose description leaves the decay's rank to the tensor's shape."""
    cfg = make_config("odd")
    weights = P.random_weights(cfg, 9)
    stored = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    folder = write_folder(str(tmp_path / "model"), cfg, stored)
    a, b = random_tokens(70, cfg["vocab"], 1), random_tokens(21, cfg["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:20], "want": [19]}], "end": []}]
    for i in range(10):
        es = [{"id": "a", "tokens": [a[60 + i]], "want": [0]}]
        if i == 0:
            es.append({"id": "b", "tokens": [b[20]], "want": [0]})
        steps.append({"step": i + 1, "entries": es, "end": ["b"] if i == 0 else []})
    # then many short requests at once: each holds a page of its own, far more pages than --max-tokens / 64
    many = [random_tokens(3, cfg["vocab"], 30 + i) for i in range(20)]
    steps.append({"step": 11, "entries": [{"id": f"m{i}", "tokens": m[:2], "want": []} for i, m in enumerate(many)], "end": []})
    steps.append({"step": 12, "entries": [{"id": f"m{i}", "tokens": m[2:], "want": [0]} for i, m in enumerate(many)], "end": [f"m{i}" for i in range(20)]})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "192"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(13)]
    cfg_full = make_config("odd")
    pa, pb = P.forward(cfg_full, weights, a).float(), P.forward(cfg_full, weights, b).float()
    V = cfg["vocab"]
    first = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V))
    rows_close(first, torch.stack([pa[0], pa[59], pb[19]]), "float32", "step 0")
    one = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V))
    rows_close(one, torch.stack([pa[60], pb[20]]), "float32", "step 1")
    last = torch.from_numpy(np.fromfile(out / "10.f32", dtype="<f4").reshape(-1, V))
    rows_close(last, pa[69:70], "float32", "step 10")
    short = torch.from_numpy(np.fromfile(out / "12.f32", dtype="<f4").reshape(-1, V))
    rows_close(short, torch.stack([P.forward(cfg_full, weights, m).float()[2] for m in many]), "float32", "twenty short requests")


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
    """A configuration drawn at random: sizes, head counts, layer order, options and constants, odd sizes included."""
    import random
    from zadinex_cases import attention, dense, model, moe, wkv
    r = random.Random(seed)
    width = r.choice([24, 40, 56, 72, 100, 136])
    blend = None                                              # (kv heads, value width) that blending layers share
    layers = []
    for i in range(r.randint(2, 5)):
        if r.random() < 0.6:
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 4])
            dim = r.choice([6, 8, 12, 16, 20, 32, 40, 64])
            vdim = r.choice([dim, dim, 8, 24, 16])
            v_mix = r.random() < 0.6
            if v_mix:
                if blend is None:
                    blend = (kv, vdim)
                kv, vdim = blend
                heads = kv * r.choice([1, 2, 4])
            rot = r.choice([d for d in (2, 4, 6, 8, 16, 32, 64) if d <= dim])
            mixer = attention(heads, kv, dim, vdim, rot, base=r.choice([100.0, 1e4, 5e5]), scale=r.choice([0.1, 0.3, dim ** -0.5]), v_mix=v_mix)
        else:
            mixer = wkv(r.choice([1, 2, 3, 5]), r.choice([4, 8, 12, 24, 48, 72]), r.choice([1, 4, 7, 16]))
        kind = r.choice(["dense", "moe", "moe", "none"])
        if kind == "dense":
            mlp = dense(r.choice([16, 33, 64, 100]))
        elif kind == "moe":
            groups = r.choice([1, 2, 3, 4])
            per = r.choice([1, 2, 3])
            n_all = groups * per
            identity = r.randint(0, n_all - 1)
            keep = r.randint(1, groups)
            mlp = moe(n_all - identity, r.randint(1, keep * per), r.choice([8, 12, 32]), r.choice([0.5, 1.5, 4.0]), identity=identity,
                      groups=(groups, keep) if r.random() < 0.8 or groups > 1 else None)
        else:
            mlp = None
        layers.append(dict(mixer, mlp=mlp))
    return model(layers, width=width, vocab=r.choice([50, 97, 300]), eps=r.choice([1e-6, 1e-5, 1e-4]))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("seed", range(int(os.environ.get("ZADINEX_DRAWN", "12"))))
def test_configurations_drawn_at_random(seed, dtype):
    """A prompt whole, then a second request as a prompt with single tokens after it, in a batch with a third."""
    from titan_b200 import Engine, StepEntry
    from titan_b200.config import config_from_dict
    cfg = drawn_config(seed)
    w = P.random_weights(cfg, 100 + seed)
    e = Engine.from_tensors(config_from_dict(cfg), w, dtype=dtype, max_tokens=1024, max_slots=4, mark_freed_pages=True)
    a, b, c = (random_tokens(n, cfg["vocab"], 7 * seed + n) for n in (75, 130, 9))
    close(run_in_pieces(e, a, [len(a)]), P.forward(cfg, w, a).float(), dtype, f"seed {seed}: whole")
    sb, sc = e.alloc_slot(), e.alloc_slot()
    got_b = [e.step([StepEntry(sb, b[:66], list(range(66))), StepEntry(sc, c[:8], [])])[:66]]
    got_b.append(e.step([StepEntry(sb, [b[66]], [0]), StepEntry(sc, [c[8]], [])]))
    e.free_slot(sc)
    for t in b[67:]:
        got_b.append(e.step([StepEntry(sb, [t], [0])]))
    e.free_slot(sb)
    close(torch.cat(got_b).float().cpu(), P.forward(cfg, w, b).float(), dtype, f"seed {seed}: prompt in a batch, then single tokens")
    e.check_kernels()
    e.cache.check()
