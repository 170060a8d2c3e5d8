"""The Tefezen design in the engine against the plain implementation (tests/plain/tefezen_plain.py): every mechanism
alone, then whole models under every way of cutting the work.  Needs a B200; float32 (true 32-bit) and bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL, random_tokens, rel_l2, rows_close, write_folder
from plain import tefezen_plain as P
from tefezen_cases import make_config

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = ["float32", "bfloat16"]


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def make_ctx(entries, starts, dtype, options=None):
    from titan_b200 import kernels as K
    from titan_b200.engine.batch import StepContext, StepLayout
    lay = StepLayout(entries, starts, "cuda")
    return StepContext(lay, K.current_stream(), dtype, torch.device("cuda"), dict(options or {}), {})


def bind(part, weights, dtype, prefix=""):
    from titan_b200.weights import held_dtype
    specs = {w.name: w for w in part.weight_specs(prefix)}
    part.bind(lambda rel: weights[prefix + rel].to("cuda", held_dtype(specs[prefix + rel].role, dtype)).contiguous())


def weights_for(part, seed, prefix=""):
    """bfloat16-representable random tensors for a part's declaration: matrices ~ N(0, 1/fan_in), vectors around one
    (or around zero, where the part says so)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for w in part.weight_specs(prefix):
        t = torch.randn(w.shape, generator=g)
        if w.role == "vector":
            t = t * 0.2 + (1.0 if w.init[0] == "one_plus_normal" else 0.0)
        else:
            t = t / (w.shape[-1] ** 0.5)
        out[w.name] = t.to(torch.bfloat16).float()
    return out


def close(got, want, dtype, what=""):
    """float32: the tensor and every row within the bound.  bfloat16: a token whose router logits nearly tie may take
    another expert than the plain implementation (with one expert a token: another feed-forward altogether), which moves
    that row and, through the state, some after it by more than rounding does; so the typical row must be within the
    bound and five in six within four times the bound.  Row by row, bfloat16 is held to its bound where no router
    decides: in the tests of the mechanisms alone."""
    if dtype == "float32":
        return rows_close(got, want, dtype, what)
    g, w = got.double().cpu().reshape(-1, got.shape[-1]), want.double().reshape(-1, want.shape[-1])
    assert g.shape == w.shape, what
    per_row = (g - w).norm(dim=1) / w.norm(dim=1).clamp_min(1e-30)
    assert float(per_row.median()) < TOL[dtype], f"{what}: median row error {float(per_row.median()):.3e}"
    if len(per_row) >= 6:
        assert float((per_row < 4 * TOL[dtype]).double().mean()) >= 5 / 6, f"{what}: too many rows over four times the bound"


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


LENGTHS = {"small": [150, 9, 66, 1], "odd": [210, 64, 3, 129], "bare": [70, 200, 17, 2]}
_worlds = {}


def world(name):
    if name not in _worlds:
        _worlds[name] = World(name, {"small": 1, "odd": 2, "bare": 3, "window": 4}[name], LENGTHS.get(name, [10]))
    return _worlds[name]


MODELS = [(n, d) for n in ("small", "odd", "bare") for d in BOTH]


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


# --------------------------------------------------------------------------- #
# mechanisms alone
# --------------------------------------------------------------------------- #
def latent_spec(H, dn, rd, dv, r, window, rot_dims, scale, cache_window=None):
    from titan_b200.config import MixerSpec, NormSpec, PositionSpec
    return MixerSpec("latent_attention", 40, H, 1, dn, window=window, softmax_scale=scale, prefix="mix.",
                     position=PositionSpec("rope", rot_dims, 300.0, "adjacent"),
                     extra=(("rot_dim", rd), ("value_dim", dv), ("kv_rank", r), ("cache_window", cache_window or window),
                            ("latent_norm", NormSpec("rmsnorm", r, 1e-5, "dkv.norm"))))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dn,rd,dv,r,window,rot_dims", [
    (3, 16, 8, 24, 20, 20, 8),         # a ring of one page that long sequences go round several times
    (2, 8, 6, 8, 27, 64, 2),           # sizes that are no multiples of 8; a window of exactly one page; four unrotated dims
    (1, 24, 16, 16, 300, 130, 16),     # rows wider than 256: the attention kernels' wide instantiation
    (3, 128, 64, 128, 96, 70, 64),     # the sizes whose whole prompts, in bfloat16, expand keys and values and take the tensor-core kernel
])
def test_latent_attention_alone(dtype, H, dn, rd, dv, r, window, rot_dims):
    """Prompts of two sequences, a further portion (on a ring: its rows are appended after the step), then single
    tokens far beyond the window; sharp scores, so that one key more or less shows."""
    from titan_b200.cache import SequenceCache
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import MIXERS
    spec = latent_spec(H, dn, rd, dv, r, window, rot_dims, scale=0.5)
    mixer = MIXERS.build(spec)
    w = weights_for(mixer, 3)
    bind(mixer, w, DT[dtype])
    m = {"heads": H, "dim": dn, "rot_dim": rd, "vdim": dv, "kv_rank": r, "mask": {"size": window}, "rot": {"base": 300.0, "dims": rot_dims}, "scale": 0.5}
    lens = [230, 90]
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, 40, generator=g).to(torch.bfloat16).double() for n in lens]
    W = {k: v.double() for k, v in w.items()}
    want = []
    for x in xs:
        pos = torch.arange(x.shape[0])
        want.append(P.latent_attention(x, m, W, "mix.", 1e-5, pos, P.latent_kv(x, m, W, "mix.", 1e-5, pos)).float())
    cache = SequenceCache([mixer.cache_need()], 1024, 4, 512, DT[dtype], "cuda", mark_freed=True)
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    at, got = [0, 0], [[], []]
    for sizes in ([70, 33], [50, 2], [9, 7]):
        live = [i for i in range(2) if at[i] < lens[i]]
        cache.reserve({slots[i]: at[i] + sizes[i] for i in live})
        ctx = make_ctx([StepEntry(slots[i], [0] * sizes[i], []) for i in live], [at[i] for i in live], DT[dtype])
        h = torch.cat([xs[i][at[i]:at[i] + sizes[i]] for i in live]).to(DT[dtype]).cuda()
        out = torch.zeros(h.shape[0], 40, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        for late in ctx.after_blocks:
            late()
        o = 0
        for i in live:
            got[i].append(out[o:o + sizes[i]].cpu())
            o += sizes[i]
            at[i] += sizes[i]
            cache.commit(slots[i], at[i])
    while any(a < n for a, n in zip(at, lens)):
        live = [i for i in range(2) if at[i] < lens[i]]
        cache.reserve({slots[i]: at[i] + 1 for i in live})
        ctx = make_ctx([StepEntry(slots[i], [0], []) for i in live], [at[i] for i in live], DT[dtype])
        h = torch.stack([xs[i][at[i]] for i in live]).to(DT[dtype]).cuda()
        out = torch.zeros(len(live), 40, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1].cpu())
            at[i] += 1
            cache.commit(slots[i], at[i])
    for i in range(2):
        rows_close(torch.cat(got[i]), want[i], dtype, f"sequence {i}", row_factor=6.0)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,dk,dv,decay", [(3, 8, 16, [0.3, 0.9, 1.0]), (1, 40, 33, [0.999]), (2, 130, 70, [0.95, 0.99]),
                                            (2, 64, 24, [0.9, 0.97]), (1, 136, 40, [0.99]), (1, 128, 128, [0.98])])     # the last three: sizes in multiples of 8, the kernel of 16-byte loads
def test_lightning_alone(dtype, H, dk, dv, decay):
    """Two sequences through whole prompts, portions of two tokens and single tokens: outputs and the final state."""
    from titan_b200.cache import SequenceCache
    from titan_b200.config import MixerSpec, NormSpec
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import MIXERS
    spec = MixerSpec("lightning", 32, H, head_dim=dk, prefix="mix.",
                     extra=(("value_dim", dv), ("decay", tuple(decay)), ("out_norm", NormSpec("rmsnorm", H * dv, 1e-6, "norm"))))
    mixer = MIXERS.build(spec)
    w = weights_for(mixer, 11)
    bind(mixer, w, DT[dtype])
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": decay}
    W = {k: v.double() for k, v in w.items()}
    lens = [120, 41]
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(n, 32, generator=g).to(torch.bfloat16).double() for n in lens]
    want = [P.lightning(x, m, W, "mix.", 1e-6) for x in xs]
    cache = SequenceCache([mixer.cache_need()], 512, 3, 512, DT[dtype], "cuda")
    spare = cache.alloc_slot()                                   # so that the sequences do not sit in slot 0
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    at, got = [0, 0], [[], []]
    plan = [[60, 7], [2, 2], [2, 1], [1, 1], [30, 2]] + [[1, 1]] * 40
    for sizes in plan:
        live = [i for i in range(2) if at[i] < lens[i]]
        if not live:
            break
        sizes = [min(sizes[i], lens[i] - at[i]) for i in range(2)]
        ctx = make_ctx([StepEntry(slots[i], [0] * sizes[i], []) for i in live], [at[i] for i in live], DT[dtype])
        h = torch.cat([xs[i][at[i]:at[i] + sizes[i]] for i in live]).to(DT[dtype]).cuda()
        out = torch.zeros(h.shape[0], 32, device="cuda")
        mixer.forward(h, ctx, cache.view_for_layer(0), out)
        o = 0
        for i in live:
            got[i].append(out[o:o + sizes[i]].cpu())
            o += sizes[i]
            at[i] += sizes[i]
    assert at == lens
    state = cache.groups[0].layer_storage(0)
    for i in range(2):
        rows_close(torch.cat(got[i]), want[i][0].float(), dtype, f"sequence {i}", row_factor=6.0)
        assert rel_l2(state[slots[i]].cpu(), want[i][1].float()) < TOL[dtype]
    assert float(state[spare].abs().sum()) == 0.0                # a slot that took no token keeps a zero state


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top,F,shared,T", [(5, 2, 24, 16, 1), (4, 1, 10, 0, 7), (3, 3, 18, 40, 33), (9, 4, 12, 8, 200), (70, 6, 8, 0, 50)])
def test_mixture_of_experts_alone(dtype, E, top, F, shared, T):
    """Few pairs (a warp per output) and many (grouped by expert); one expert a token, all experts a token, more experts
    than a warp has lanes; with and without the expert that every token uses."""
    from titan_b200.config import FeedForwardSpec
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import FEED_FORWARDS
    spec = FeedForwardSpec("moe", 48, F, prefix="mlp.", extra=(("experts", E), ("top", top), ("shared_size", shared)))
    part = FEED_FORWARDS.build(spec)
    w = weights_for(part, 21)
    bind(part, w, DT[dtype])
    f = {"expert": {"ff": F}, "router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    h = torch.randn(T, 48, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    W = {k: v.double() for k, v in w.items()}
    want = P.mixture_of_experts(h.double(), f, W, "mlp.").float()
    ctx = make_ctx([StepEntry(0, [0] * T, [])], [0], DT[dtype])
    out = torch.full((T, 48), 0.25, device="cuda")               # the part adds into what is there
    part.forward(h.to(DT[dtype]).cuda(), ctx, out)
    rows_close(out.cpu() - 0.25, want, dtype, "mixture", row_factor=6.0)


def test_routing_kernel_choices_and_weights():
    from titan_b200 import kernels as K
    g = torch.Generator().manual_seed(8)
    for E, top, gate in ((6, 2, True), (40, 5, False), (3, 3, True), (129, 1, False)):
        z = torch.randn(37, E + int(gate), generator=g)
        z[5, :E] = 0.5                                            # a row of equal logits: the lowest indices are taken
        ids = torch.empty(37, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(37, top, device="cuda")
        sg = torch.empty(37, device="cuda") if gate else None
        K.moe_route(z.cuda(), E, top, gate, ids, wts, sg, K.current_stream())
        want = torch.topk(z[:, :E], top, dim=-1)
        rows = [i for i in range(37) if i != 5]
        assert torch.equal(ids.cpu()[rows].long(), want.indices[rows])
        assert torch.allclose(wts.cpu()[rows], torch.softmax(want.values[rows], dim=-1), atol=1e-6)
        assert ids.cpu()[5].tolist() == list(range(top)) and torch.allclose(wts.cpu()[5], torch.full((top,), 1.0 / top))
        if gate:
            assert torch.allclose(sg.cpu(), torch.sigmoid(z[:, E]), atol=1e-6)


@pytest.mark.parametrize("dtype", BOTH)
def test_token_table_input_and_output_norm_block(dtype):
    """A block of the output-norm arrangement with a lightning mixer, no feed-forward and a token-table sublayer,
    against its formula; twice in a row, so that the rounded rows one block leaves are what the next one reads."""
    from titan_b200.cache import SequenceCache
    from titan_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec
    from titan_b200.engine.batch import StepEntry
    from titan_b200.parts import build_block
    Wd, V, D = 40, 30, 6
    mixer = MixerSpec("lightning", Wd, 2, head_dim=8, prefix="mix.", extra=(("value_dim", 12), ("decay", (0.8, 0.99)), ("out_norm", NormSpec("rmsnorm", 24, 1e-5, "norm"))))
    blocks, weights = [], {}
    for i in range(2):
        side = FeedForwardSpec("token_table", Wd, D, "gelu_tanh", prefix="side.", extra=(("table", "tab"), ("offset", 3 + i * D)))
        spec = LayerSpec(i, "output_norm", mixer, None, NormSpec("rmsnorm", Wd, 1e-5, "norm1", 1.0), None, f"b{i}.",
                         norms=(NormSpec("rmsnorm", Wd, 1e-5, "side.norm"),), extra=(("sublayers", (side,)),))
        b = build_block(spec)
        w = weights_for(b, 30 + i)
        bind(b, w, DT[dtype])
        weights.update(w)
        blocks.append(b)
    table = torch.randn(V, 3 + 2 * D + 2, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    for b in blocks:
        b.bind_shared({"tab": table.to("cuda", DT[dtype])})
    tokens = random_tokens(25, V, 3)
    x0 = torch.randn(25, Wd, generator=torch.Generator().manual_seed(4))
    W = {k: v.double() for k, v in weights.items()}
    x = x0.double()
    for i in range(2):
        p = f"b{i}."
        y, _ = P.lightning(x, {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.8, 0.99]}, W, p + "mix.", 1e-5)
        x = x + P.norm_around_zero(y, W[p + "norm1"], 1e-5)
        e = table.double()[torch.tensor(tokens)][:, 3 + i * D: 3 + (i + 1) * D]
        y = P.lin(P.gelu_tanh(P.lin(x, W[p + "side.gate"])) * e, W[p + "side.proj"])
        x = x + P.norm_plain(y, W[p + "side.norm"], 1e-5)
    cache = SequenceCache([blocks[0].mixer.cache_need(), blocks[1].mixer.cache_need()], 64, 2, 64, DT[dtype], "cuda")
    slot = cache.alloc_slot()
    ctx = make_ctx([StepEntry(slot, tokens, [])], [0], DT[dtype])
    xg = x0.clone().cuda()
    for i, b in enumerate(blocks):
        ctx.run = i
        b.forward(xg, ctx, cache.view_for_layer(i))
    rows_close(xg.cpu(), x.float(), dtype, "two blocks")


def test_norm_add_kernel_and_batched_product():
    from titan_b200 import kernels as K
    g = torch.Generator().manual_seed(12)
    y, w, x = torch.randn(9, 77, generator=g), torch.randn(77, generator=g), torch.randn(9, 77, generator=g)
    want = x + y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-3) * w
    yd, xd, low = y.cuda(), x.cuda(), torch.empty(9, 77, dtype=torch.bfloat16, device="cuda")
    K.rmsnorm_add(yd, w.cuda(), xd, 1e-3, K.current_stream(), lowp=low, zero_y=True)
    assert torch.allclose(xd.cpu(), want, atol=1e-5) and float(yd.abs().sum()) == 0.0
    assert torch.equal(low.cpu(), xd.cpu().to(torch.bfloat16))
    # three heads side by side in the rows of one buffer, each with its own matrix
    for dt in (torch.float32, torch.bfloat16):
        a = torch.randn(50, 3 * 10 + 4, generator=g).to(dt)
        m = torch.randn(3, 7, 10, generator=g).to(dt)
        out = torch.zeros(50, 3 * 9, dtype=dt, device="cuda")
        K.gemm_simt_batched(a.cuda()[:, :10], m.cuda(), out[:, :7], K.EPI_STORE, K.current_stream(), 3, 10, 9)
        for hd in range(3):
            ref = a[:, hd * 10: hd * 10 + 10].float() @ m[hd].float().t()
            assert rel_l2(out[:, hd * 9: hd * 9 + 7].float().cpu(), ref) < (1e-5 if dt == torch.float32 else 1e-2)
            assert float(out[:, hd * 9 + 7: hd * 9 + 9].abs().sum()) == 0.0        # the gap between heads is not written


def test_products_and_token_gate_of_a_few_rows():
    """The warp-per-output kernels of a decode step: a small product with each of its epilogues, and the token gate with
    its product, at widths that 16-byte loads take and at odd ones."""
    from titan_b200 import kernels as K
    g = torch.Generator().manual_seed(14)
    st = K.current_stream()
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        for M, N, Kd in ((1, 33, 64), (5, 7, 50), (8, 130, 136)):
            x, w = torch.randn(M, Kd, generator=g).to(dt), torch.randn(N, Kd, generator=g).to(dt)
            ref = x.float() @ w.float().t()
            out = torch.empty(M, N, dtype=dt, device="cuda")
            K.gemm_rows(x.cuda(), w.cuda(), out, K.EPI_STORE, st)
            assert rel_l2(out.float().cpu(), ref) < tol
            out32 = torch.full((M, N + 3), 2.0, device="cuda")
            K.gemm_rows(x.cuda(), w.cuda(), out32[:, :N], K.EPI_F32, st)
            assert rel_l2(out32[:, :N].cpu(), ref) < 1e-5 and float((out32[:, N:] - 2.0).abs().sum()) == 0.0
            K.gemm_rows(x.cuda(), w.cuda(), out32[:, :N], K.EPI_ADD, st)
            assert rel_l2(out32[:, :N].cpu(), 2 * ref) < 1e-5
        for T, D, Kd, off in ((1, 16, 64, 0), (3, 5, 50, 4)):
            x, w = torch.randn(T, Kd, generator=g).to(dt), (torch.randn(D, Kd, generator=g) / Kd ** 0.5).to(dt)
            table = torch.randn(11, off + D + 2, generator=g).to(dt)
            tokens = torch.tensor([10, 0, 3][:T], dtype=torch.int32)
            ref = P.gelu_tanh(x.double() @ w.double().t()) * table.double()[tokens.long()][:, off:off + D]
            out = torch.empty(T, D, dtype=dt, device="cuda")
            K.token_gate_rows(x.cuda(), w.cuda(), table.cuda(), tokens.cuda(), off, out, st)
            assert rel_l2(out.float().cpu(), ref.float()) < tol


# --------------------------------------------------------------------------- #
# whole models
# --------------------------------------------------------------------------- #
@pytest.mark.parametrize("name,dtype", MODELS)
def test_whole_prompts_each_alone(name, dtype):
    w = world(name)
    e = w.engine(dtype)
    for toks in w.requests:
        close(run_in_pieces(e, toks, [len(toks)]), w.plain(toks), dtype, f"{name}: {len(toks)} tokens")
    e.check_kernels()
    e.cache.check()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_prompt_then_token_by_token_and_all_by_single_tokens(name, dtype):
    """A prompt, then up to 150 single tokens (over page borders, and round the ring of every window); and a sequence
    fed one token at a time from its first token on."""
    w = world(name)
    e = w.engine(dtype)
    long = max(w.requests, key=len)
    close(run_in_pieces(e, long, [max(1, len(long) - 150)]), w.plain(long), dtype, f"{name}: prompt then single tokens")
    short = w.requests[2] if len(w.requests[2]) > 1 else w.requests[1]
    close(run_in_pieces(e, short, []), w.plain(short), dtype, f"{name}: single tokens only")


@pytest.mark.parametrize("name,dtype", MODELS)
def test_portions_of_several_sizes(name, dtype):
    w = world(name)
    e = w.engine(dtype)
    toks = max(w.requests, key=len)
    for pieces in ([64, 64, 2, 2, 3, 40], [2] * 40 + [63, 1, 1, 30], [129, 7]):
        close(run_in_pieces(e, toks, pieces), w.plain(toks), dtype, f"{name}: portions {pieces[:4]}")
    e.cache.check()


@pytest.mark.parametrize("name,dtype", MODELS)
def test_a_batch_of_unequal_requests_against_each_alone(name, dtype):
    """All requests start together with prompts of unequal length and go on together one token each; the shorter ones
    leave earlier.  Every row must match the plain implementation, and, in float32, the same request run alone
    to within rounding."""
    from titan_b200 import StepEntry
    w = world(name)
    e = w.engine(dtype)
    reqs = w.requests
    first = [max(1, len(t) - 12 - 3 * i) for i, t in enumerate(reqs)]
    slots = [e.alloc_slot() for _ in reqs]
    out = e.step([StepEntry(s, t[:n], list(range(n))) for s, t, n in zip(slots, reqs, first)])
    got, o = [], 0
    for n in first:
        got.append([out[o:o + n]])
        o += n
    at = list(first)
    for i, t in enumerate(reqs):
        if at[i] == len(t):
            e.free_slot(slots[i])                                  # its prompt was all of it
    while any(a < len(t) for a, t in zip(at, reqs)):
        live = [i for i in range(len(reqs)) if at[i] < len(reqs[i])]
        out = e.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1])
            at[i] += 1
            if at[i] == len(reqs[i]):
                e.free_slot(slots[i])
    for i, t in enumerate(reqs):
        mine = torch.cat(got[i]).float().cpu()
        close(mine, w.plain(t), dtype, f"{name}: request {i} in the batch")
        if dtype == "float32":
            alone = run_in_pieces(e, t, [first[i]])
            assert rel_l2(mine, alone) < 2e-5
    e.cache.check()


@pytest.mark.parametrize("dtype", BOTH)
def test_slots_pages_and_states_are_used_again(dtype):
    """A small cache: requests come and go, so every slot, page and state is handed out again (freed pages are
    overwritten with a large value, and a state that was not cleared would carry the former sequence on)."""
    from titan_b200 import StepEntry
    w = world("small")
    e = w.engine(dtype, max_tokens=320, max_slots=2)
    for round_ in range(3):
        for toks in (w.requests[0], w.requests[2], w.requests[1]):
            close(run_in_pieces(e, toks, [max(1, len(toks) - 5)]), w.plain(toks), dtype, f"round {round_}")
    a, b = e.alloc_slot(), e.alloc_slot()
    e.step([StepEntry(a, w.requests[2], []), StepEntry(b, w.requests[1], [])])
    e.free_slot(a)
    c = e.alloc_slot()
    assert c == a
    out = e.step([StepEntry(c, w.requests[0][:100], list(range(100)))])
    close(out.float().cpu(), w.plain(w.requests[0])[:100], dtype, "a slot used again beside a live one")
    e.free_slot(b), e.free_slot(c)
    e.cache.check()


@pytest.mark.parametrize("dtype", BOTH)
def test_window_edges_in_prompts_and_in_decoding(dtype):
    """One latent-attention layer: a position's logits depend on the tokens inside its window only.  Two sequences
    that differ in ONE token j, which in the second is a token with a loud embedding (its unnormed rotated key part makes
    its scores stand out; of a few such tokens the one that the plain implementation says moves the last position that sees
    it most): the logits differ up to position j + window - 1, there by what the plain implementation says, and are equal
    from j + window on; in a prompt and in single-token steps, with j at a page's border and not."""
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    cfg = make_config("window")
    V = cfg["vocab"]
    weights = P.random_weights(cfg, 4)
    loud = list(range(V - 8, V))
    for t in loud:
        weights["embed"][t] = (weights["embed"][t].float() * 5).to(torch.bfloat16)
    e = Engine.from_tensors(config_from_dict(cfg), weights, dtype=dtype, max_tokens=1024, max_slots=2, mark_freed_pages=True)
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    base = [t % (V - 8) for t in random_tokens(200, V, 77)]
    pa = P.forward(cfg, weights, base).float()
    for j in (0, 63, 64, 101):
        inside, outside = j + window - 1, j + window
        gap, other, pb = 0.0, None, None
        for t in loud:
            cand = list(base)
            cand[j] = t
            pc = P.forward(cfg, weights, cand).float()
            g = float((pa[inside] - pc[inside]).norm() / pa[inside].norm())
            if g > gap:
                gap, other, pb = g, cand, pc
        assert gap > 0.05, f"the test is blunt: the last position that sees token {j} moves by {gap:.3f} only"
        assert float((pa[outside:] - pb[outside:]).abs().max()) < 1e-9
        for pieces in ([200], [j + 1], [max(1, j - 2)]):
            ga, gb = run_in_pieces(e, base, pieces), run_in_pieces(e, other, pieces)
            close(ga, pa, dtype, f"token {j}: base")
            close(gb, pb, dtype, f"token {j}: changed")
            assert rel_l2(ga[inside] - gb[inside], pa[inside] - pb[inside]) < (1e-3 if dtype == "float32" else 0.5)
            assert float((ga[outside:] - gb[outside:]).abs().max()) <= (1e-5 if dtype == "float32" else 5e-2)


@pytest.mark.parametrize("dtype", BOTH)
def test_a_token_far_back_reaches_through_the_state(dtype):
    """A model of lightning layers with slow decays: a FIRST token with a loud embedding moves the logits hundreds of
    positions later, by the plain implementation; the engine follows, in a prompt and in decoding."""
    from tefezen_cases import lightning, model, moe, with_mlp
    cfg = model([with_mlp(lightning(2, 16, 16, [1.0, 0.999]), moe(3, 1, 16)), dict(lightning(2, 8, 24, [0.9995, 0.5]), mlp=None)],
                width=32, vocab=50, eps=1e-5)
    weights = P.random_weights(cfg, 9)
    weights["embed"][49] = (weights["embed"][49].float() * 8).to(torch.bfloat16)
    from titan_b200 import Engine
    from titan_b200.config import config_from_dict
    e = Engine.from_tensors(config_from_dict(cfg), weights, dtype=dtype, max_tokens=1024, max_slots=2)
    a = [t % 49 for t in random_tokens(400, 50, 5)]
    b = [49] + a[1:]
    pa, pb = P.forward(cfg, weights, a).float(), P.forward(cfg, weights, b).float()
    gap = float((pa[399] - pb[399]).norm() / pa[399].norm())
    assert gap > 0.5, f"the test is blunt: position 399 moves by {gap:.3f} only"
    for pieces in ([400], [340]):
        ga, gb = run_in_pieces(e, a, pieces), run_in_pieces(e, b, pieces)
        close(ga, pa, dtype, "base"), close(gb, pb, dtype, "changed")
        assert rel_l2(ga[399] - gb[399], pa[399] - pb[399]) < (1e-3 if dtype == "float32" else 0.3)


@pytest.mark.parametrize("name", ["small", "odd"])
def test_greedy_generation_through_the_loop_and_captured_steps(name):
    """Engine.generate: prompts of unequal length batched by the scheduler, decode steps replayed from graphs, one
    request leaving early; every token is the plain implementation's choice."""
    from titan_b200 import SamplerParams
    from titan_b200.engine import GenerationRequest, generate
    w = world(name)
    e = w.engine("float32")
    prompts = [w.requests[1][:20], w.requests[0][:70], w.requests[3][:1]]
    budgets = (25, 9, 16)
    before = e.graph_launches
    outs = generate(e, [GenerationRequest(list(p), n, SamplerParams.greedy(), (), False) for p, n in zip(prompts, budgets)])
    assert e.graph_launches > before
    for p, o, n in zip(prompts, outs, budgets):
        assert len(o.tokens) == n
        logits = w.plain(list(p) + o.tokens)
        for k, tok in enumerate(o.tokens):
            row = logits[len(p) - 1 + k]
            assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-3 * float(row.abs().max()), (k, tok)
    e.check_kernels()
    e.cache.check()


def test_generation_in_bfloat16_stays_near_the_plain_choice():
    from titan_b200 import SamplerParams
    w = world("small")
    e = w.engine("bfloat16")
    p = w.requests[2][:30]
    out = e.generate([p], max_tokens=20, params=SamplerParams.greedy(), stop_tokens=[])[0].tokens
    logits = w.plain(list(p) + out)
    for k, tok in enumerate(out):
        row = logits[len(p) - 1 + k]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 0.1 * float(row.abs().max())


@pytest.mark.parametrize("dtype", BOTH)
def test_trace_runner_on_a_model_folder(tmp_path, dtype):
    """bin/trace_run as a subprocess on a folder of this design: requests whole, a batch that starts together and decodes
    together, names used again after their request ended."""
    w = world("odd" if dtype == "float32" else "small")          # with one expert a token, bfloat16 takes other experts too often to compare rows
    folder = write_folder(str(tmp_path / "model"), w.cfg, w.weights)
    V = w.cfg["vocab"]
    long = w.requests[0]
    reqs = {"a": long[:90], "b": long[100:140], "c": long[50:120]}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"], "want": list(range(90))}], "end": ["a"]},
             {"step": 1, "entries": [{"id": k, "tokens": t[:30], "want": [29] if k != "b" else []} for k, t in reqs.items()], "end": []}]
    n, at = 2, 30
    while any(at < len(t) for t in reqs.values()):
        live = [k for k, t in reqs.items() if at < len(t)]
        steps.append({"step": n, "entries": [{"id": k, "tokens": [reqs[k][at]], "want": [0]} for k in live],
                      "end": [k for k in live if at == len(reqs[k]) - 1]})
        n, at = n + 1, at + 1
    out = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                        "--max-tokens", "320"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    read = lambda step, rows: torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(rows, V))
    close(read(0, 90), w.plain(reqs["a"]), dtype, "whole")
    close(read(1, 2), torch.stack([w.plain(reqs["a"])[29], w.plain(reqs["c"])[29]]), dtype, "the batch's prompts")
    got = {k: [] for k in reqs}
    for s in steps[2:]:
        rows = read(s["step"], len(s["entries"]))
        for r, en in zip(rows, s["entries"]):
            got[en["id"]].append(r)
    for k, t in reqs.items():
        close(torch.stack(got[k]), w.plain(t)[30:], dtype, f"request {k} decoded")


def test_command_line_generates_from_a_folder_and_from_random_weights(tmp_path):
    """bin/titan_b200 run: a model folder of this design (greedy tokens equal the engine's own), and random weights made from
    its config.json alone."""
    w = world("small")
    folder = write_folder(str(tmp_path / "model"), w.cfg, w.weights)
    prompt = w.requests[1]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "titan_b200"), "run"]
    common = ["--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "7", "-t", "0", "--repetition-penalty", "1.0", "--dtype", "float32", "-c", "256"]
    p = subprocess.run(cmd + ["-m", folder] + common, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    made = json.loads(p.stdout.strip().splitlines()[0])["tokens"]
    assert len(made) == 7
    logits = w.plain(list(prompt) + made)
    for k, tok in enumerate(made):
        row = logits[len(prompt) - 1 + k]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-3 * float(row.abs().max())
    p = subprocess.run(cmd + ["--random", os.path.join(folder, "config.json"), "--weights-seed", "3"] + common, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(json.loads(p.stdout.strip().splitlines()[0])["tokens"]) == 7
