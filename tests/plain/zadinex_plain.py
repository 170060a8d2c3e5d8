"""Plain, slow, whole-sequence forward pass of the Zadinex design on the CPU.

The oracle of the Zadinex tests.  It shares no code with ``titan_b200``: the
configuration is a plain dict, weights are a dict of tensors by their file
names, there is no cache, no batch and no kernel, and every mechanism is one
function.  All arithmetic runs in one dtype (float64 by default, so that the
oracle itself adds no rounding of its own).

Notation.  ``x`` is the residual stream [T, width].  A layer does

    x <- x + s1 * mixer(D1(x));   x <- x + s2 * ff(D2(x))

with D a norm that takes no statistics, D(x) = tanh(a x) * w + b (a a scalar), and s1, s2 vectors that scale each
sublayer's output element by element.  Mixers: ``attention`` (grouped queries, partly rotated heads, unit-RMS heads, a
learned sink in the softmax's denominator, values blended with an earlier layer's) and ``wkv`` (a recurrence with a
decay made from the token, over a state of key x value outer products).  Feed-forwards: a gated dense one, or a mixture
of small experts among which a router with group limits chooses, some of the choices being the input itself.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# --------------------------------------------------------------------------- #
# small pieces
# --------------------------------------------------------------------------- #
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def tanh_norm(x, W, name):
    """D(x) = tanh(a x) * w + b; no mean, no variance."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def lin(x, w):
    """W x for a matrix stored [out, in]."""
    return x @ w.t()


def rotate_halves(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary encoding over the first ``dims`` dimensions of a head, dimension i paired with i + dims/2: at position p the
    pair (a, b) becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims).  v: [T, heads, D]."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = torch.as_tensor(base, dtype=v.dtype) ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]               # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# --------------------------------------------------------------------------- #
# attention
# --------------------------------------------------------------------------- #
def attention_values(h, m, W, p, v_first):
    """The values of this layer [T, kv_heads, vdim]: W_v h, blended with ``v_first`` (the values of the first blending
    layer, same tokens) unless this is that layer (v_first None)."""
    T = h.shape[0]
    v = lin(h, W[p + "v"]).reshape(T, m["kv_heads"], m["vdim"])
    if m.get("v_mix") and v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    return v


def attention(h, m, W, p, eps, positions, v):
    """Causal softmax attention with a sink.  ``v`` are the (blended) values [T, kv_heads, vdim] of these tokens; the
    sequence starts at positions[0] == 0 (the oracle has no cache)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = lin(h, W[p + "q"]).reshape(T, H, D)
    k = lin(h, W[p + "k"]).reshape(T, G, D)
    rot = m["rot"]
    q = unit_rms(rotate_halves(q, positions, rot["base"], rot["dims"]), eps)
    k = unit_rms(rotate_halves(k, positions, rot["base"], rot["dims"]), eps)
    out = torch.zeros(T, H, m["vdim"], dtype=h.dtype)
    causal = positions[None, :] <= positions[:, None]
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].t()) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, W[p + "sink"][hq])
        e = torch.exp(s - top)
        denom = e.sum(dim=-1, keepdim=True) + torch.exp(W[p + "sink"][hq] - top)      # the sink: no key, no value, once
        out[:, hq] = (e / denom) @ v[:, g]
    return lin(out.reshape(T, H * m["vdim"]), W[p + "o"])


# --------------------------------------------------------------------------- #
# the wkv recurrence
# --------------------------------------------------------------------------- #
def wkv(h, m, W, p, eps, state=None):
    """h: [T, width] of ONE sequence in order.  state: None (start) or (S [heads, dim, dim], last h [width]).
    Returns (output [T, width], new state)."""
    T, width = h.shape
    H, D = m["heads"], m["dim"]
    if state is None:
        S, last = torch.zeros(H, D, D, dtype=h.dtype), torch.zeros(width, dtype=h.dtype)
    else:
        S, last = state[0].clone(), state[1].clone()
    before = torch.cat([last[None, :], h[:-1]], dim=0)                 # the token before each token
    mix = lambda s: h + (before - h) * W[p + "mu." + s]
    r = lin(mix("r"), W[p + "r"]).reshape(T, H, D)
    k = lin(mix("k"), W[p + "k"]).reshape(T, H, D)
    v = lin(mix("v"), W[p + "v"]).reshape(T, H, D)
    gate = silu(lin(mix("g"), W[p + "g"]))
    decay = torch.exp(-torch.exp(lin(torch.tanh(lin(mix("w"), W[p + "w1"])), W[p + "w2"]) + W[p + "w0"])).reshape(T, H, D)
    u = W[p + "u"]                                                     # [H, D]
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                       # [H, key, value]
        o[t] = torch.einsum("hij,hi->hj", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    y = unit_rms(o, eps).reshape(T, H * D) * W[p + "norm"] * gate
    return lin(y, W[p + "o"]), (S, h[-1].clone())


# --------------------------------------------------------------------------- #
# feed-forwards
# --------------------------------------------------------------------------- #
def dense_ff(h, W, p):
    return lin(gelu_tanh(lin(h, W[p + "gate"])) * lin(h, W[p + "up"]), W[p + "down"])


def clamped_expert(h, W, p, limit):
    g = torch.clamp(lin(h, W[p + "gate"]), max=limit)
    u = torch.clamp(lin(h, W[p + "up"]), min=-limit, max=limit)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), W[p + "down"])


def routed_choice(h, f, W, p):
    """(indices [T, top], weights [T, top]) over the experts and the identity experts together."""
    r = f["router"]
    n_all = r["experts"] + r.get("identity", 0)
    s = torch.softmax(lin(h, W[p + "router"]), dim=-1)                 # [T, n_all]
    choice = s + W[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = n_all // groups["count"]
    best_of_group = choice.reshape(-1, groups["count"], per).max(dim=-1).values
    kept = torch.topk(best_of_group, groups["keep"], dim=-1).indices   # [T, keep]
    allowed = torch.zeros_like(best_of_group, dtype=torch.bool).scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, n_all)
    idx = torch.topk(choice.masked_fill(~allowed, -math.inf), r["top"], dim=-1).indices
    w = torch.gather(s, 1, idx)
    return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def mixture_of_experts(h, f, W, p):
    r = f["router"]
    E = r["experts"]
    idx, w = routed_choice(h, f, W, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            y = h[t] if e >= E else clamped_expert(h[t][None, :], W, f"{p}e{e}.", f["expert"]["limit"])[0]
            out[t] += w[t, j] * y
    return out


# --------------------------------------------------------------------------- #
# the model
# --------------------------------------------------------------------------- #
def forward(cfg: dict, weights: dict, tokens, dtype=F64, trace=None):
    """Logits [T, vocab] of one sequence from its first token.  ``trace``: a list that receives the residual stream
    after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tok.numel())
    x = W["embed"][tok]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = tanh_norm(x, W, p + "norm1")
        if layer["type"] == "attention":
            v = attention_values(h, m, W, p + "mix.", v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
            y = attention(h, m, W, p + "mix.", eps, positions, v)
        else:
            y, _ = wkv(h, m, W, p + "mix.", eps)
        x = x + W[p + "ls1"] * y
        f = layer.get("mlp")
        if f is not None:
            h = tanh_norm(x, W, p + "norm2")
            y = dense_ff(h, W, p + "mlp.") if f["kind"] == "dense" else mixture_of_experts(h, f, W, p + "mlp.")
            x = x + W[p + "ls2"] * y
        if trace is not None:
            trace.append(x.clone())
    return lin(tanh_norm(x, W, "final.norm"), W["head"])


def tensor_list(cfg: dict):
    """(name, shape, kind) of every tensor of a model; kind says how random weights are drawn."""
    Wd, V = cfg["width"], cfg["vocab"]
    out = [("embed", (V, Wd), "embed")]
    norm = lambda n: [(n, (Wd,), "norm_w"), (n + ".b", (Wd,), "bias"), (n + ".alpha", (), "alpha")]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out += norm(p + "norm1")
        if layer.get("mlp") is not None:
            out += norm(p + "norm2")
        q = p + "mix."
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out += [(q + "q", (H * D, Wd), "matrix"), (q + "k", (G * D, Wd), "matrix"), (q + "v", (G * Dv, Wd), "matrix"),
                    (q + "sink", (H,), "sink"), (q + "o", (Wd, H * Dv), "matrix")]
            if m.get("v_mix"):
                out.append((q + "vmix", (), "lambda"))
        else:
            H, D = m["heads"], m["dim"]
            N = H * D
            rank = m.get("rank", 8)
            out += [(q + "mu." + s, (Wd,), "mu") for s in "rkvgw"]
            out += [(q + s, (N, Wd), "matrix") for s in "rkvg"]
            out += [(q + "w1", (rank, Wd), "matrix"), (q + "w2", (N, rank), "matrix_in_rank"), (q + "w0", (N,), "decay"),
                    (q + "u", (H, D), "bonus"), (q + "norm", (N,), "norm_w"), (q + "o", (Wd, N), "matrix")]
        f = layer.get("mlp")
        if f is not None:
            q = p + "mlp."
            if f["kind"] == "dense":
                out += [(q + "gate", (f["ff"], Wd), "matrix"), (q + "up", (f["ff"], Wd), "matrix"), (q + "down", (Wd, f["ff"]), "matrix_ff")]
            else:
                r = f["router"]
                for e in range(r["experts"]):
                    F = f["expert"]["ff"]
                    out += [(f"{q}e{e}.gate", (F, Wd), "matrix"), (f"{q}e{e}.up", (F, Wd), "matrix"), (f"{q}e{e}.down", (Wd, F), "matrix_ff")]
                n_all = r["experts"] + r.get("identity", 0)
                out += [(q + "router", (n_all, Wd), "router"), (q + "correction", (n_all,), "correction")]
        out += [(p + "ls1", (Wd,), "layer_scale")]
        if f is not None:
            out += [(p + "ls2", (Wd,), "layer_scale")]
    out += norm("final.norm")
    out.append(("head", (V, Wd), "matrix"))
    return out


def random_weights(cfg: dict, seed: int):
    """Random weights, as exact bfloat16 values held in float32, drawn so that every mechanism moves the logits."""
    g = torch.Generator().manual_seed(seed)
    n = lambda shape, std, mean=0.0: torch.randn(shape, generator=g) * std + mean
    W = {}
    for name, shape, kind in tensor_list(cfg):
        fan_in = shape[-1] if len(shape) == 2 else 1
        if kind == "embed":
            t = n(shape, 1.0)
        elif kind in ("matrix", "matrix_ff", "matrix_in_rank"):
            t = n(shape, 1.0 / math.sqrt(fan_in))
        elif kind == "router":
            t = n(shape, 2.0 / math.sqrt(fan_in))
        elif kind == "norm_w":
            t = n(shape, 0.1, 1.0)
        elif kind == "bias":
            t = n(shape, 0.1)
        elif kind == "alpha":
            t = n(shape, 0.05, 0.7)
        elif kind == "sink":
            t = n(shape, 1.0)
        elif kind == "lambda":
            t = torch.rand(shape, generator=g) * 0.6 + 0.2
        elif kind == "mu":
            t = torch.rand(shape, generator=g)
        elif kind == "decay":
            t = n(shape, 1.0, -1.5)
        elif kind == "bonus":
            t = n(shape, 0.5)
        elif kind == "correction":
            t = n(shape, 0.1)
        elif kind == "layer_scale":
            t = n(shape, 0.1, 0.6)
        else:
            raise KeyError(kind)
        W[name] = t.to(torch.bfloat16).to(torch.float32)
    return W
