"""Plain, slow, whole-sequence forward pass of the Tefezen design on the CPU.

The oracle of the Tefezen tests.  It shares no code with ``titan_b200``: the
configuration is a plain dict, weights are a dict of tensors by their file
names, there is no cache, no batch and no kernel, and every mechanism is one
function.  All arithmetic runs in one dtype (float64 by default, so that the
oracle itself adds no rounding of its own).

Notation.  ``x`` is the residual stream [T, width].  A layer does

    x <- x + N1(mixer(x));  x <- x + N2(ff(x));  x <- x + S(side(x, token))

where the sublayers read ``x`` itself and the norms sit on their OUTPUTS.
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


def norm_plain(x, w, eps):
    """RMS norm whose weight multiplies as stored."""
    return unit_rms(x, eps) * w


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def lin(x, w):
    """W x for a matrix stored [out, in]."""
    return x @ w.t()


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary encoding with neighbouring dimensions paired: for i < dims/2 the pair (v[2i], v[2i+1]) turns by
    the angle position * base^(-2i/dims); dimensions from ``dims`` on pass unchanged.  v: [T, ..., D]."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=v.dtype)
    freq = torch.as_tensor(base, dtype=v.dtype) ** (-2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]                  # [T, dims/2]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- #
# mixers
# --------------------------------------------------------------------------- #
def latent_kv(h, m, W, p, eps, positions):
    """What a latent-attention layer caches per token: the normed latent [T, kv_rank] and the rotated shared
    key part [T, rot_dim]."""
    r, rd = m["kv_rank"], m["rot_dim"]
    d = lin(h, W[p + "dkv"])
    c = norm_plain(d[:, :r], W[p + "dkv.norm"], eps)
    kr = rotate_pairs(d[:, r:r + rd], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, m, W, p, eps, positions, kv):
    """Attention whose keys and values are expanded per head from a shared latent; ``kv`` = (latent, rotated key
    part) of this layer or of the layer it borrows them from.  A query at position i sees keys at j with
    0 <= i - j < mask.size."""
    T = h.shape[0]
    H, dn, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = kv
    q = lin(h, W[p + "q"]).view(T, H, dn + rd)
    qn = q[..., :dn]
    qr = rotate_pairs(q[..., dn:], positions, m["rot"]["base"], m["rot"]["dims"])
    kn = lin(c, W[p + "uk"]).view(T, H, dn)
    v = lin(c, W[p + "uv"]).view(T, H, dv)
    score = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    i = positions[:, None]
    j = positions[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    score = score.masked_fill(~seen[None], float("-inf"))
    w = torch.softmax(score, dim=-1)
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * dv)
    return lin(o, W[p + "o"])


def lightning(h, m, W, p, eps, state=None):
    """Linear attention with a per-head decay, token by token: S <- decay_h S + k v^T, o = S^T q; the heads'
    outputs are normed together, gated and projected.  Returns (output, final state [H, dim, vdim])."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(h, W[p + "q"])).view(T, H, dk)
    k = silu(lin(h, W[p + "k"])).view(T, H, dk)
    v = silu(lin(h, W[p + "v"])).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype).view(H, 1, 1)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        rows.append(torch.einsum("hkv,hk->hv", S, q[t]).reshape(H * dv))
    o = torch.stack(rows)
    o = norm_plain(o, W[p + "norm"], eps) * torch.sigmoid(lin(h, W[p + "g"]))
    return lin(o, W[p + "o"]), S


# --------------------------------------------------------------------------- #
# feed-forward
# --------------------------------------------------------------------------- #
def gated_expert(h, W, p):
    return lin(silu(lin(h, W[p + "gate"])) * lin(h, W[p + "up"]), W[p + "down"])


def routed_choice(h, f, W, p):
    """(chosen expert ids [T, top], their weights [T, top]): the largest router logits, softmax over the chosen."""
    z = lin(h, W[p + "router"])
    top = torch.topk(z, f["router"]["top"], dim=-1)
    return top.indices, torch.softmax(top.values, dim=-1)


def mixture_of_experts(h, f, W, p):
    ids, wts = routed_choice(h, f, W, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(ids[t].tolist(), wts[t]):
            out[t] += g * gated_expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + torch.sigmoid(lin(h, W[p + "shared.sg"])) * gated_expert(h, W, p + "shared.")
    return out


# --------------------------------------------------------------------------- #
# per-layer token input
# --------------------------------------------------------------------------- #
def token_side(x, tokens, layer, dim, W, p, eps):
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = lin(gelu_tanh(lin(x, W[p + "gate"])) * e, W[p + "proj"])
    return norm_plain(y, W[p + "norm"], eps)


# --------------------------------------------------------------------------- #
# the model
# --------------------------------------------------------------------------- #
def forward(cfg: dict, weights: dict, tokens, dtype=F64, trace=None, start: int = 0):
    """Logits [T, vocab] of a whole sequence.  ``trace``: a list that receives the residual stream after every
    layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    tok = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(start, start + len(tok))
    eps = cfg["norm"]["eps"]
    x = W["embed"][tok] * (cfg.get("embedding") or {}).get("scale", 1.0)
    side = (cfg.get("token_side") or {}).get("dim")
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_kv(x, m, W, p + "mix.", eps, positions)
            y = latent_attention(x, m, W, p + "mix.", eps, positions, kept[i if src is None else src])
        elif layer["type"] == "lightning":
            y, _ = lightning(x, m, W, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_around_zero(y, W[p + "norm1"], eps)
        if layer.get("mlp"):
            x = x + norm_around_zero(mixture_of_experts(x, layer["mlp"], W, p + "mlp."), W[p + "norm2"], eps)
        if side:
            x = x + token_side(x, tok, i, side, W, p + "side.", eps)
        if trace is not None:
            trace.append(x.clone())
    return lin(norm_around_zero(x, W["final.norm"], eps), W["head"])


# --------------------------------------------------------------------------- #
# tensors of a model of this design: (name, shape, kind), kind in matrix | around_zero | around_one
# --------------------------------------------------------------------------- #
def tensor_list(cfg: dict):
    width, vocab = cfg["width"], cfg["vocab"]
    side = (cfg.get("token_side") or {}).get("dim")
    out = [("embed", (vocab, width), "matrix")]
    if side:
        out.append(("side.embed", (vocab, side * len(cfg["layers"])), "matrix"))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out.append((p + "norm1", (width,), "around_zero"))
        if layer.get("mlp"):
            out.append((p + "norm2", (width,), "around_zero"))
        if layer["type"] == "latent_attention":
            H, dn, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.append((p + "mix.q", (H * (dn + rd), width), "matrix"))
            if m.get("kv_from") is None:
                out += [(p + "mix.dkv", (r + rd, width), "matrix"), (p + "mix.dkv.norm", (r,), "around_one")]
            out += [(p + "mix.uk", (H * dn, r), "matrix"), (p + "mix.uv", (H * dv, r), "matrix"),
                    (p + "mix.o", (width, H * dv), "matrix")]
        else:
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            out += [(p + "mix.q", (H * dk, width), "matrix"), (p + "mix.k", (H * dk, width), "matrix"),
                    (p + "mix.v", (H * dv, width), "matrix"), (p + "mix.g", (H * dv, width), "matrix"),
                    (p + "mix.o", (width, H * dv), "matrix"), (p + "mix.norm", (H * dv,), "around_one")]
        f = layer.get("mlp")
        if f:
            ff = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                out += [(f"{p}mlp.e{e}.gate", (ff, width), "matrix"), (f"{p}mlp.e{e}.up", (ff, width), "matrix"),
                        (f"{p}mlp.e{e}.down", (width, ff), "matrix")]
            out.append((p + "mlp.router", (f["router"]["experts"], width), "matrix"))
            if f.get("shared"):
                sf = f["shared"]["ff"]
                out += [(p + "mlp.shared.gate", (sf, width), "matrix"), (p + "mlp.shared.up", (sf, width), "matrix"),
                        (p + "mlp.shared.down", (width, sf), "matrix"), (p + "mlp.shared.sg", (1, width), "matrix")]
        if side:
            out += [(p + "side.gate", (side, width), "matrix"), (p + "side.proj", (width, side), "matrix"),
                    (p + "side.norm", (width,), "around_one")]
    out += [("final.norm", (width,), "around_zero"), ("head", (vocab, width), "matrix")]
    return out


def random_weights(cfg: dict, seed: int, scale: float = 1.0):
    """bfloat16 tensors: matrices ~ N(0, scale / sqrt(fan_in)), norm weights around zero or around one."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape, kind in tensor_list(cfg):
        t = torch.randn(shape, generator=g)
        if kind == "matrix":
            t = t * (scale / math.sqrt(shape[-1])) if name not in ("embed", "side.embed") else t
        else:
            t = t * 0.2 + (1.0 if kind == "around_one" else 0.0)
        w[name] = t.to(torch.bfloat16)
    return w
