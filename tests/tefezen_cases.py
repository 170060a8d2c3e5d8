"""Small Tefezen configurations for the tests, each unlike the others in every size, option and layer order."""
import copy
import math


def latent(heads, dim, rot_dim, vdim, kv_rank, window, rot_dims=None, base=10000.0, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dims or rot_dim}, "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def model(layers, width, vocab, eps, side=None, scale=None):
    cfg = {"architecture": "Tefezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    return cfg


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


CASES = {
    # latent / lightning / reader of layer 0, a shared expert everywhere, window below one page
    "small": lambda: model([with_mlp(latent(2, 16, 8, 16, 24, 20), moe(4, 2, 24, shared=32)),
                            with_mlp(lightning(2, 8, 16, [0.7, 0.98]), moe(4, 2, 24, shared=32)),
                            with_mlp(latent(2, 16, 8, 16, 24, 20, kv_from=0), moe(4, 2, 24, shared=32))],
                           width=48, vocab=97, eps=1e-5, side=8, scale=0.5),
    # lightning first; sizes that are no multiples of 8; part of the rotated vector passes unrotated; one expert a token;
    # a layer without feed-forward; a reader with a longer window than its owner's; windows beyond one page
    "odd": lambda: model([with_mlp(latent(3, 12, 6, 20, 22, 70, rot_dims=4, base=500.0, scale=0.3), moe(5, 1, 18)),
                          with_mlp(lightning(3, 12, 10, [0.5, 0.9, 0.999]), moe(3, 3, 10, shared=14)),
                          dict(lightning(1, 40, 33, [1.0]), mlp=None),
                          with_mlp(latent(5, 8, 6, 12, 22, 100, rot_dims=4, base=500.0, kv_from=0, scale=0.2), moe(7, 2, 16, shared=8)),
                          with_mlp(latent(1, 32, 16, 8, 64, 64), moe(2, 2, 40))],
                         width=56, vocab=131, eps=3e-6, side=5, scale=1.7),
    # no embedding scale, no token input, no shared expert; a window longer than any test sequence
    "bare": lambda: model([with_mlp(lightning(4, 16, 16, [0.9, 0.95, 0.99, 0.8]), moe(6, 2, 32)),
                           with_mlp(latent(4, 16, 16, 16, 32, 4096), moe(6, 2, 32))],
                          width=64, vocab=211, eps=1e-6),
    # one latent layer only: a position's logits depend on the window's tokens alone
    "window": lambda: model([with_mlp(latent(2, 16, 8, 16, 24, 64, scale=0.45), moe(3, 1, 16))], width=40, vocab=61, eps=1e-5, side=4),
}


def make_config(name):
    return copy.deepcopy(CASES[name]())
