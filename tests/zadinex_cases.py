"""Small Zadinex configurations for the tests, each unlike the others in every size, option and layer order."""
import copy


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=0.25, v_mix=False):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
                                           "scale": scale, "v_mix": v_mix}}


def wkv(heads, dim, rank):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "rank": rank}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, identity=0, groups=None):
    r = {"experts": experts, "top": top, "identity": identity}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def model(layers, width, vocab, eps):
    return {"architecture": "Zadinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


CASES = {
    # attention / wkv / attention; values blended in both attention layers; groups of two experts of which half are open;
    # two experts that pass their input on
    "mix": lambda: model([with_mlp(attention(4, 2, 16, 16, 8, v_mix=True), dense(40)),
                          with_mlp(wkv(3, 8, 5), moe(6, 2, 24, 1.5, identity=2, groups=(4, 2))),
                          with_mlp(attention(4, 2, 16, 16, 8, v_mix=True), moe(6, 2, 24, 1.5, identity=2, groups=(4, 2)))],
                         width=48, vocab=97, eps=1e-5),
    # wkv first; keys and values of unequal widths that are no multiples of 8; one kv head; a layer without feed-forward;
    # a rotation over the whole head; one expert a token and no groups; as many pass-through experts as real ones; a
    # blending layer that is the only one (its factor is unused); an odd feed-forward width
    "odd": lambda: model([with_mlp(wkv(1, 40, 3), dense(33)),
                          dict(attention(3, 1, 12, 20, 4, base=500.0, scale=0.3), mlp=None),
                          with_mlp(attention(6, 3, 8, 8, 8, base=77.0, scale=0.6, v_mix=True), moe(5, 1, 18, 0.7)),
                          with_mlp(wkv(2, 20, 9), moe(3, 2, 10, 2.5, identity=3, groups=(3, 1)))],
                         width=56, vocab=131, eps=3e-6),
    # heads of 64 and of 128: in bfloat16 the tensor-core attention kernels and the tensor-core products; a first attention
    # layer that does not blend, then two that do
    "wide": lambda: model([with_mlp(attention(4, 2, 64, 64, 16, base=30000.0, scale=0.14), dense(192)),
                           with_mlp(attention(4, 2, 64, 64, 16, base=30000.0, scale=0.14, v_mix=True), moe(10, 2, 80, 1.25, identity=2, groups=(3, 1))),
                           with_mlp(wkv(4, 64, 24), moe(8, 3, 64, 1.0, groups=(4, 3))),
                           with_mlp(attention(2, 2, 64, 64, 64, scale=0.11, v_mix=True), dense(128)),
                           with_mlp(attention(2, 1, 128, 128, 64, scale=0.09), dense(128))],
                          width=128, vocab=211, eps=1e-6),
}


def make_config(name):
    return copy.deepcopy(CASES[name]())
