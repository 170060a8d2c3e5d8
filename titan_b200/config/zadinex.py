"""Typed configuration of the Zadinex design, from its config.json.

A Zadinex model is a list of pre-norm layers, x += s1 * mixer(N1(x)); x += s2 * ff(N2(x)), whose norm takes no
statistics (``dyt``: tanh(alpha x) * w + b) and whose sublayer outputs are scaled element by element (s1, s2).  Mixers:
``attention`` (grouped queries, the first rot.dims dimensions of a head rotated in halves, Q and K heads divided by their
root mean square after the rotation, a learned sink in the softmax's denominator, values blended with those of the first
such layer) and ``wkv`` (a recurrence whose decay is made from the token).  Feed-forwards: ``dense`` (gelu-gated) or
``moe`` (clamped-swish experts; scores over all experts with a correction for the choice, groups of experts of which
only the best are open, experts without matrices that pass their input on), or none.  The keys read here:

    architecture "Zadinex";  vocab, width;  norm.eps
    layers[i].type "attention": mixer {heads, kv_heads, dim, vdim, rot {base, dims}, scale, v_mix}
    layers[i].type "wkv":       mixer {heads, dim}; the decay's rank is the first dimension of tensor l<i>.mix.w1
                                (or the key ``rank``, which a description without a weight file must give)
    layers[i].mlp  null | {kind "dense", ff} | {kind "moe", expert {ff, limit}, router {experts, top, identity, groups {count, keep}}}

Tensor names: embed, l<i>.norm1|norm2 (+ .b, .alpha), l<i>.mix.*, l<i>.mlp.*, l<i>.ls1|ls2, final.norm, head.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec
from .tefezen import _get

# No position limit is part of the design; positions are exact in float32 up to here.
MAX_POSITIONS = 1 << 24


@dataclass(frozen=True)
class ZadinexConfig:
    raw: Any                       # the config.json dict, checked, with every wkv layer's rank filled in
    architecture: str = "Zadinex"
    reads_tensor_shapes = True     # ``from_dict`` takes the shapes of the folder's tensors (name -> shape) where there is a folder

    def __hash__(self):
        return id(self)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], shapes: Optional[Dict[str, tuple]] = None) -> "ZadinexConfig":
        d = copy.deepcopy(d)
        _get(d, "vocab", int), _get(d, "width", int)
        if not _get(d, "norm.eps", float) > 0:
            raise ConfigError("norm.eps must be positive")
        layers = _get(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        first_mixing = None
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(layer, "type")
            m = _get(layer, "mixer")
            heads, dim = _get(m, "heads", int), _get(m, "dim", int)
            if kind == "attention":
                kv, vdim = _get(m, "kv_heads", int), _get(m, "vdim", int)
                if heads % kv:
                    raise ConfigError(f"{where}: {heads} query heads are not a multiple of {kv} key/value heads")
                dims, base = _get(m, "rot.dims", int), _get(m, "rot.base", float)
                if dims % 2 or dims > dim or not base > 0:
                    raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {dim}, rot.base positive")
                _get(m, "scale", float)
                if m.get("v_mix"):
                    if first_mixing is None:
                        first_mixing = i
                    else:
                        f = layers[first_mixing]["mixer"]
                        if (f["kv_heads"], f["vdim"]) != (kv, vdim):
                            raise ConfigError(f"{where}: values of {kv} x {vdim} cannot be blended with layer {first_mixing}'s {f['kv_heads']} x {f['vdim']}")
            elif kind == "wkv":
                if m.get("rank") is None:
                    shape = (shapes or {}).get(f"l{i}.mix.w1")
                    if shape is None or len(shape) != 2:
                        raise ConfigError(f"{where}: the decay's rank is neither in the description ('rank') nor given by a tensor l{i}.mix.w1")
                    m["rank"] = int(shape[0])
                _get(m, "rank", int)
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not known (attention, wkv)")
            f = layer.get("mlp")
            if f is None:
                continue
            if f.get("kind") == "dense":
                _get(f, "ff", int)
            elif f.get("kind") == "moe":
                E, top = _get(f, "router.experts", int), _get(f, "router.top", int)
                ident = f["router"].get("identity") or 0
                if isinstance(ident, bool) or not isinstance(ident, int) or ident < 0:
                    raise ConfigError(f"{where}: router.identity {ident!r} must be a count")
                groups = f["router"].get("groups")
                count, keep = (1, 1) if groups is None else (_get(groups, "count", int), _get(groups, "keep", int))
                n_all = E + ident
                if keep > count or n_all % count or top > keep * (n_all // count):
                    raise ConfigError(f"{where}: {top} of {n_all} experts in {count} groups of which {keep} are open")
                _get(f, "expert.ff", int)
                if not _get(f, "expert.limit", float) > 0:
                    raise ConfigError(f"{where}: expert.limit must be positive")
            else:
                raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not known (dense, moe)")
        return cls(raw=d, architecture=d.get("architecture") or (d.get("architectures") or ["Zadinex"])[0])

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    # ------------------------------------------------------------------ #
    def to_model_spec(self) -> ModelSpec:
        d = self.raw
        W, V, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        norm = lambda name: NormSpec("dyt", W, eps, name)
        first_mixing = next((i for i, l in enumerate(d["layers"]) if l["type"] == "attention" and l["mixer"].get("v_mix")), None)
        layers, unused = [], []
        for i, layer in enumerate(d["layers"]):
            m = layer["mixer"]
            if layer["type"] == "attention" and (not m.get("v_mix") or i == first_mixing):
                unused.append(f"l{i}.mix.vmix")                # a file may carry the factor of a layer that does not blend, or that the others blend with
            if layer.get("mlp") is None:
                unused += [f"l{i}.norm2", f"l{i}.norm2.b", f"l{i}.norm2.alpha", f"l{i}.ls2"]
            if layer["type"] == "attention":
                extra = [("value_dim", m["vdim"]), ("unit_norm", "after_rotation"), ("unit_norm_eps", eps), ("sink", "sink"), ("layer_index", i)]
                if m.get("v_mix"):
                    extra.append(("value_mix", (None if i == first_mixing else first_mixing, "vmix")))
                mixer = MixerSpec(
                    kind="attention", hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                    softmax_scale=float(m["scale"]), prefix="mix.",
                    position=PositionSpec("rope", rotary_dim=m["rot"]["dims"], theta=float(m["rot"]["base"]), pairing="half"),
                    names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")), extra=tuple(extra))
            else:
                mixer = MixerSpec(kind="wkv", hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], prefix="mix.",
                                  extra=(("rank", m["rank"]), ("norm_eps", eps)))
            f = layer.get("mlp")
            ffn = None
            if f is not None and f["kind"] == "dense":
                ffn = FeedForwardSpec(kind="gated_mlp", hidden_size=W, intermediate_size=f["ff"], activation="gelu_tanh", prefix="mlp.",
                                      names=(("gate", "gate"), ("up", "up"), ("down", "down")))
            elif f is not None:
                r = f["router"]
                groups = r.get("groups") or {"count": 1, "keep": 1}
                ffn = FeedForwardSpec(kind="moe", hidden_size=W, intermediate_size=f["expert"]["ff"], activation="swish_clamped", prefix="mlp.",
                                      extra=(("experts", r["experts"]), ("top", r["top"]), ("identity", r.get("identity") or 0),
                                             ("routing", "softmax_all"), ("groups", groups["count"]), ("keep", groups["keep"]),
                                             ("limit", float(f["expert"]["limit"]))))
            layers.append(LayerSpec(index=i, arrangement="pre_norm_scaled", mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
                                    feed_forward_norm=None if ffn is None else norm("norm2"), prefix=f"l{i}.",
                                    extra=(("scales", ("ls1",) if ffn is None else ("ls1", "ls2")),)))
        spec = ModelSpec(architecture=self.architecture, hidden_size=W, vocab_size=V, layers=tuple(layers), order=tuple(range(len(layers))),
                         final_norm=norm("final.norm"), embedding="embed", lm_head="head", max_positions=MAX_POSITIONS,
                         ignorable_tensors=tuple(unused))
        spec.validate()
        return spec
