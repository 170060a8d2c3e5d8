"""Typed configuration of the Tefezen design, from its config.json.

A Tefezen model is a list of layers, each with a mixer (``latent_attention`` over a sliding window, or ``lightning``
linear attention with per-head decays), an optional mixture-of-experts feed-forward, and, if the model has one, a
per-layer input looked up by the token.  Sublayers read the residual stream itself; an RMS norm whose weight is stored
around zero follows each sublayer's output.  The keys read here:

    architecture "Tefezen";  vocab, width;  embedding.scale;  norm.eps;  token_side.dim (absent: no such input);
    layers[i].type, .mixer {heads, dim, vdim, and per type: kv_rank, rot_dim, rot {base, dims}, mask {size}, scale,
    kv_from | decay [heads]}, .mlp null | {kind "moe", expert {ff}, router {experts, top}, shared {ff} (optional)}

Tensor names: embed, side.embed, l<i>.norm1|norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.side.*, final.norm, head.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)

# No position limit is part of the design; positions are exact in float32 up to here.
MAX_POSITIONS = 1 << 24


def _get(d: Dict[str, Any], path: str, kind=None, default=...):
    node: Any = d
    for key in path.split("."):
        if not isinstance(node, dict) or key not in node or node[key] is None:
            if default is not ...:
                return default
            raise ConfigError(f"config.json lacks the key '{path}'")
        node = node[key]
    if kind is int:
        if isinstance(node, bool) or not isinstance(node, (int, float)) or node != int(node) or node <= 0:
            raise ConfigError(f"config.json key '{path}' must be a positive integer, found {node!r}")
        return int(node)
    if kind is float:
        if isinstance(node, bool) or not isinstance(node, (int, float)) or not math.isfinite(node):
            raise ConfigError(f"config.json key '{path}' must be a number, found {node!r}")
        return float(node)
    return node


@dataclass(frozen=True)
class TefezenConfig:
    raw: Any                       # the config.json dict, checked
    architecture: str = "Tefezen"

    def __hash__(self):
        return id(self)

    # ------------------------------------------------------------------ #
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TefezenConfig":
        d = copy.deepcopy(d)
        _get(d, "vocab", int), _get(d, "width", int)
        eps = _get(d, "norm.eps", float)
        if not eps > 0:
            raise ConfigError("norm.eps must be positive")
        layers = _get(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(layer, "type")
            m = _get(layer, "mixer")
            heads = _get(m, "heads", int)
            _get(m, "dim", int), _get(m, "vdim", int)
            if kind == "latent_attention":
                rd = _get(m, "rot_dim", int)
                _get(m, "kv_rank", int), _get(m, "mask.size", int), _get(m, "scale", float)
                dims, base = _get(m, "rot.dims", int), _get(m, "rot.base", float)
                if dims % 2 or dims > rd or not base > 0:
                    raise ConfigError(f"{where}: rot.dims {dims} must be even and at most rot_dim {rd}, rot.base positive")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{where}: kv_from {src!r} must name an earlier layer")
                    o = layers[src]
                    if o.get("type") != "latent_attention" or (o.get("mixer") or {}).get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from {src} names a layer that keeps no latents of its own")
            elif kind == "lightning":
                decay = _get(m, "decay")
                if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(x, (int, float)) and 0 <= x <= 1 for x in decay):
                    raise ConfigError(f"{where}: 'decay' must list one number in [0, 1] for each of the {heads} heads")
            else:
                raise ConfigError(f"{where}: mixer type '{kind}' is not known (latent_attention, lightning)")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind") != "moe":
                    raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not known (moe)")
                E, top = _get(f, "router.experts", int), _get(f, "router.top", int)
                if top > E:
                    raise ConfigError(f"{where}: {top} of {E} experts")
                _get(f, "expert.ff", int)
                if f.get("shared") is not None:
                    _get(f, "shared.ff", int)
        if d.get("token_side") is not None:
            _get(d, "token_side.dim", int)
        return cls(raw=d, architecture=d.get("architecture") or (d.get("architectures") or ["Tefezen"])[0])

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    # ------------------------------------------------------------------ #
    def to_model_spec(self) -> ModelSpec:
        d = self.raw
        W, V, eps = d["width"], d["vocab"], float(d["norm"]["eps"])
        side = _get(d, "token_side.dim", int, None)
        layers_cfg = d["layers"]
        n_layers = len(layers_cfg)
        around_zero = lambda name, size=W: NormSpec("rmsnorm", size, eps, name, weight_offset=1.0)
        plain = lambda name, size: NormSpec("rmsnorm", size, eps, name)
        # what an owner of latents must keep: the longest look-back among itself and the layers that read its rows
        keeps: Dict[int, int] = {}
        for i, layer in enumerate(layers_cfg):
            if layer["type"] == "latent_attention":
                owner = layer["mixer"].get("kv_from")
                owner = i if owner is None else owner
                keeps[owner] = max(keeps.get(owner, 0), int(layer["mixer"]["mask"]["size"]))
        layers = []
        for i, layer in enumerate(layers_cfg):
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                src = m.get("kv_from")
                mixer = MixerSpec(
                    kind="latent_attention", hidden_size=W, num_heads=m["heads"], num_kv_heads=1, head_dim=m["dim"],
                    window=int(m["mask"]["size"]), softmax_scale=float(m["scale"]), cache_from=src, prefix="mix.",
                    position=PositionSpec("rope", rotary_dim=m["rot"]["dims"], theta=float(m["rot"]["base"]), pairing="adjacent"),
                    extra=(("rot_dim", m["rot_dim"]), ("value_dim", m["vdim"]), ("kv_rank", m["kv_rank"]),
                           ("cache_window", keeps[i if src is None else src]), ("latent_norm", plain("dkv.norm", m["kv_rank"]))))
            else:
                mixer = MixerSpec(
                    kind="lightning", hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], prefix="mix.",
                    extra=(("value_dim", m["vdim"]), ("decay", tuple(float(x) for x in m["decay"])),
                           ("out_norm", plain("norm", m["heads"] * m["vdim"]))))
            f = layer.get("mlp")
            ffn = None
            if f is not None:
                shared = f.get("shared")
                ffn = FeedForwardSpec(kind="moe", hidden_size=W, intermediate_size=f["expert"]["ff"], activation="silu", prefix="mlp.",
                                      extra=(("experts", f["router"]["experts"]), ("top", f["router"]["top"]),
                                             ("shared_size", 0 if shared is None else shared["ff"])))
            more, norms = (), ()
            if side:
                more = (FeedForwardSpec(kind="token_table", hidden_size=W, intermediate_size=side, activation="gelu_tanh", prefix="side.",
                                        extra=(("table", "side.embed"), ("offset", i * side))),)
                norms = (plain("side.norm", W),)
            layers.append(LayerSpec(index=i, arrangement="output_norm", mixer=mixer, feed_forward=ffn, mixer_norm=around_zero("norm1"),
                                    feed_forward_norm=None if ffn is None else around_zero("norm2"), prefix=f"l{i}.",
                                    norms=norms, extra=(("sublayers", more),)))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=W, vocab_size=V, layers=tuple(layers), order=tuple(range(n_layers)),
            final_norm=around_zero("final.norm"), embedding="embed", lm_head="head", max_positions=MAX_POSITIONS,
            embedding_scale=_get(d, "embedding.scale", float, None),
            shared_tensors=((("side.embed", (V, side * n_layers)),) if side else ()))
        spec.validate()
        return spec
