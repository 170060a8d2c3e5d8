"""Linear attention with a per-head decay ("lightning" attention) as a mixer.

    [q | k | v | g] = h . [W_q ; W_k ; W_v ; W_g]^T                 one product
    q, k, v <- silu(.)                                              heads x dim, heads x dim, heads x value_dim
    S_t = decay_h S_{t-1} + k_t v_t^T ;  o_t = S_t^T q_t            per head; S float32 [dim, value_dim], zero at the start
    y = rmsnorm(concat_h o_t) * w * sigmoid(g) ;  out += y . W_o^T

The state is what the mixer asks of the cache: a ``state`` group of shape [heads, dim, value_dim] in float32 per
sequence, zeroed when a slot is handed out, read and written through the step's slot indices on the device (nothing
of the layout is read on the host, so decode steps with this mixer are captured as graphs like any other).  The
recurrence takes a sequence's tokens in order whatever the step brings: a whole prompt, a piece of it, or one token.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, StateGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, NORMS, Mixer


class LightningMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.dk, self.dv = s.num_heads, s.head_dim, int(s.option("value_dim", s.head_dim))
        decay = tuple(float(d) for d in s.option("decay", ()))
        if self.H <= 0 or self.dk <= 0 or self.dv <= 0:
            raise ValueError("lightning attention needs positive heads, dim and value_dim")
        if self.dk > 256:
            raise ValueError(f"{self.dk} key dimensions a head: the recurrence kernel holds up to 256")
        if len(decay) != self.H:
            raise ValueError(f"{len(decay)} decays for {self.H} heads")
        self.decay_values = decay
        self.out_norm_spec = s.option("out_norm")
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", state_shape=(self.H, self.dk, self.dv), state_dtype=torch.float32)

    def _names(self):
        return {role: self.spec.name(role, role) for role in ("q", "k", "v", "g", "o")}

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        W, Nk, Nv = s.hidden_size, self.H * self.dk, self.H * self.dv
        return ([WeightSpec(p + n["q"], (Nk, W)), WeightSpec(p + n["k"], (Nk, W)), WeightSpec(p + n["v"], (Nv, W)),
                 WeightSpec(p + n["g"], (Nv, W)), WeightSpec(p + n["o"], (W, Nv))]
                + NORMS.build(self.out_norm_spec).weight_specs(p))

    def bind(self, get) -> None:
        p, n = self.spec.prefix, self._names()
        self.w_in = torch.cat([get(p + n[role]) for role in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = get(p + n["o"])
        norm = NORMS.build(self.out_norm_spec)
        norm.bind(lambda name: get(p + name))
        self.norm_w = norm.weight
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        lay = ctx.layout
        T, H, dk, dv = lay.T, self.H, self.dk, self.dv
        group, index = cache
        if not isinstance(group, StateGroup):
            raise TypeError(f"lightning attention keeps its state in a 'state' cache group, not in {type(group).__name__}")
        proj = ctx.empty((T, self.w_in.shape[0]))
        linear.matmul(h, self.w_in, proj, linear.EPI_STORE, ctx)
        o = ctx.empty((T, H * dv), torch.float32)
        a = K.LightningArgs()
        a.proj, a.stride = proj.data_ptr(), proj.stride(0)
        a.out, a.out_stride = o.data_ptr(), o.stride(0)
        a.state, a.decay = group.layer_storage(index).data_ptr(), self.decay.data_ptr()
        a.q_start, a.slot_of_seq = lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr()
        a.B, a.H, a.dk, a.dv, a.max_new = lay.B, H, dk, dv, lay.max_new
        K.lightning_scan(a, proj.dtype, ctx.stream)
        y = ctx.empty((T, H * dv))
        K.gated_rmsnorm(o, self.norm_w, proj[:, 2 * H * dk + H * dv:], y, self.out_norm_spec.eps, ctx.stream)
        linear.matmul(y, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("lightning", LightningMixer)
