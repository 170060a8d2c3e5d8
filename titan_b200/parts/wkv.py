"""A linear recurrence with a decay made from the token ("wkv" time mixing) as a mixer.

With h the mixer's input rows and h' the row of the token before (zeros before a sequence's first token):

    mix_s = h + (h' - h) * mu_s                       s in r, k, v, g, w: five inputs, each its own blend of the two rows
    r, k, v = W_r mix_r, W_k mix_k, W_v mix_v         heads x dim each;   gate = silu(W_g mix_g)
    w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))         the decay, per head and key channel, float32
    o_t = (S + diag(u) k_t v_t^T)^T r_t               per head; the bonus u counts for the current token only
    S   = diag(w_t) S + k_t v_t^T                     S float32 [dim, dim] per head, zero at the start
    y   = concat_h(o / rms(o)) * weight * gate;       out += W_o y

What the mixer asks of the cache is one float32 row per sequence in the ``state`` group: every head's S, then the
sequence's last input row (the h' of the next step's first token); zeroed when a slot is handed out, read and written
through the step's slot indices on the device, so decode steps are captured as graphs.  The recurrence takes a
sequence's tokens in order whatever the step brings.  The four large projections are one batched product (a product a
mix); the low-rank decay's second half, tanh, w0 and the two exponentials are one kernel.  The rank of the decay's
low-rank product is a spec option (``rank``).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed, StateGroup
from ..weights.loader import WeightSpec
from . import linear
from .base import MIXERS, Mixer


class WkvMixer(Mixer):
    def __init__(self, spec):
        s = spec
        self.spec = s
        self.H, self.dk, self.W, self.rank = s.num_heads, s.head_dim, s.hidden_size, int(s.option("rank", 0))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.dk <= 0 or self.rank <= 0:
            raise ValueError("the wkv mixer needs positive heads, dim and rank")
        if self.dk > 256:
            raise ValueError(f"{self.dk} key channels a head: the recurrence kernel holds up to 256")
        self.N = self.H * self.dk
        self.state_size = self.H * self.dk * self.dk + self.W
        self.w_in = self.w_1 = self.w_2 = self.w_0 = self.w_o = self.mu = self.u = self.norm_w = None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def _name(self, role: str) -> str:
        return self.spec.name(role, role)

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        p, W, N = prefix + self.spec.prefix, self.W, self.N
        mu = self._name("mu")
        return ([WeightSpec(p + mu + "." + s, (W,), "vector", ("normal", 0.3)) for s in "rkvgw"]
                + [WeightSpec(p + self._name(s), (N, W)) for s in "rkvg"]
                + [WeightSpec(p + self._name("w1"), (self.rank, W)), WeightSpec(p + self._name("w2"), (N, self.rank)),
                   WeightSpec(p + self._name("w0"), (N,), "vector", ("normal", 1.0)),
                   WeightSpec(p + self._name("u"), (self.H, self.dk), "vector", ("normal", 0.3)),
                   WeightSpec(p + self._name("norm"), (N,), "vector", ("one_plus_normal", 0.1)),
                   WeightSpec(p + self._name("o"), (W, N))])

    def bind(self, get) -> None:
        p = self.spec.prefix
        g = lambda role: get(p + self._name(role))
        self.mu = torch.stack([get(p + self._name("mu") + "." + s) for s in "rkvgw"]).contiguous()
        self.w_in = torch.stack([g(s) for s in "rkvg"]).contiguous()           # [4, N, W]: one product a mix
        self.w_1, self.w_2, self.w_0 = g("w1"), g("w2"), g("w0")
        self.u, self.norm_w, self.w_o = g("u").contiguous(), g("norm"), g("o")

    def forward(self, h, ctx, cache, out: torch.Tensor) -> None:
        lay = ctx.layout
        T, N, W = lay.T, self.N, self.W
        group, index = cache
        if not isinstance(group, StateGroup):
            raise TypeError(f"the wkv mixer keeps its state in a 'state' cache group, not in {type(group).__name__}")
        state = group.layer_storage(index)
        f32 = torch.float32
        mixes, proj = ctx.empty((T, 5 * W)), ctx.empty((T, 4 * N))
        lora = ctx.empty((T, -(-self.rank // 8) * 8))[:, :self.rank]          # rows of whole 16 bytes
        decay, o, y = ctx.empty((T, N), f32), ctx.empty((T, N), f32), ctx.empty((T, N))
        a = K.WkvArgs()
        a.h, a.h_stride = h.data_ptr(), h.stride(0)
        a.mixes, a.mix_stride, a.mu = mixes.data_ptr(), mixes.stride(0), self.mu.data_ptr()
        a.proj, a.proj_stride = proj.data_ptr(), proj.stride(0)
        a.lora, a.lora_stride, a.w2, a.w0 = lora.data_ptr(), lora.stride(0), self.w_2.data_ptr(), self.w_0.data_ptr()
        a.decay, a.u = decay.data_ptr(), self.u.data_ptr()
        a.out, a.out_stride = o.data_ptr(), o.stride(0)
        a.state, a.state_stride = state.data_ptr(), state.stride(0)
        a.norm_w, a.y, a.y_stride, a.eps = self.norm_w.data_ptr(), y.data_ptr(), y.stride(0), self.eps
        a.q_start, a.slot_of_seq, a.seq_of = lay.q_start.data_ptr(), lay.slot_of_seq.data_ptr(), lay.seq_of.data_ptr()
        a.T, a.B, a.H, a.dk, a.W, a.rank, a.max_new = T, lay.B, self.H, self.dk, W, self.rank, lay.max_new
        dt = h.dtype
        K.wkv(a, K.WKV_SHIFT, dt, ctx.stream)
        linear.matmul_heads(mixes, self.w_in, proj, 4, W, N, ctx)
        linear.matmul(mixes[:, 4 * W:], self.w_1, lora, linear.EPI_STORE, ctx)
        K.wkv(a, K.WKV_DECAY, dt, ctx.stream)
        K.wkv(a, K.WKV_SCAN, dt, ctx.stream)
        K.wkv(a, K.WKV_OUT, dt, ctx.stream)
        linear.matmul(y, self.w_o, out, linear.EPI_ADD, ctx)


MIXERS.register("wkv", WkvMixer)
