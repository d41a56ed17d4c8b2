"""`Retention`: linear attention with a fixed decay per head, no softmax and no denominator.

    [q, k, v, g] = x W^T                     (one product; no biases)
    q, k rotated on the leading `rotary_dim` dims of each head (the mixer's position encoding; pairs (i, i + dims/2)),
    k *= head_dim^-1/2 after the rotation
    S_t = decay_h * S_(t-1) + k_t v_t^T      per head, S [head_dim, value_dim] float32 (kept transposed), zero for a new request
    o_t = S_t^T q_t,   each head of o divided by its root mean square,
    out = (concat_h(o) * silu(g)) W_o^T

Angles, the rotated q and k, the state and the head norm are float32.  The state is the layer's cache entry
(kind "state"): the cache manager clears a request's slot when it admits the request, so a portion of a
prompt simply continues from what the slot holds.
"""
from __future__ import annotations

import torch

from ..config.specs import CacheNeed
from .base import ParamSpec, Part


class Retention(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads = spec.width, spec.heads
        self.head_dim, self.value_dim = spec.head_dim, spec.value_dim or spec.head_dim
        self.position = position                       # None: nothing is rotated
        self.rotary_dim = getattr(position, "rotary_dim", 0) if position is not None else 0
        self.eps = float(spec.option("eps", 1e-6))
        decay = spec.option("decay")
        if decay is None or len(decay) != self.heads:
            raise ValueError("retention: one decay per head")
        self._decay_host = [float(d) for d in decay]
        self.decay = None
        self.cols = 2 * self.heads * (self.head_dim + self.value_dim)
        self.qkv = self.o = None

    @classmethod
    def parameters(cls, spec) -> dict:
        qk, v = spec.heads * spec.head_dim, spec.heads * (spec.value_dim or spec.head_dim)
        return {"qkv": ParamSpec((2 * qk + 2 * v, spec.width), pieces=(("q", qk), ("k", qk), ("v", v), ("g", v))),
                "o": ParamSpec((spec.width, v))}

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(spec.heads, spec.value_dim or spec.head_dim, spec.head_dim),
                         state_dtype="float32")

    def subparts(self) -> tuple:
        return (self.position,) if self.position is not None else ()

    def load(self, tensors: dict) -> None:
        super().load(tensors)
        self.decay = torch.tensor(self._decay_host, dtype=torch.float32, device=self.qkv.device)

    def forward(self, ctx, x, call):
        t = x.shape[0]
        _, state = ctx.cache.view(call.cache)
        proj = ctx.buffer("ret.proj", (t, self.cols), self.dtype)
        self.k.linear(x, self.qkv, proj)
        tables = self.position.tables(ctx) if self.rotary_dim else None
        o = ctx.buffer("ret.o", (t, self.heads * self.value_dim), torch.float32)
        self.k.retention(proj, tables, self.rotary_dim, self.decay, state, ctx.state_slots, ctx.cu_seqlens, o,
                         self.heads, self.head_dim, self.value_dim, self.head_dim ** -0.5, write=call.write,
                         longest=max(ctx.query_lens) if ctx.query_lens else 0)
        gated = ctx.buffer("ret.gated", (t, self.heads * self.value_dim), self.dtype)
        self.k.headnorm_gate(o, proj, 2 * self.heads * self.head_dim + self.heads * self.value_dim, gated,
                             self.heads, self.value_dim, self.eps)
        out = ctx.buffer("ret.out", (t, self.width), self.dtype)
        return self.k.linear(gated, self.o, out, defer=True)
