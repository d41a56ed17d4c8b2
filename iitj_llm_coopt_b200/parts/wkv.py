"""`WKV`: a recurrent mixer with a matrix state per head whose decay each token chooses per key channel.

    x' = the previous token's x (zeros before a request's first token; part of the state)
    m_s = x + (x' - x) * mu_s                      for s in r, k, v, g, w
    r, k, v = W_r m_r, W_k m_k, W_v m_v            (heads x head_dim each),   gate = silu(W_g m_g)
    w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))        per head and key channel, float32
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t      the bonus u lets the current token into its own output
    S_t = diag(w_t) S_(t-1) + k_t v_t^T            S [head_dim (key), head_dim (value)] float32 per head, zero for a new request
    out = ((each head of o divided by its root mean square) * gain * gate) W_o^T

The state is the layer's cache entry (kind "state", [heads, head_dim, head_dim] float32); the previous token's row is a
second entry of the call (`LayerCall.state`, [width] float32).  The cache manager clears both when it admits a request, so
a portion of a prompt simply continues from what the slots hold.  The decay and everything else that enters the recurrence
after the projections is float32.
"""
from __future__ import annotations

import torch

from ..config.specs import CacheNeed
from .base import ParamSpec, Part

STREAMS = ("r", "k", "v", "g", "w")


class WKV(Part):
    graph_safe = True

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads, self.head_dim = spec.width, spec.heads, spec.head_dim
        self.rank = int(spec.option("decay_rank"))
        self.eps = float(spec.option("eps", 1e-6))
        self.inner = self.heads * self.head_dim
        self.mu = self.rkvg = self.w1 = self.w2 = self.w0 = self.u = self.norm = self.o = None

    @classmethod
    def parameters(cls, spec) -> dict:
        n, w, rank = spec.heads * spec.head_dim, spec.width, int(spec.option("decay_rank"))
        return {"mu": ParamSpec((len(STREAMS) * w,), kind="vector", pieces=tuple((s, w) for s in STREAMS)),
                "rkvg": ParamSpec((4 * n, w), pieces=tuple((s, n) for s in STREAMS[:4])),
                "w1": ParamSpec((rank, w)),
                "w2": ParamSpec((n, rank), kind="vector"),
                "w0": ParamSpec((n,), kind="vector"),
                "u": ParamSpec((spec.heads, spec.head_dim), kind="vector"),
                "norm": ParamSpec((n,), kind="vector"),
                "o": ParamSpec((w, n))}

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(spec.heads, spec.head_dim, spec.head_dim), state_dtype="float32")

    @classmethod
    def state_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(spec.width,), state_dtype="float32")

    def load(self, tensors: dict) -> None:
        for name, t in tensors.items():        # the small tensors enter float32 arithmetic: kept in float32
            setattr(self, name, t if name in ("rkvg", "w1", "o") else t.float().contiguous())

    def forward(self, ctx, x, call):
        t = x.shape[0]
        if call.state is None:
            raise ValueError("wkv: the previous token's row needs a state entry (LayerCall.state)")
        _, state = ctx.cache.view(call.cache)
        _, before = ctx.cache.view(call.state)
        mixes = ctx.buffer("wkv.mixes", (len(STREAMS) * t, self.width), self.dtype)
        self.k.token_shift(x, self.mu, before, ctx.state_slots, ctx.token_request, ctx.cu_seqlens, mixes)
        rkvg = ctx.buffer("wkv.rkvg", (4 * t, self.inner), self.dtype)        # the rows of r, then of k, v and g
        for s in range(4):
            self.k.linear(mixes[s * t:(s + 1) * t], self.rkvg[s * self.inner:(s + 1) * self.inner], rkvg[s * t:(s + 1) * t])
        low = ctx.buffer("wkv.low", (t, self.rank), torch.float32)
        self.k.linear(mixes[4 * t:], self.w1, low)
        decay = ctx.buffer("wkv.decay", (t, self.inner), torch.float32)
        self.k.wkv_decay(low, self.w2, self.w0, decay)
        gated = ctx.buffer("wkv.gated", (t, self.inner), self.dtype)
        self.k.wkv_scan(rkvg, decay, self.u, self.norm, self.eps, state, ctx.state_slots, ctx.cu_seqlens, gated,
                        self.heads, self.head_dim, write=call.write, last_rows=(x, before) if call.write else None)
        out = ctx.buffer("attn.out", (t, self.width), self.dtype)
        return self.k.linear(gated, self.o, out)
