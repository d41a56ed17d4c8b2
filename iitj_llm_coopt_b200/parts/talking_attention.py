"""`TalkingAttention`: grouped-query attention whose heads' scores are mixed before the softmax, with a short
causal convolution over time on the projections, norms on queries, keys and values, a distance bias in place
of a rotation, and an optional chunked mask.  Every constant is a parameter of the spec.

    u   = x W^T + b                         (q, k and v as one product; b when `bias`)
    c_t = sum_j taps[:, j] * u_(t - n + 1 + j)      n = `conv_taps` (0: c = u); zeros before the request's first token; the
                                            last n - 1 rows of u of every request are its convolution state
    q   = rmsnorm(c_q over all query heads at once) * q_gain,    k likewise with k_gain,
    v   = each value head of c_v divided by its root mean square (no gain);   k and v are what the cache holds
    s[g, i, j] = scale * q[g, i] . k[kv(g), j] - slope_g * (i - j),    slope_g = 2^(-slope_exponent * (g + 1) / heads)
    a[h, i, j] = sum_g talk[h, g] * s[g, i, j]
    p[h, i, :] = softmax of a over the keys j <= i (with `chunk` c > 0: only those with j // c == i // c)
    out = concat_h(p[h] v[kv(h)]) W_o^T

Norms, scores, bias, mixing and softmax run in float32.  With `own_kv` false the layer has no key and value
tensors: the run order points its `call.cache` at the entry of the layer whose keys and values it reads
(`call.write` false), and only its queries pass through projection, convolution and norm.

The convolution state is a second cache entry of the call (`LayerCall.state`): [conv_taps - 1, channels]
float32 per request, zero when the request is admitted.
"""
from __future__ import annotations

import torch

from ..config.specs import CacheNeed
from .base import ParamSpec, Part, StepPlan


class TalkingAttention(Part):
    graph_safe = True
    prepare_key = "talking_attention"      # every such layer of a model shares one plan of the step's query tiles
    TILE = 16                              # query tokens of one request a block of the tensor-core kernel takes

    def __init__(self, spec, kernels, dtype, position=None):
        self.spec, self.k, self.dtype = spec, kernels, dtype
        self.width, self.heads, self.kv_heads = spec.width, spec.heads, spec.kv_heads
        self.head_dim, self.value_dim = spec.head_dim, spec.value_dim or spec.head_dim
        if self.heads % self.kv_heads:
            raise ValueError(f"talking attention: heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        self.scale = spec.softmax_scale or self.head_dim ** -0.5
        self.chunk, self.taps = int(spec.option("chunk", 0)), int(spec.option("conv_taps", 0))      # 0 taps: no convolution
        self.bias, self.own_kv = bool(spec.option("bias", False)), bool(spec.option("own_kv", True))
        self.eps = float(spec.option("eps", 1e-6))
        self.channels = self._channels(spec)
        e = float(spec.option("slope_exponent", 8.0))
        self._slopes_host = [2.0 ** (-e * (h + 1) / self.heads) for h in range(self.heads)]
        self.slopes = None
        self.qkv = self.o = self.qkv_bias = self.qkv_conv = self.q_norm = self.k_norm = self.talk = None

    @staticmethod
    def _rows(spec) -> tuple:
        q = spec.heads * spec.head_dim
        if not spec.option("own_kv", True):
            return (("q", q),)
        return (("q", q), ("k", spec.kv_heads * spec.head_dim), ("v", spec.kv_heads * (spec.value_dim or spec.head_dim)))

    @classmethod
    def _channels(cls, spec) -> int:
        return sum(n for _, n in cls._rows(spec))

    @classmethod
    def parameters(cls, spec) -> dict:
        rows, c = cls._rows(spec), cls._channels(spec)
        q = spec.heads * spec.head_dim
        out = {"qkv": ParamSpec((c, spec.width), pieces=rows),
               "q_norm": ParamSpec((q,), kind="vector"),
               "talk": ParamSpec((spec.heads, spec.heads), kind="vector"),
               "o": ParamSpec((spec.width, spec.heads * (spec.value_dim or spec.head_dim)))}
        if spec.option("bias", False):
            out["qkv_bias"] = ParamSpec((c,), kind="vector", pieces=rows)
        if int(spec.option("conv_taps", 0)) >= 1:
            out["qkv_conv"] = ParamSpec((c, int(spec.option("conv_taps"))), kind="vector", pieces=rows)
        if spec.option("own_kv", True):
            out["k_norm"] = ParamSpec((spec.kv_heads * spec.head_dim,), kind="vector")
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="paged_kv", kv_heads=spec.kv_heads, head_dim=spec.head_dim,
                         value_dim=spec.value_dim or spec.head_dim)

    @classmethod
    def state_need(cls, spec) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(max(int(spec.option("conv_taps", 0)) - 1, 0), cls._channels(spec)),
                         state_dtype="float32")

    def prepare_step(self, shape):
        """A step with prompt portions: its tokens cut into runs of up to TILE tokens of one request (first token row,
        rows, position of the first row, request), for the kernel that takes a tile of queries at a time.  A step of
        single decoded tokens needs none (the one-token kernel runs)."""
        if shape.decode_shaped or shape.num_tokens == len(shape.query_lens):
            return None
        tiles, row = [], 0
        for b, (n, total) in enumerate(zip(shape.query_lens, shape.seq_lens)):
            for s in range(0, n, self.TILE):
                tiles += [row + s, min(self.TILE, n - s), total - n + s, b]
            row += n
        return StepPlan(arrays={"tiles": tiles})

    def load(self, tensors: dict) -> None:
        for name, t in tensors.items():        # the small tensors enter float32 arithmetic: kept in float32
            setattr(self, name, t if name in ("qkv", "o") else t.float().contiguous())
        self.slopes = torch.tensor(self._slopes_host, dtype=torch.float32, device=self.qkv.device)

    def forward(self, ctx, x, call):
        t = x.shape[0]
        if call.write != self.own_kv:
            raise ValueError("talking attention: a layer with keys and values of its own writes its cache entry, a borrowing one does not")
        group, view = ctx.cache.view(call.cache)
        meta = ctx.group(group)
        u = ctx.buffer("tattn.u", (t, self.channels), self.dtype)
        self.k.linear(x, self.qkv, u)
        state = None
        if self.taps > 1:
            if call.state is None:
                raise ValueError("talking attention: a convolution needs a state entry (LayerCall.state)")
            state = ctx.cache.view(call.state)[1]
        q = ctx.buffer("tattn.q", (t, self.heads * self.head_dim), self.dtype)
        self.k.conv_norm_store(u, self.qkv_bias, self.qkv_conv, self.q_norm, self.k_norm, state, ctx.state_slots,
                               ctx.token_request, ctx.cu_seqlens, q, view if self.own_kv else None,
                               meta.slots if self.own_kv else None, self.heads, self.kv_heads, self.head_dim,
                               self.value_dim, self.eps)
        attn = ctx.buffer("tattn.ctx", (t, self.heads * self.value_dim), self.dtype)
        plan = ctx.prepared.get(self.prepare_key)
        tiles = plan.device_arrays.get("tiles") if plan is not None else None
        self.k.talking_attention(q, view, meta, self.talk, self.slopes, attn, self.heads, self.kv_heads, self.head_dim,
                                 self.value_dim, self.chunk, self.scale, tiles=tiles.view(-1, 4) if tiles is not None else None)
        out = ctx.buffer("tattn.out", (t, self.width), self.dtype)
        return self.k.linear(attn, self.o, out, defer=True)
