"""Lifusun: layers of chunked talking-heads attention (short convolutions on q, k and v, keys and values that a
later layer may borrow) and of retention (linear attention with a fixed decay per head), each with an optional
dense feed-forward, under norms with one gain for the whole width.

Checkpoint tensor names: embed, head, final.norm, and for layer i: l<i>.norm1, l<i>.norm2, l<i>.mix.<name>,
l<i>.mlp.{gate,up,down}.  A mixer's tensors: q, k, v, o (and g for retention); for attention also the biases
q.b, k.b, v.b, the convolution taps q.conv, k.conv, v.conv, the gains q.norm and k.norm, and talk.
"""
from __future__ import annotations

import re

from ..config.lifusun import NAME, LifusunConfig
from ..config.registry import register_architecture
from .base import Architecture

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")

_MIXER = {            # (parameter, piece) -> what follows "l<i>.mix."
    ("qkv", "q"): "q", ("qkv", "k"): "k", ("qkv", "v"): "v", ("qkv", "g"): "g",
    ("qkv_bias", "q"): "q.b", ("qkv_bias", "k"): "k.b", ("qkv_bias", "v"): "v.b",
    ("qkv_conv", "q"): "q.conv", ("qkv_conv", "k"): "k.conv", ("qkv_conv", "v"): "v.conv",
    ("q_norm", None): "q.norm", ("k_norm", None): "k.norm", ("talk", None): "talk", ("o", None): "o",
}
_IN_LAYER = {
    ("mixer_norm.weight", None): "norm1", ("feed_forward_norm.weight", None): "norm2",
    ("feed_forward.gate_up", "gate"): "mlp.gate", ("feed_forward.gate_up", "up"): "mlp.up",
    ("feed_forward.down", None): "mlp.down",
}
_TOP = {"embedding.weight": "embed", "final_norm.weight": "final.norm", "lm_head.weight": "head"}


class Lifusun(Architecture):
    name = NAME
    config_class = LifusunConfig

    def checkpoint_name(self, path: str, piece: str | None) -> str:
        if path in _TOP and piece is None:
            return _TOP[path]
        m = _LAYER.match(path)
        if m:
            rest = m.group(2)
            if (rest, piece) in _IN_LAYER:
                return f"l{m.group(1)}." + _IN_LAYER[(rest, piece)]
            if rest.startswith("mixer.") and (rest[6:], piece) in _MIXER:
                return f"l{m.group(1)}.mix." + _MIXER[(rest[6:], piece)]
        raise KeyError(f"{NAME} has no checkpoint tensor for parameter {path!r} piece {piece!r}")


register_architecture(Lifusun())
