"""Rodapel: layers of latent attention (one low-rank row per token serves every head as key and as value), of
windowed grouped attention with normed heads and a gate per head, and of wkv (a matrix state per head whose decay each
token chooses), each followed by a dense or a routed gated feed-forward; the norms sit on the sub-layers' outputs.

Checkpoint tensor names: embed, embed.norm, head, final.norm, and for layer i: l<i>.norm1, l<i>.norm2,
l<i>.mix.<name>, l<i>.mlp.<name>.  Mixer tensors: latent attention q, dkv, dkv.norm, uk, uv, o; attention q, k, v,
q.norm, k.norm, g, o; wkv mu.{r,k,v,g,w}, r, k, v, g, w1, w2, w0, u, norm, o.  Feed-forward tensors: gate, up, down;
routed: router, correction and e<j>.{gate,up,down} for every expert j.
"""
from __future__ import annotations

import re

from ..config.registry import register_architecture
from ..config.rodapel import NAME, RodapelConfig
from .base import Architecture

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")

_MIXER = {            # (parameter, piece) -> what follows "l<i>.mix."
    ("q_dkv", "q"): "q", ("q_dkv", "dkv"): "dkv", ("dkv_norm", None): "dkv.norm", ("uk", None): "uk", ("uv", None): "uv",
    ("qkv", "q"): "q", ("qkv", "k"): "k", ("qkv", "v"): "v", ("q_norm", None): "q.norm", ("k_norm", None): "k.norm",
    ("gate", None): "g", ("o", None): "o",
    ("mu", "r"): "mu.r", ("mu", "k"): "mu.k", ("mu", "v"): "mu.v", ("mu", "g"): "mu.g", ("mu", "w"): "mu.w",
    ("rkvg", "r"): "r", ("rkvg", "k"): "k", ("rkvg", "v"): "v", ("rkvg", "g"): "g",
    ("w1", None): "w1", ("w2", None): "w2", ("w0", None): "w0", ("u", None): "u", ("norm", None): "norm",
}
_IN_LAYER = {
    ("mixer_norm.weight", None): "norm1", ("feed_forward_norm.weight", None): "norm2",
    ("feed_forward.gate_up", "gate"): "mlp.gate", ("feed_forward.gate_up", "up"): "mlp.up",
    ("feed_forward.down", None): "mlp.down",
    ("feed_forward.router", None): "mlp.router", ("feed_forward.correction", None): "mlp.correction",
}
_TOP = {"embedding.weight": "embed", "embedding.norm": "embed.norm", "final_norm.weight": "final.norm", "lm_head.weight": "head"}
_EXPERT_PIECE = re.compile(r"^e(\d+)\.(gate|up|down)$")


class Rodapel(Architecture):
    name = NAME
    config_class = RodapelConfig

    def checkpoint_name(self, path: str, piece: str | None) -> str:
        if path in _TOP and piece is None:
            return _TOP[path]
        m = _LAYER.match(path)
        if m:
            rest = m.group(2)
            if (rest, piece) in _IN_LAYER:
                return f"l{m.group(1)}." + _IN_LAYER[(rest, piece)]
            if rest in ("feed_forward.expert_gate_up", "feed_forward.expert_down") and piece and _EXPERT_PIECE.match(piece):
                return f"l{m.group(1)}.mlp.{piece}"
            if rest.startswith("mixer.") and (rest[6:], piece) in _MIXER:
                return f"l{m.group(1)}.mix." + _MIXER[(rest[6:], piece)]
        raise KeyError(f"{NAME} has no checkpoint tensor for parameter {path!r} piece {piece!r}")


register_architecture(Rodapel())
