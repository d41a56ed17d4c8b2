"""Typed configuration of the Lifusun family, read from its config.json.

Keys: "architecture" ("Lifusun"), "width", "vocab", "norm" {"eps"} and "layers", a list whose entries give
"type" ("attention" or "retention"), the mixer's sizes under "mixer" and the feed-forward under "mlp"
({"kind": "dense", "ff": inner width}, or null for a layer without one).

An attention mixer: "heads", "kv_heads", "dim" (query/key head size), "vdim" (value head size), "scale" (of the
scores), "conv" (taps of the short convolution over time on q, k and v; absent: none), "mask" {"size"} (queries see keys of
their own chunk of that many positions) and optionally "kv_from" (the index of an earlier attention layer whose
cached keys and values this layer reads; it then has no key/value tensors of its own).
A retention mixer: "heads", "dim", "vdim", "decay" (one per head) and "rot" {"dims", "base"} (the leading dims of
each head that are rotated, and the base of the frequencies).

Every size is read from the file; a missing key is an error at once.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field

from .errors import ConfigError
from .specs import FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec

NAME = "Lifusun"
_MAX_POSITION = 1 << 30          # the design has no position table: int32 positions are the only bound


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json lacks required key {key!r} in {where}")
    return d[key]


@dataclass
class LifusunConfig:
    width: int
    vocab: int
    eps: float
    layers: list = field(default_factory=list)       # the file's "layers" entries, as read

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, c: dict) -> "LifusunConfig":
        cfg = cls(width=int(_get(c, "width", "the file")), vocab=int(_get(c, "vocab", "the file")),
                  eps=float(_get(_get(c, "norm", "the file"), "eps", "norm")),
                  layers=copy.deepcopy(list(_get(c, "layers", "the file"))))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "LifusunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": NAME, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                "layers": copy.deepcopy(self.layers)}

    # ---- checks --------------------------------------------------------------------------
    def validate(self) -> None:
        if self.width <= 0 or self.vocab <= 0:
            raise ConfigError("width and vocab must be positive")
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if not self.layers:
            raise ConfigError("layers is empty")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind, m = _get(layer, "type", where), _get(layer, "mixer", where)
            if kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    _get(m, k, where + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
                if not 0 <= int(m.get("conv") or 0) <= 8:
                    raise ConfigError(f"{where}: conv {m['conv']} taps are not supported (up to 8)")
                if m.get("mask") is not None and int(_get(m["mask"], "size", where + ".mixer.mask")) <= 0:
                    raise ConfigError(f"{where}: mask.size must be positive")
                if m.get("kv_from") is not None:
                    j = int(m["kv_from"])
                    if not 0 <= j < i or self.layers[j].get("type") != "attention" or \
                            self.layers[j]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from {j} must name an earlier attention layer with keys and values of its own")
                    o = self.layers[j]["mixer"]
                    if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"{where}: kv_from {j} has other key/value sizes than this layer")
            elif kind == "retention":
                for k in ("heads", "dim", "vdim", "decay"):
                    _get(m, k, where + ".mixer")
                if len(m["decay"]) != int(m["heads"]):
                    raise ConfigError(f"{where}: decay has {len(m['decay'])} entries for {m['heads']} heads")
                rot = m.get("rot")
                if rot is not None:
                    dims = int(_get(rot, "dims", where + ".mixer.rot"))
                    _get(rot, "base", where + ".mixer.rot")
                    if dims % 2 or dims < 0 or dims > int(m["dim"]):
                        raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {m['dim']}")
            else:
                raise ConfigError(f"{where}: type {kind!r} is not known (attention, retention)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _get(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"{where}: mlp.kind {mlp['kind']!r} is not known (dense)")
                if int(_get(mlp, "ff", where + ".mlp")) <= 0:
                    raise ConfigError(f"{where}: mlp.ff must be positive")

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """The layers as data.  Cache entry i belongs to layer i (pages of keys and values, or a retention state);
        entry L + i holds what layer i's short convolution remembers of each request.  A layer with `kv_from` reads
        the entry of the layer it names and writes none of its own."""
        norm = NormSpec(kind="rmsnorm_scalar", width=self.width, eps=self.eps)
        n = len(self.layers)
        layers, order = [], []
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "attention":
                shared = m.get("kv_from")
                mask = m.get("mask") or {}
                mixer = MixerSpec(kind="talking_attention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), softmax_scale=float(m["scale"]),
                                  options=(("bias", True), ("chunk", int(mask.get("size", 0))), ("conv_taps", int(m.get("conv") or 0)),
                                           ("eps", self.eps), ("own_kv", shared is None), ("slope_exponent", 8.0)))
                order.append(LayerCall(layer=i, cache=i if shared is None else int(shared), write=shared is None,
                                       state=n + i if int(m.get("conv") or 0) > 1 else None))
            else:
                rot = m.get("rot") or {"dims": 0, "base": 10000.0}
                pos = PositionSpec(kind="rope", head_dim=int(m["dim"]), rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   max_position=_MAX_POSITION)
                mixer = MixerSpec(kind="retention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), position=pos if pos.rotary_dim else None,
                                  options=(("decay", tuple(float(d) for d in m["decay"])), ("eps", self.eps)))
                order.append(LayerCall(layer=i, cache=i, write=True))
            if layer.get("mlp") is None:
                layers.append(LayerSpec.of("prenorm_mixer", mixer_norm=norm, mixer=mixer))
            else:
                ff = FeedForwardSpec(kind="swiglu", width=self.width, inner=int(layer["mlp"]["ff"]), activation="silu")
                layers.append(LayerSpec.of("prenorm", mixer_norm=norm, mixer=mixer, feed_forward_norm=norm, feed_forward=ff))
        return ModelSpec(width=self.width, vocab=self.vocab, layers=tuple(layers), order=tuple(order), final_norm=norm,
                         tie_embeddings=False, max_position=_MAX_POSITION)
