"""Typed configuration of the Rodapel family, read from its config.json.

Keys: "architecture" ("Rodapel"), "width", "vocab", "norm" {"eps"} and "layers", a list whose entries give "type"
(which mixer the layer has), the mixer's sizes under "mixer" and the feed-forward under "mlp" (null: none).

Mixers:
  "latent_attention"  "heads", "dim" (unrotated query/key numbers of a head), "rot_dim" (rotated ones), "vdim",
                      "kv_rank" (width of the latent row that is cached), "scale", "rot" {"dims", "base"}.
  "attention"         "heads", "kv_heads", "dim", "vdim", "scale", "mask" {"size"} (sliding window; absent: causal).
  "wkv"               "heads", "dim".  The rank of the decay's two-matrix projection is the row count of the
                      checkpoint's tensor `l<i>.mix.w1`; a config without a checkpoint (random weights) names it
                      as "decay_rank".
Feed-forwards:
  {"kind": "dense", "ff", "limit"}
  {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "identity"}}

Every size is read from the file (or from a tensor's shape); a missing key is an error at once.
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field

from .errors import ConfigError
from .specs import EmbeddingSpec, FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec

NAME = "Rodapel"
_MAX_POSITION = 1 << 30          # the design has no position table: int32 positions are the only bound
GLU_SLOPE = 1.702                # the design fixes the slope of the gate's sigmoid


def _get(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json lacks required key {key!r} in {where}")
    return d[key]


@dataclass
class RodapelConfig:
    width: int
    vocab: int
    eps: float
    layers: list = field(default_factory=list)       # the file's "layers" entries, as read

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, c: dict) -> "RodapelConfig":
        cfg = cls(width=int(_get(c, "width", "the file")), vocab=int(_get(c, "vocab", "the file")),
                  eps=float(_get(_get(c, "norm", "the file"), "eps", "norm")),
                  layers=copy.deepcopy(list(_get(c, "layers", "the file"))))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "RodapelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": NAME, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                "layers": copy.deepcopy(self.layers)}

    def with_checkpoint_shapes(self, shapes: dict) -> "RodapelConfig":
        """The sizes that only a tensor's shape gives (`shapes`: {checkpoint tensor name: shape})."""
        for i, layer in enumerate(self.layers):
            if layer["type"] == "wkv":
                shape = shapes.get(f"l{i}.mix.w1")
                if shape is not None and len(shape) == 2:
                    layer["mixer"]["decay_rank"] = int(shape[0])
        return self

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
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    _get(m, k, where + ".mixer")
                rot = _get(m, "rot", where + ".mixer")
                dims = int(_get(rot, "dims", where + ".mixer.rot"))
                _get(rot, "base", where + ".mixer.rot")
                if dims % 2 or dims < 0 or dims > int(m["rot_dim"]):
                    raise ConfigError(f"{where}: rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
            elif kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim", "scale"):
                    _get(m, k, where + ".mixer")
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
                if m.get("mask") is not None and int(_get(m["mask"], "size", where + ".mixer.mask")) <= 0:
                    raise ConfigError(f"{where}: mask.size must be positive")
            elif kind == "wkv":
                for k in ("heads", "dim"):
                    _get(m, k, where + ".mixer")
            else:
                raise ConfigError(f"{where}: type {kind!r} is not known (latent_attention, attention, wkv)")
            if any(int(v) <= 0 for k, v in m.items() if k in ("heads", "kv_heads", "dim", "vdim", "kv_rank", "rot_dim")):
                raise ConfigError(f"{where}: sizes must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            ff_kind = _get(mlp, "kind", where + ".mlp")
            if ff_kind == "dense":
                if int(_get(mlp, "ff", where + ".mlp")) <= 0:
                    raise ConfigError(f"{where}: mlp.ff must be positive")
                _get(mlp, "limit", where + ".mlp")
            elif ff_kind == "moe":
                e, r = _get(mlp, "expert", where + ".mlp"), _get(mlp, "router", where + ".mlp")
                if int(_get(e, "ff", where + ".mlp.expert")) <= 0:
                    raise ConfigError(f"{where}: mlp.expert.ff must be positive")
                _get(e, "limit", where + ".mlp.expert")
                experts, top = int(_get(r, "experts", where + ".mlp.router")), int(_get(r, "top", where + ".mlp.router"))
                identity = int(r.get("identity") or 0)
                if experts < 0 or identity < 0 or not 1 <= top <= experts + identity:
                    raise ConfigError(f"{where}: router takes {top} of {experts} + {identity} experts")
            else:
                raise ConfigError(f"{where}: mlp.kind {ff_kind!r} is not known (dense, moe)")

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        """The layers as data.  Cache entry i belongs to layer i (pages of latent rows, pages of keys and values under
        a window, or a wkv state); entry L + i holds the previous token's input row of a wkv layer i."""
        norm = NormSpec(kind="rmsnorm", width=self.width, eps=self.eps)
        n = len(self.layers)
        layers, order = [], []
        for i, layer in enumerate(self.layers):
            m, kind = layer["mixer"], layer["type"]
            state = None
            if kind == "latent_attention":
                rot = m["rot"]
                pos = PositionSpec(kind="rope", head_dim=int(m["rot_dim"]), rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   max_position=_MAX_POSITION, pairing="interleaved")
                mixer = MixerSpec(kind="latent_attention", width=self.width, heads=int(m["heads"]), kv_heads=1,
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), softmax_scale=float(m["scale"]),
                                  position=pos if pos.rotary_dim else None,
                                  options=(("eps", self.eps), ("kv_rank", int(m["kv_rank"])), ("rot_dim", int(m["rot_dim"]))))
            elif kind == "attention":
                mask = m.get("mask") or {}
                mixer = MixerSpec(kind="gated_attention", width=self.width, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["vdim"]), window=int(mask.get("size", 0)),
                                  softmax_scale=float(m["scale"]),
                                  options=(("eps", self.eps), ("head_gate", True), ("qk_norm", True)))
            else:
                rank = m.get("decay_rank")
                if rank is None:
                    raise ConfigError(f"layers[{i}]: the rank of the wkv decay projection is neither in the file (decay_rank) "
                                      "nor known from a checkpoint's tensor shapes")
                mixer = MixerSpec(kind="wkv", width=self.width, heads=int(m["heads"]), kv_heads=int(m["heads"]),
                                  head_dim=int(m["dim"]), value_dim=int(m["dim"]),
                                  options=(("decay_rank", int(rank)), ("eps", self.eps)))
                state = n + i
            order.append(LayerCall(layer=i, cache=i, write=True, state=state))
            mlp = layer.get("mlp")
            if mlp is None:
                layers.append(LayerSpec.of("branchnorm_mixer", mixer=mixer, mixer_norm=norm))
                continue
            if mlp["kind"] == "dense":
                ff = FeedForwardSpec(kind="clamped_glu", width=self.width, inner=int(mlp["ff"]), activation="sigmoid_glu",
                                     options=(("limit", float(mlp["limit"])), ("slope", GLU_SLOPE)))
            else:
                r = mlp["router"]
                ff = FeedForwardSpec(kind="routed_glu", width=self.width, inner=int(mlp["expert"]["ff"]), activation="sigmoid_glu",
                                     experts=int(r["experts"]), experts_per_token=int(r["top"]),
                                     options=(("identity", int(r.get("identity") or 0)), ("limit", float(mlp["expert"]["limit"])),
                                              ("slope", GLU_SLOPE)))
            layers.append(LayerSpec.of("branchnorm", mixer=mixer, mixer_norm=norm, feed_forward=ff, feed_forward_norm=norm))
        emb = EmbeddingSpec(kind="table_norm", vocab=self.vocab, width=self.width, options=(("eps", self.eps),))
        return ModelSpec(width=self.width, vocab=self.vocab, layers=tuple(layers), order=tuple(order), final_norm=norm,
                         tie_embeddings=False, max_position=_MAX_POSITION, embedding=emb)
