"""Typed configuration of the Kovusun decoder, read from its config.json.

config.json carries ``architecture``, ``width``, ``vocab``, ``norm.eps`` and ``layers``: one entry per layer with
``type`` (``attention``, ``attention_2`` or ``attention_3``), the mixer's sizes and constants under ``mixer`` (``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, and by type ``mask.keep_first``, ``rot.base`` / ``rot.dims``,
``kv_from``: an earlier layer with projections of its own whose cached keys and values this one reads, as that layer's
cache holds them), and the feed-forward under ``mlp``
(``{"kind": "dense", "ff": n, "limit": x}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": e, "top": k},
"shared": {"ff": n}}`` or null).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

LAYER_TYPES = ("attention", "attention_2", "attention_3")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class KovusunLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None  # None: no feed-forward
    kv_from: int | None  # the layer whose cached keys and values this one reads, or None

    @property
    def window(self) -> int:
        return int(self.mixer["mask"]["size"])

    @property
    def keep_first(self) -> int:
        return int(self.mixer["mask"].get("keep_first", 0) or 0) if self.type == "attention_3" else 0


@dataclass(frozen=True)
class KovusunConfig:
    width: int
    vocab: int
    eps: float
    layers: tuple[KovusunLayer, ...]
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KovusunConfig":
        missing = [k for k in ("width", "vocab", "layers", "norm") if k not in raw]
        if missing:
            raise KeyError(f"config.json lacks {missing}")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            kind = entry.get("type")
            if kind not in LAYER_TYPES:
                raise NotImplementedError(f"layer {i}: type {kind!r} is not one of {LAYER_TYPES}")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind") not in MLP_KINDS:
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not one of {MLP_KINDS}")
            src = entry["mixer"].get("kv_from")
            layers.append(KovusunLayer(kind, entry["mixer"], mlp, None if src is None else int(src)))
        cfg = cls(width=int(raw["width"]), vocab=int(raw["vocab"]), eps=float(raw["norm"]["eps"]), layers=tuple(layers), raw=raw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1 or not self.layers:
            raise ValueError("width, vocab and the number of layers must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if int(m[key]) < 1:
                    raise ValueError(f"layer {i}: {key}={m[key]} must be positive")
            if int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"layer {i}: {m['heads']} query heads are not a multiple of {m['kv_heads']} key/value heads")
            if layer.window < 1 or layer.keep_first < 0:
                raise ValueError(f"layer {i}: mask {dict(m['mask'])} needs a positive size and no negative keep_first")
            if layer.type == "attention_3":
                rot = m.get("rot")
                if rot is not None and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["dim"])):
                    raise ValueError(f"layer {i}: rot.dims={rot['dims']} must be even and at most dim={m['dim']}")
            if layer.kv_from is not None:
                j = layer.kv_from
                if not 0 <= j < i or self.layers[j].kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from={j} must name an earlier layer with keys and values of its own")
                o = self.layers[j].mixer
                if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                    raise ValueError(f"layer {i} cannot read the keys and values of layer {j}: kv_heads, dim and vdim must agree")
            mlp = layer.mlp
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp["router"]
                if not 1 <= int(r["top"]) <= int(r["experts"]):
                    raise ValueError(f"layer {i}: top={r['top']} of {r['experts']} experts")
