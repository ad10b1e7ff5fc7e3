"""Typed configuration of the Rofozen decoder, read from its config.json.

config.json carries ``architecture``, ``width``, ``vocab``, ``norm.eps`` and ``layers``: one entry per layer with
``type`` (``mamba2`` or ``latent_attention``), the mixer's sizes and constants under ``mixer``, the feed-forward under
``mlp`` (``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {...}}`` or null), and
optionally ``weights_of``: the index of the layer whose tensors this one runs with (a cache and state of its own).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

LAYER_TYPES = ("mamba2", "latent_attention")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RofozenLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None  # None: no feed-forward
    weights_of: int | None  # the layer whose tensors this one runs with (the end of a chain), or None


@dataclass(frozen=True)
class RofozenConfig:
    width: int
    vocab: int
    eps: float
    layers: tuple[RofozenLayer, ...]
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RofozenConfig":
        missing = [k for k in ("width", "vocab", "layers", "norm") if k not in raw]
        if missing:
            raise KeyError(f"config.json lacks {missing}")
        entries = raw["layers"]
        layers = []
        for i, entry in enumerate(entries):
            kind = entry.get("type")
            if kind not in LAYER_TYPES:
                raise NotImplementedError(f"layer {i}: type {kind!r} is not one of {LAYER_TYPES}")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind") not in MLP_KINDS:
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not one of {MLP_KINDS}")
            of = entry.get("weights_of")
            if of is not None:
                of, seen = int(of), {i}
                while 0 <= of < len(entries) and of not in seen and entries[of].get("weights_of") is not None:
                    seen.add(of)  # a layer that borrows from a borrower runs with the tensors at the end of the chain
                    of = int(entries[of]["weights_of"])
                if not 0 <= of < len(entries) or of in seen:
                    raise ValueError(f"layer {i}: weights_of={entry.get('weights_of')} must lead to another layer that has tensors of its own")
                if entries[of].get("type") != kind:
                    raise ValueError(f"layer {i} ({kind}) cannot run with the weights of layer {of} ({entries[of].get('type')})")
            layers.append(RofozenLayer(kind, entry["mixer"], mlp, of))
        cfg = cls(width=int(raw["width"]), vocab=int(raw["vocab"]), eps=float(raw["norm"]["eps"]), layers=tuple(layers), raw=raw)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1 or not self.layers:
            raise ValueError("width, vocab and the number of layers must be positive")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "mamba2":
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    if int(m[key]) < 1:
                        raise ValueError(f"layer {i}: {key}={m[key]} must be positive")
                if int(m["heads"]) % int(m["groups"]):
                    raise ValueError(f"layer {i}: {m['heads']} heads are not a multiple of {m['groups']} groups")
                if (int(m["heads"]) * int(m["vdim"])) % int(m["norm_groups"]):
                    raise ValueError(f"layer {i}: {int(m['heads']) * int(m['vdim'])} channels do not split into {m['norm_groups']} equal parts")
            else:
                for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                    if int(m[key]) < 1:
                        raise ValueError(f"layer {i}: {key}={m[key]} must be positive")
                rd = int(m.get("rot_dim", 0))
                rot = m.get("rot")
                if rd and (rot is None or int(rot["dims"]) != rd or rd % 2):
                    raise ValueError(f"layer {i}: the rotated part ({rd}) must be even and equal rot.dims")
                mask = m.get("mask")
                if mask is not None and int(mask["size"]) < 1:
                    raise ValueError(f"layer {i}: mask.size={mask['size']} must be positive")
            mlp = layer.mlp
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp["router"]
                total = int(r["experts"]) + int(r.get("identity", 0))
                if not 1 <= int(r["top"]) <= total:
                    raise ValueError(f"layer {i}: top={r['top']} of {total} experts")
                g = r.get("groups")
                if g is not None:
                    count, keep = int(g["count"]), int(g["keep"])
                    if count < 1 or total % count or not 1 <= keep <= count:
                        raise ValueError(f"layer {i}: {total} experts in {count} groups, {keep} kept")
                    if keep * (total // count) < int(r["top"]):
                        raise ValueError(f"layer {i}: {keep} groups of {total // count} experts cannot give {r['top']} choices")
