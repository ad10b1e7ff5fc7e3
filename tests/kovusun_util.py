"""Helpers of the Kovusun tests: small configurations, a model folder with random weights written from the
checkpoint format alone (names and shapes are stated here, not taken from the product), and the oracle's logits.
The runner that steps the product's own model, cache manager and step function is the one of the Fekulix tests."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from tests.fekulix_util import Runner, rel_err  # noqa: F401  (shared, architecture-free)
from tests.plain import kovusun_plain as plain
from tests.rofozen_util import position_errors, rounded_ok  # noqa: F401  (architecture-free)


def dense(ff=80, limit=1.5):
    return {"ff": ff, "kind": "dense", "limit": limit}


def moe(ff=24, experts=6, top=2, shared=40):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def biased_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=20, scale=0.3, kv_from=None, mlp=None):
    """``attention``: biases, unit norm of q and k, a distance bias."""
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def sink_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=12, scale=0.3, mlp=None):
    """``attention_2``: unit norm, a learned sink, a gate per head."""
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": scale, "vdim": vdim}}


def rotary_layer(heads=4, kv_heads=1, dim=24, vdim=16, window=9, keep_first=3, rot=8, base=100.0, scale=0.2, mlp=None):
    """``attention_3``: rotation of adjacent pairs, a temperature per head, kept first keys."""
    mask = {"size": window}
    if keep_first is not None:
        mask["keep_first"] = keep_first
    return {"type": "attention_3", "mlp": mlp,
            "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": mask, "rot": {"base": base, "dims": rot}, "scale": scale,
                      "vdim": vdim}}


def config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Kovusun", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}


def config_a():
    """Every mixer and both feed-forwards; a layer that reads an earlier layer's keys and values with a LONGER window
    than the owner's (21 against 13, neither a multiple of a page of 16)."""
    return config([
        biased_layer(window=13, mlp=dense()),
        rotary_layer(mlp=moe()),
        biased_layer(window=21, kv_from=0, mlp=moe(top=3, shared=0)),
        sink_layer(mlp=moe(ff=32, experts=4, top=1)),
    ])


def config_b():
    """Sizes that are no multiples of 8 where the format allows: a width of 36, five heads on one key/value head, heads
    of 12 and values of 20, a window of 5 (shorter than a page), a window of one, no kept keys, a whole head rotated, a
    layer without feed-forward, a rotary layer first, one expert chosen of three without a shared expert."""
    return config([
        rotary_layer(heads=5, kv_heads=1, dim=12, vdim=20, window=5, keep_first=0, rot=12, base=37.0, scale=0.4, mlp=moe(ff=20, experts=3, top=1, shared=0)),
        sink_layer(heads=3, kv_heads=3, dim=20, vdim=12, window=1, scale=0.25, mlp=None),
        biased_layer(heads=6, kv_heads=3, dim=12, vdim=12, window=40, scale=0.5, mlp=dense(44, limit=0.75)),
        rotary_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=7, keep_first=9, rot=4, base=1000.0, scale=0.3, mlp=dense(52, limit=3.0)),
    ], width=36, vocab=61, eps=1e-6)


def config_c():
    """Larger and rounder: a width of 256, heads of 128 in one layer (the tensor-core kernels' size) and of 64 and 32
    in others, windows beyond several pages, two readers of one layer's keys and values of which one is the
    last layer, sixteen kept keys (a whole page), eight experts of which two are chosen beside a shared one."""
    own = biased_layer(heads=8, kv_heads=4, dim=32, vdim=32, window=48, scale=0.18, mlp=moe(ff=64, experts=8, top=2, shared=96))
    return config([
        own,
        rotary_layer(heads=4, kv_heads=2, dim=128, vdim=128, window=40, keep_first=16, rot=64, base=50000.0, scale=0.09, mlp=dense(320, limit=2.0)),
        biased_layer(heads=8, kv_heads=4, dim=32, vdim=32, window=96, scale=0.18, kv_from=0, mlp=dense(192, limit=1.0)),
        sink_layer(heads=4, kv_heads=4, dim=64, vdim=32, window=80, scale=0.11, mlp=moe(ff=64, experts=8, top=2, shared=96)),
        biased_layer(heads=8, kv_heads=4, dim=32, vdim=32, window=24, scale=0.18, kv_from=0, mlp=None),
    ], width=256, vocab=640)


def tensor_shapes(raw) -> dict[str, tuple]:
    """Names and shapes of a checkpoint of this configuration."""
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,), "final.norm.b": (w,), "head": (raw["vocab"], w)}
    for i, layer in enumerate(raw["layers"]):
        p, m, q = f"l{i}.", layer["mixer"], f"l{i}.mix."
        h, g, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (w,), p + "norm1.b": (w,), p + "shift": (w,), q + "q": (h * dk, w), q + "o": (w, h * dv)})
        if m.get("kv_from") is None:
            out.update({q + "k": (g * dk, w), q + "v": (g * dv, w)})
        if layer["type"] == "attention":
            out.update({q + "q.b": (h * dk,), q + "r1": (h,), q + "r2": (h,)})
            if m.get("kv_from") is None:
                out.update({q + "k.b": (g * dk,), q + "v.b": (g * dv,)})
        elif layer["type"] == "attention_2":
            out.update({q + "sink": (h,), q + "g": (h, w)})
        else:
            out[q + "temp"] = (h,)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out.update({p + "norm2": (w,), p + "norm2.b": (w,)})
        f = p + "mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            out.update({f + "gate": (ff, w), f + "gate.b": (ff,), f + "up": (ff, w), f + "up.b": (ff,), f + "down": (w, ff), f + "down.b": (w,)})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            out.update({f + "router": (r["experts"], w), f + "router.b": (r["experts"],)})
            for e in range(r["experts"]):
                out.update({f"{f}e{e}.gate": (ff, w), f"{f}e{e}.up": (ff, w), f"{f}e{e}.down": (w, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({f + "shared.gate": (sf, w), f + "shared.up": (sf, w), f + "shared.down": (w, sf), f + "shared.sg": (1, w)})
    return out


def random_weights(raw, seed: int, sharpen: float = 2.5) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices about 1/sqrt(fan-in) so that activations are of size one, the query and key side
    times ``sharpen`` where no unit norm undoes it, routers large enough for clear choices, distance numbers that keep
    the logarithm's argument positive, shift weights between 0 and 1, norm weights around one."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(".b") and len(shape) == 1:
            t = 0.2 * torch.randn(shape, generator=gen)
            if name.endswith("router.b"):
                t = t * 3.0
        elif leaf == "router":
            t = torch.randn(shape, generator=gen) * (3.0 / shape[1] ** 0.5)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=gen) * (1.2 / shape[1] ** 0.5)
            if leaf in ("q", "k"):
                t = t * sharpen ** 0.5
        elif leaf == "shift":
            t = torch.rand(shape, generator=gen)
        elif leaf == "r1":
            t = torch.randn(shape, generator=gen)
        elif leaf == "r2":
            t = 0.05 + torch.rand(shape, generator=gen) * 1.5
        elif leaf == "sink":
            t = torch.randn(shape, generator=gen) * 2.0
        elif leaf == "temp":
            t = 0.5 + torch.rand(shape, generator=gen) * 1.5
        else:  # norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(folder, raw, seed: int, sharpen: float = 2.5, change=None) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=1))
    w = random_weights(raw, seed, sharpen)
    if change:
        change(w)
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return folder


def read_weights(folder) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: v.float() for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}


def oracle(folder, dtype=torch.float32):
    """ids -> logits [T, vocab] of the plain implementation (32-bit: products summed in 64-bit)."""
    raw = json.loads((Path(folder) / "config.json").read_text())
    w = read_weights(folder)
    return lambda ids: plain.forward(w, raw, ids, dtype)


def layer_streams(folder, ids) -> torch.Tensor:
    raw = json.loads((Path(folder) / "config.json").read_text())
    return plain.forward(read_weights(folder), raw, ids, torch.float32, return_layers=True)[1]
