"""Helpers of the Rofozen tests: small configurations, a model folder with random weights written from the
checkpoint format alone (names and shapes are stated here, not taken from the product), and the oracle's logits.
The runner that steps the product's own model, cache manager and step function is the one of the Fekulix tests."""

from __future__ import annotations

import copy
import json
from pathlib import Path

import torch

from tests.fekulix_util import Runner, rel_err  # noqa: F401  (shared, architecture-free)
from tests.plain import rofozen_plain as plain


def dense(ff=80):
    return {"ff": ff, "kind": "dense"}


def moe(ff=24, experts=6, identity=2, top=2, count=2, keep=1, scale=1.5):
    router = {"experts": experts, "identity": identity, "scale": scale, "top": top}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return {"expert": {"ff": ff}, "kind": "moe", "router": router}


def ssm_layer(heads=4, vdim=16, state=8, groups=2, conv=3, norm_groups=2, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}


def latent_layer(heads=3, dim=16, rot=8, vdim=24, rank=24, q_rank=20, window=20, base=100.0, scaling=True, scale=0.3, mlp=None):
    mixer = {"dim": dim, "heads": heads, "kv_rank": rank, "q_rank": q_rank, "rot_dim": rot, "scale": scale, "vdim": vdim}
    if rot:
        mixer["rot"] = {"base": base, "dims": rot}
        if scaling:
            mixer["rot"]["scaling"] = {"factor": 4.0, "fast": 8.0, "original": 64, "slow": 0.5} if scaling is True else dict(scaling)
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Rofozen", "layers": copy.deepcopy(layers), "norm": {"eps": eps}, "vocab": vocab, "width": width}


def shared(layer, of: int):
    """The entry of a layer that runs with layer ``of``'s tensors."""
    out = copy.deepcopy(layer)
    out["weights_of"] = of
    return out


def config_a():
    """Both mixers and both feed-forwards; a latent layer that runs twice with one set of tensors; a window of 20
    (more than a page of 16, no multiple of it)."""
    lat = latent_layer(mlp=moe())
    return config([ssm_layer(mlp=dense()), lat, ssm_layer(heads=2, vdim=24, state=16, groups=1, conv=4, norm_groups=1, mlp=moe(top=3, count=0)),
                   shared(lat, 1)])


def config_b():
    """Sizes that are no multiples of 8 where the format allows: a width of 36, five heads on one group, a state of
    12, two taps, a window of 5 (shorter than a page), one choice per token among experts without identity experts or
    groups, three groups of which two are kept, a layer without feed-forward, a latent layer first, no rescaling."""
    return config([
        latent_layer(heads=5, dim=12, rot=4, vdim=20, rank=28, q_rank=12, window=5, base=37.0, scaling=None, scale=0.5,
                     mlp=moe(ff=20, experts=5, identity=0, top=1, count=0, scale=1.0)),
        ssm_layer(heads=5, vdim=12, state=12, groups=1, conv=2, norm_groups=5, mlp=None),
        ssm_layer(heads=6, vdim=8, state=20, groups=3, conv=4, norm_groups=3, mlp=moe(ff=28, experts=7, identity=2, top=4, count=3, keep=2, scale=0.7)),
        latent_layer(heads=2, dim=24, rot=16, vdim=8, rank=40, q_rank=36, window=None, scaling={"factor": 1.5, "fast": 4.0, "original": 16,
                                                                                                 "slow": 1.0}, mlp=dense(44)),
    ], width=36, vocab=61, eps=1e-6)


def config_c():
    """Larger and rounder: a width of 256, a state of 64 under heads of 32, a latent of 112 with 16 rotated channels
    (a cache entry of 128 numbers), a window of 96, eight experts and no identity expert, a state-space layer that runs
    three times (a chain of borrowed tensors), one tap (no convolution state)."""
    s = ssm_layer(heads=8, vdim=32, state=64, groups=4, conv=4, norm_groups=4, mlp=moe(ff=64, experts=8, identity=0, top=2, count=4, keep=2))
    return config([
        s, shared(s, 0), shared(s, 1),
        latent_layer(heads=4, dim=48, rot=16, vdim=64, rank=112, q_rank=64, window=96, base=5000.0, scale=0.12, mlp=dense(320)),
        ssm_layer(heads=4, vdim=64, state=16, groups=4, conv=1, norm_groups=1, mlp=dense(192)),
    ], width=256, vocab=576)


def tensor_shapes(raw) -> dict[str, tuple]:
    """Names and shapes of a checkpoint of this configuration."""
    w = raw["width"]
    out = {"embed": (raw["vocab"], w), "final.norm": (w,), "head": (raw["vocab"], w)}
    for i, layer in enumerate(raw["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m, q = f"l{i}.", layer["mixer"], f"l{i}.mix."
        out[p + "norm1"] = (w,)
        if layer["type"] == "mamba2":
            inner, gn, h = m["heads"] * m["vdim"], m["groups"] * m["state"], m["heads"]
            out.update({q + "in": (2 * inner + 2 * gn + h, w), q + "conv": (inner + 2 * gn, m["conv"]), q + "conv.b": (inner + 2 * gn,),
                        q + "dt_bias": (h,), q + "A_log": (h,), q + "D": (h,), q + "norm": (inner,), q + "o": (w, inner)})
        else:
            h, dk, rd, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({q + "dq": (qr, w), q + "dq.norm": (qr,), q + "uq": (h * (dk + rd), qr), q + "dkv": (r + rd, w), q + "dkv.norm": (r,),
                        q + "uk": (h * dk, r), q + "uv": (h * dv, r), q + "sink": (h,), q + "o": (w, h * dv)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (w,)
        f = p + "mlp."
        if mlp["kind"] == "dense":
            out.update({f + "gate": (mlp["ff"], w), f + "up": (mlp["ff"], w), f + "down": (w, mlp["ff"])})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            total = r["experts"] + r.get("identity", 0)
            out.update({f + "router": (total, w), f + "correction": (total,)})
            for e in range(r["experts"]):
                out.update({f"{f}e{e}.gate": (ff, w), f"{f}e{e}.up": (ff, w), f"{f}e{e}.down": (w, ff)})
    return out


def random_weights(raw, seed: int, sharpen: float = 2.5) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices about 1/sqrt(fan-in) so that activations are of size one, the query and key side
    times ``sharpen`` so that attention is peaked, routers large enough for clear choices, decays between slow and
    fast, norm weights around one."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(raw).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith("conv.b"):
            t = 0.2 * torch.randn(shape, generator=gen)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) * 0.6
        elif leaf == "router":
            t = torch.randn(shape, generator=gen) * (3.0 / shape[1] ** 0.5)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=gen) * (1.2 / shape[1] ** 0.5)
            if leaf in ("uq", "uk", "dkv"):
                t = t * sharpen ** 0.5
        elif leaf == "correction":
            t = 0.1 * torch.randn(shape, generator=gen)
        elif leaf == "sink":
            t = torch.randn(shape, generator=gen)
        elif leaf == "A_log":
            t = torch.rand(shape, generator=gen) * 2.5 - 2.0  # exp(A) from 0.14 to 1.6
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=gen) - 1.0
        elif leaf == "D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
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
    return lambda ids: plain.forward(raw, w, ids, dtype)


def layer_streams(folder, ids) -> list[torch.Tensor]:
    raw = json.loads((Path(folder) / "config.json").read_text())
    out: list = []
    plain.forward(raw, read_weights(folder), ids, torch.float32, out)
    return out


def position_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: the distance of the logits (mean taken off, root mean square over the vocabulary) over the
    oracle's spread."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    spread = (want.double() - want.double().mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(dim=-1).sqrt() / spread


def rounded_ok(got: torch.Tensor, want: torch.Tensor, want_rounded: torch.Tensor, floor: float = 0.1) -> tuple[bool, str]:
    """Whether bfloat16 logits are as near the 32-bit oracle's as rounding allows. ``want_rounded`` is the oracle
    run in bfloat16: its own distance says what rounding alone costs. Random weights make single positions sharp
    (two keys that nearly tie, a choice of experts on the edge), and the engine rounds in other places than the oracle,
    so a single position says little (one other expert early in a short sequence moves every position behind it a little); the median stays under 0.1 or twice the
    oracle's, and at most a quarter of the positions are farther than three times the oracle's distance there
    (at least 0.3). A lost key, a stale state or a wrong slot costs 0.3 to 1 at every position behind it; faults
    of single positions are what the 32-bit runs and the tests of each mechanism are for."""
    err, noise = position_errors(got, want), position_errors(want_rounded, want)
    far = err > torch.clamp(3.0 * noise, min=0.3)
    ok = err.median() <= max(floor, 2.0 * noise.median().item()) and int(far.sum()) <= max(1, err.numel() // 4)
    return bool(ok), (f"median {err.median():.3f} against the oracle's {noise.median():.3f}; {int(far.sum())} of {err.numel()} positions far off "
                      f"(worst {err.max():.3f} at {int(err.argmax())})")
