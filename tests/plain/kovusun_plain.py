"""The Kovusun decoder restated in plain PyTorch: whole sequences, no cache, one function per mechanism.

Written from the design's equations and used as the oracle of the tests; it shares no code with the engine.
``weights`` maps tensor names to tensors; ``cfg`` is the config.json dict. ``dtype`` float32 computes everything
in 32-bit; bfloat16 rounds the products' inputs and outputs to bfloat16 where the engine may, and keeps in
32-bit what the design keeps there (norms, routers, angles, scores and softmax weights, the residual sum)."""

from __future__ import annotations

import math

import torch


def _lin(x: torch.Tensor, w: torch.Tensor, dtype, b: torch.Tensor | None = None) -> torch.Tensor:
    """W x (+ b) with the operands in ``dtype`` and the sum in 32-bit (64-bit sums for float32: the order does not matter then)."""
    if dtype == torch.float32:
        y = (x.double() @ w.double().t()).float()
        return y if b is None else y + b.float()
    y = (x.to(dtype).float() @ w.to(dtype).float().t()).to(dtype).float()
    return y if b is None else (y + b.float()).to(dtype).float()


def _r(x: torch.Tensor, dtype) -> torch.Tensor:
    return x if dtype == torch.float32 else x.to(dtype).float()


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = x.float()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.float() + b.float()


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """h_t + (h_(t-1) - h_t) * mix, with zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * mix.float()


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i+1) for i < dims / 2 turn by positions * base^(-2i/dims); the rest pass."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).float()
    ang = positions.float()[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(n: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """[n, n] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attend(q, k, v, scale, mask, head_scale=None, dist=None, sink=None, dtype=torch.float32):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]. ``head_scale`` [H] multiplies the scaled scores;
    ``dist`` = (r1 [H], r2 [H]) takes r1 ln(1 + r2 (i - j)) off them; ``sink`` [H] adds exp(sink_h) to the denominator."""
    t, heads, _ = q.shape
    rep = heads // k.shape[1]
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", _r(q, dtype), _r(kk, dtype)) * scale
    if head_scale is not None:
        s = s * head_scale.float()[:, None, None]
    if dist is not None:
        r1, r2 = dist
        gap = (torch.arange(t)[:, None] - torch.arange(t)[None, :]).clamp(min=0).float()
        s = s - r1.float()[:, None, None] * torch.log(1.0 + r2.float()[:, None, None] * gap[None])
    s = s.masked_fill(~mask[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.float()[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.float()[:, None, None] - m)
    p = e / den
    return torch.einsum("hij,jhd->ihd", _r(p, dtype), _r(vv, dtype))


def keys_values(weights, prefix: str, c: dict, kind: str, h, positions, eps, dtype):
    """A layer's own normed (and rotated) keys [T, G, d] and values [T, G, dv]."""
    t = h.shape[0]
    g, d, dv = int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    bias = kind == "attention"
    k = _lin(h, weights[prefix + "k"], dtype, weights[prefix + "k.b"] if bias else None).view(t, g, d)
    v = _lin(h, weights[prefix + "v"], dtype, weights[prefix + "v.b"] if bias else None).view(t, g, dv)
    if kind == "attention_3":
        k = rotate_pairs(k, positions, int(c["rot"]["dims"]), float(c["rot"]["base"]))
    else:
        k = unit_rms(k, eps)
    return _r(k, dtype), _r(v, dtype)


def attention_mixer(weights, prefix: str, c: dict, kind: str, h, positions, eps, dtype, kv=None):
    """One of the three attention mixers on its (shifted) input h [T, width]. ``kv``: another layer's keys and values."""
    t = h.shape[0]
    heads, d, dv = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    q = _lin(h, weights[prefix + "q"], dtype, weights[prefix + "q.b"] if kind == "attention" else None).view(t, heads, d)
    k, v = kv if kv is not None else keys_values(weights, prefix, c, kind, h, positions, eps, dtype)
    mask = c["mask"]
    if kind == "attention":
        q = unit_rms(q, eps)
        o = attend(q, k, v, float(c["scale"]), visible(t, int(mask["size"])),
                   dist=(weights[prefix + "r1"], weights[prefix + "r2"]), dtype=dtype)
    elif kind == "attention_2":
        q = unit_rms(q, eps)
        o = attend(q, k, v, float(c["scale"]), visible(t, int(mask["size"])), sink=weights[prefix + "sink"], dtype=dtype)
        gate = torch.sigmoid(_lin(h, weights[prefix + "g"], dtype))
        o = o * gate[:, :, None]
    elif kind == "attention_3":
        q = rotate_pairs(q, positions, int(c["rot"]["dims"]), float(c["rot"]["base"]))
        o = attend(q, k, v, float(c["scale"]), visible(t, int(mask["size"]), int(mask.get("keep_first", 0))),
                   head_scale=weights[prefix + "temp"], dtype=dtype)
    else:
        raise ValueError(kind)
    return _lin(_r(o.reshape(t, heads * dv), dtype), weights[prefix + "o"], dtype), (k, v)


def dense_ff(weights, prefix: str, mlp: dict, h, dtype):
    lim = float(mlp["limit"])
    g = torch.clamp(_lin(h, weights[prefix + "gate"], dtype, weights[prefix + "gate.b"]), max=lim)
    u = torch.clamp(_lin(h, weights[prefix + "up"], dtype, weights[prefix + "up.b"]), min=-lim, max=lim)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return _lin(_r(y, dtype), weights[prefix + "down"], dtype, weights[prefix + "down.b"])


def gated_expert(weights, prefix: str, h, dtype):
    g = _lin(h, weights[prefix + "gate"], dtype)
    u = _lin(h, weights[prefix + "up"], dtype)
    return _lin(_r(g * torch.sigmoid(g) * u, dtype), weights[prefix + "down"], dtype)


def route(weights, prefix: str, mlp: dict, h, dtype):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen logits only."""
    z = _r(h, dtype).double() @ weights[prefix + "router"].double().t() + weights[prefix + "router.b"].double()
    z = z.float()
    top = int(mlp["router"]["top"])
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(weights, prefix: str, mlp: dict, h, dtype):
    idx, wgt = route(weights, prefix, mlp, h, dtype)
    out = torch.zeros_like(h, dtype=torch.float32)
    for e in range(int(mlp["router"]["experts"])):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += wgt[rows, slot][:, None] * gated_expert(weights, f"{prefix}e{e}.", h[rows], dtype)
    if mlp.get("shared"):
        share = torch.sigmoid(_lin(h, weights[prefix + "shared.sg"], dtype))  # [T, 1]
        out = out + share * gated_expert(weights, prefix + "shared.", h, dtype)
    return out


def forward(weights, cfg: dict, tokens, dtype=torch.float32, return_layers: bool = False):
    """Logits [T, vocab] (float32) of one whole sequence; with ``return_layers`` also the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = weights["embed"].float()[tokens]
    kept: dict[int, tuple] = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        c = layer["mixer"]
        h1 = _r(layer_norm(x, weights[p + "norm1"], weights[p + "norm1.b"], eps), dtype)
        h1 = _r(token_shift(h1, weights[p + "shift"]), dtype)
        src = c.get("kv_from")
        y, kept[i] = attention_mixer(weights, p + "mix.", c, layer["type"], h1, positions, eps, dtype,
                                     kv=kept[int(src)] if src is not None else None)
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = _r(layer_norm(x, weights[p + "norm2"], weights[p + "norm2.b"], eps), dtype)
            y = y + (dense_ff(weights, p + "mlp.", mlp, h2, dtype) if mlp["kind"] == "dense" else moe_ff(weights, p + "mlp.", mlp, h2, dtype))
        x = x + y
        streams.append(x.clone())
    h = _r(layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps), dtype)
    logits = _lin(h, weights["head"], dtype) if dtype == torch.float32 else (h.to(dtype).float() @ weights["head"].to(dtype).float().t())
    return (logits, torch.stack(streams)) if return_layers else logits
