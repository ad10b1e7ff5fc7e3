"""The Rofozen decoder restated in plain PyTorch: whole sequences, no cache, one function per mechanism.

Written from the design's equations and used as the oracle of the tests; it shares no code with the engine.
``weights`` maps tensor names to tensors; ``cfg`` is the config.json dict. ``dtype`` float32 computes everything
in 32-bit; bfloat16 rounds the products' inputs and outputs to bfloat16 where the engine may, and keeps in
32-bit what the design keeps there (norms, routers, angles, scores, the recurrence and what enters it)."""

from __future__ import annotations

import math

import numpy as np
import torch


def _lin(x: torch.Tensor, w: torch.Tensor, dtype) -> torch.Tensor:
    """W x with the operands in ``dtype`` and the sum in 32-bit (64-bit sums for float32: the order does not matter then)."""
    if dtype == torch.float32:
        return (x.double() @ w.double().t()).float()
    return (x.to(dtype).float() @ w.to(dtype).float().t()).to(dtype).float()


def _r(x: torch.Tensor, dtype) -> torch.Tensor:
    return x if dtype == torch.float32 else x.to(dtype).float()


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w.float()


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------------------------------------- rotation
def yarn_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[np.ndarray, float]:
    """(frequencies of the dims / 2 pairs in float64, factor on cos and sin)."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """x [T, ..., d]: the first ``dims`` channels turn by halves (channel i with i + dims / 2), the rest pass."""
    f, mag = yarn_frequencies(dims, base, scaling)
    f32 = torch.from_numpy(f.astype(np.float32))
    ang = positions.float()[:, None] * f32[None, :]  # 32-bit angle
    cos = torch.from_numpy(np.cos(ang.double().numpy())).float() * mag
    sin = torch.from_numpy(np.sin(ang.double().numpy())).float() * mag
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = cos.view(shape), sin.view(shape)
    u, v = x[..., : dims // 2].float(), x[..., dims // 2: dims].float()
    return torch.cat((u * cos - v * sin, v * cos + u * sin, x[..., dims:].float()), dim=-1)


# ---------------------------------------------------------------------------------------------- mixers
def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x [T, C]; w [C, taps], the last column is the current token's; zeros before the start."""
    t, c = x.shape
    taps = w.shape[1]
    pad = torch.cat((torch.zeros(taps - 1, c), x.float()), dim=0)
    out = b.float()[None, :].repeat(t, 1)
    for j in range(taps):
        out = out + pad[j: j + t] * w.float()[:, j][None, :]
    return out


def mamba2(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, dtype) -> torch.Tensor:
    heads, vd, n, g = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * vd
    t = h.shape[0]
    proj = _lin(h, w[p + "in"], dtype)
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * g * n], proj[:, 2 * inner + 2 * g * n:]
    xbc = _r(silu(_r(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]), dtype)), dtype)
    x = xbc[:, :inner].view(t, heads, vd)
    bm = xbc[:, inner: inner + g * n].view(t, g, n)
    cm = xbc[:, inner + g * n:].view(t, g, n)
    dt = torch.nn.functional.softplus(dt.float() + w[p + "dt_bias"].float(), threshold=1e9)
    a = torch.exp(-torch.exp(w[p + "A_log"].float())[None, :] * dt)  # [T, heads]
    d = w[p + "D"].float()
    per = heads // g
    y = torch.zeros(t, heads, vd)
    state = torch.zeros(heads, n, vd)
    for s in range(t):
        for hd in range(heads):
            grp = hd // per
            state[hd] = a[s, hd] * state[hd] + dt[s, hd] * torch.outer(bm[s, grp], x[s, hd])
            y[s, hd] = state[hd].t() @ cm[s, grp] + d[hd] * x[s, hd]
    y = y.reshape(t, inner) * silu(z.float())
    parts = int(m["norm_groups"])
    y = rms(y.view(t, parts, inner // parts), eps).reshape(t, inner) * w[p + "norm"].float()
    return _lin(_r(y, dtype), w[p + "o"], dtype)


def mamba2_fast(h, w, p, m, eps, dtype, acc=torch.float32):
    """The same as ``mamba2`` with the recurrence over all heads at once (for long sequences). ``acc`` float64 keeps
    everything that ``mamba2`` keeps in 32-bit in 64-bit instead: what the equations give before rounding, to tell a
    position where the layer itself amplifies rounding (a part of y with a tiny root mean square) from an error."""
    heads, vd, n, g = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = heads * vd
    t = h.shape[0]
    proj = (h.double() @ w[p + "in"].double().t()).to(acc) if dtype == torch.float32 else _lin(h, w[p + "in"], dtype)
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * g * n], proj[:, 2 * inner + 2 * g * n:]
    taps = w[p + "conv"].shape[1]
    pad = torch.cat((torch.zeros(taps - 1, xbc.shape[1], dtype=acc), xbc.to(acc)), dim=0)
    conv = w[p + "conv.b"].to(acc)[None, :].repeat(t, 1)
    for j in range(taps):
        conv = conv + pad[j: j + t] * w[p + "conv"].to(acc)[:, j][None, :]
    xbc = _r(silu(_r(conv, dtype)), dtype)
    x = xbc[:, :inner].view(t, heads, vd)
    per = heads // g
    bm = xbc[:, inner: inner + g * n].view(t, g, n).repeat_interleave(per, dim=1)
    cm = xbc[:, inner + g * n:].view(t, g, n).repeat_interleave(per, dim=1)
    dt = torch.nn.functional.softplus(dt.to(acc) + w[p + "dt_bias"].to(acc), threshold=1e9)
    a = torch.exp(-torch.exp(w[p + "A_log"].to(acc))[None, :] * dt)
    d = w[p + "D"].to(acc)
    y = torch.zeros(t, heads, vd, dtype=acc)
    state = torch.zeros(heads, n, vd, dtype=acc)
    for s in range(t):
        state = a[s][:, None, None] * state + dt[s][:, None, None] * (bm[s][:, :, None] * x[s][:, None, :])
        y[s] = (state * cm[s][:, :, None]).sum(1) + d[:, None] * x[s]
    y = y.reshape(t, inner) * silu(z.to(acc))
    parts = int(m["norm_groups"])
    y = y.view(t, parts, inner // parts)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(t, inner) * w[p + "norm"].to(acc)
    if dtype == torch.float32:
        return (y.double() @ w[p + "o"].double().t()).to(acc)
    return _lin(_r(y.float(), dtype), w[p + "o"], dtype)


def latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float, dtype) -> torch.Tensor:
    heads, dim, rd, vd, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    t = h.shape[0]
    pos = torch.arange(t)
    rot = m.get("rot") or {}
    cq = _r(rms_norm(_lin(h, w[p + "dq"], dtype), w[p + "dq.norm"], eps), dtype)
    q = _lin(cq, w[p + "uq"], dtype).view(t, heads, dim + rd)
    kv = _lin(h, w[p + "dkv"], dtype)
    c = _r(rms_norm(kv[:, :rank], w[p + "dkv.norm"], eps), dtype)
    k_rot = kv[:, rank:]
    q_rot = q[..., dim:]
    if rd:
        k_rot = _r(rotate(k_rot, pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling")), dtype)
        q_rot = _r(rotate(q_rot, pos, int(rot["dims"]), float(rot["base"]), rot.get("scaling")), dtype)
    k = _lin(c, w[p + "uk"], dtype).view(t, heads, dim)
    v = _lin(c, w[p + "uv"], dtype).view(t, heads, vd)
    scores = torch.einsum("ihd,jhd->hij", q[..., :dim].float(), k.float()) + torch.einsum("ihd,jd->hij", q_rot.float(), k_rot.float())
    scores = scores * float(m["scale"])
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i)
    mask = m.get("mask")
    if mask:
        seen = seen & (i - j < int(mask["size"]))
    scores = scores.masked_fill(~seen[None], float("-inf"))
    sink = w[p + "sink"].float()[:, None, None].expand(heads, t, 1)
    full = torch.cat((scores, sink), dim=-1)
    probs = torch.softmax(full, dim=-1)[..., :t]
    out = torch.einsum("hij,jhd->ihd", _r(probs, dtype), v.float()).reshape(t, heads * vd)
    return _lin(_r(out, dtype), w[p + "o"], dtype)


# ---------------------------------------------------------------------------------------------- feed-forward
def dense_ff(h, w, p, dtype):
    a = _r(gelu_tanh(_lin(h, w[p + "gate"], dtype)), dtype) * _lin(h, w[p + "up"], dtype)
    return _lin(_r(a, dtype), w[p + "down"], dtype)


def route(h: torch.Tensor, w: dict, p: str, router: dict, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen [T, top] indices among experts + identity experts, their weights [T, top])."""
    z = _r(h, dtype).double() @ w[p + "router"].double().t()
    s = torch.softmax(z.float(), dim=-1)
    choice = s + w[p + "correction"].float()[None, :]
    total = s.shape[1]
    groups = router.get("groups")
    if groups and int(groups["count"]) > 1:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = choice.view(-1, count, total // count).max(-1).values  # [T, count]
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = allowed[:, :, None].expand(-1, -1, total // count).reshape(-1, total)
        choice = choice.masked_fill(~allowed, float("-inf"))
    chosen = torch.topk(choice, int(router["top"]), dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * float(router["scale"])


def moe_ff(h, w, p, mlp: dict, dtype):
    router = mlp["router"]
    experts = int(router["experts"])
    chosen, weights = route(h, w, p, router, dtype)
    out = torch.zeros(h.shape[0], h.shape[1])
    hr = _r(h, dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t].tolist()):
            if e >= experts:
                y = hr[t]
            else:
                q = f"{p}e{e}."
                a = _r(silu(_lin(hr[t:t + 1], w[q + "gate"], dtype)), dtype) * _lin(hr[t:t + 1], w[q + "up"], dtype)
                y = _lin(_r(a, dtype), w[q + "down"], dtype)[0]
            out[t] += g * y
    return out


# ---------------------------------------------------------------------------------------------- the model
def forward(cfg: dict, w: dict, tokens, dtype=torch.float32, layers_out: list | None = None, fast: bool = True) -> torch.Tensor:
    """Logits [T, vocab] (float32) of one sequence; ``layers_out`` receives the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"].float()[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = i
        while cfg["layers"][src].get("weights_of") is not None:
            src = int(cfg["layers"][src]["weights_of"])
        p = f"l{src}."
        h = _r(rms_norm(x, w[p + "norm1"], eps), dtype)
        if layer["type"] == "mamba2":
            x = x + (mamba2_fast if fast else mamba2)(h, w, p + "mix.", layer["mixer"], eps, dtype)
        elif layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", layer["mixer"], eps, dtype)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = _r(rms_norm(x, w[p + "norm2"], eps), dtype)
            x = x + (dense_ff(h, w, p + "mlp.", dtype) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp, dtype))
        if layers_out is not None:
            layers_out.append(x.clone())
    h = _r(rms_norm(x, w["final.norm"], eps), dtype)
    return _lin(h, w["head"], dtype)
