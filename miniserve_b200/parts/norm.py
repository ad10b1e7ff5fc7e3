"""Norms with the residual add (and an optional row gather) fused in: RMSNorm, Dynamic Tanh, layer norm."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightDecl, param, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in float32, no bias and no ``1 +``
    offset (miniserve/model/qwen3.py:78-82). Parameters: ``size``, ``eps``; optional ``unit_offset`` (the
    stored weight is the scale's distance from one: y = x * rsqrt(mean(x^2) + eps) * (1 + weight); the weight
    then stays float32 whatever the run's dtype, so that 1 + weight is not rounded) and ``name`` (the
    tensor's name relative to the part's prefix, default ``weight``)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = param(spec, "size", int)
        self.eps = param(spec, "eps", float)
        self.unit_offset = bool(spec.get("unit_offset", False))
        self.name = spec.get("name", "weight")
        self._w_f32 = None

    def weights(self):
        if self.unit_offset:
            return {self.name: WeightDecl((self.size,), precision="float32")}
        return {self.name: WeightDecl((self.size,), init="ones_normal")}

    def bind(self, tensors):
        self.w_weight = tensors[self.name].contiguous()
        self._w_f32 = self.w_weight if self.w_weight.dtype == torch.float32 else None

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None,
                num_rows: int | None = None, write_residual: bool = True, delta_scale: float = 1.0, role: str = "norm.out") -> torch.Tensor:
        """Normalise ``residual (+ delta_scale * delta)``; without ``rows`` the sum is stored back into
        ``residual``. With ``rows`` (int32 indices) only those rows are produced. ``role``: the name of the output's
        buffer, for a caller that keeps two norms' outputs alive at once."""
        n = residual.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.buffer(role, (n, self.size), self.env.dtype, residual.device)
        if self.unit_offset or delta_scale != 1.0:
            if self._w_f32 is None:
                self._w_f32 = self.w_weight.float()
            ops.add_rmsnorm_scaled(out, residual, delta, delta_scale, self._w_f32, 1.0 if self.unit_offset else 0.0, self.eps,
                                   rows=rows, num_rows=n, write_residual=write_residual, stream=ctx.stream)
            return out
        ops.add_rmsnorm(out, residual, delta, self.w_weight, self.eps, rows=rows, num_rows=n,
                        write_residual=write_residual, stream=ctx.stream)
        return out


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Part):
    """y = tanh(alpha x) * weight + bias in the place of a norm: no mean, no variance, so no reduction
    over the row; alpha is one learned scalar. Computed in float32 from float32 parameters, with the
    residual add fused in as for RMSNorm. Parameters: ``size``; ``names`` maps weight / bias / alpha to
    tensor names relative to the part's prefix (default ``weight``, ``bias``, ``alpha``)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = param(spec, "size", int)
        names = dict(spec.get("names") or {})
        self.names = {k: names.get(k, k) for k in ("weight", "bias", "alpha")}

    def weights(self):
        n = self.names
        return {n["weight"]: WeightDecl((self.size,), precision="float32", init="ones_normal"),
                n["bias"]: WeightDecl((self.size,), precision="float32"),
                n["alpha"]: WeightDecl((), precision="float32", init="ones_normal")}

    def bind(self, tensors):
        n = self.names
        self.w_weight = tensors[n["weight"]].contiguous()
        self.w_bias = tensors[n["bias"]].contiguous()
        self.w_alpha = tensors[n["alpha"]].reshape(1).contiguous()

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None,
                num_rows: int | None = None, write_residual: bool = True, delta_scale: float = 1.0, role: str = "norm.out") -> torch.Tensor:
        if delta_scale != 1.0:
            raise NotImplementedError("dynamic_tanh takes its addend unscaled")
        n = residual.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.buffer(role, (n, self.size), self.env.dtype, residual.device)
        ops.add_dyt(out, residual, delta, self.w_weight, self.w_bias, self.w_alpha, rows=rows, num_rows=n,
                    write_residual=write_residual, stream=ctx.stream)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * weight + bias, var the mean of the squared deviations; statistics and
    parameters in float32, the residual add fused in as for RMSNorm. Parameters: ``size``, ``eps``; ``names`` maps
    weight / bias to tensor names relative to the part's prefix (default ``weight``, ``bias``). ``forward_pair``
    applies this norm and another of the same size to the same rows in one launch (the statistics are shared)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = param(spec, "size", int)
        self.eps = param(spec, "eps", float)
        names = dict(spec.get("names") or {})
        self.names = {k: names.get(k, k) for k in ("weight", "bias")}

    def weights(self):
        n = self.names
        return {n["weight"]: WeightDecl((self.size,), precision="float32", init="ones_normal"),
                n["bias"]: WeightDecl((self.size,), precision="float32")}

    def bind(self, tensors):
        self.w_weight = tensors[self.names["weight"]].float().contiguous()
        self.w_bias = tensors[self.names["bias"]].float().contiguous()

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None,
                num_rows: int | None = None, write_residual: bool = True, delta_scale: float = 1.0, role: str = "norm.out") -> torch.Tensor:
        n = residual.shape[0] if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = ctx.buffer(role, (n, self.size), self.env.dtype, residual.device)
        ops.add_layernorm(out, residual, delta, self.w_weight, self.w_bias, self.eps, rows=rows, num_rows=n,
                          write_residual=write_residual, delta_scale=delta_scale, stream=ctx.stream)
        return out

    def forward_pair(self, other: "LayerNorm", residual: torch.Tensor, delta: torch.Tensor | None, ctx, delta_scale: float = 1.0,
                     roles: tuple[str, str] = ("norm.out", "norm.out2")) -> tuple[torch.Tensor, torch.Tensor]:
        """(this norm, ``other``) of residual + delta_scale * delta; the sum is written back to ``residual``."""
        if other.size != self.size or other.eps != self.eps:
            raise ValueError("two norms of one row share its statistics: they need the same size and eps")
        n = residual.shape[0]
        a = ctx.buffer(roles[0], (n, self.size), self.env.dtype, residual.device)
        b = ctx.buffer(roles[1], (n, self.size), self.env.dtype, residual.device)
        ops.add_layernorm(a, residual, delta, self.w_weight, self.w_bias, self.eps, delta_scale=delta_scale, out2=b,
                          weight2=other.w_weight, bias2=other.w_bias, stream=ctx.stream)
        return a, b
