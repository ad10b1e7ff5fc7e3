"""Linear-attention mixers: a matrix state per head and request instead of keys and values of every
past token. Both run the token-by-token recurrence of ``csrc/recurrence.cu`` (prompt portions and
decoded tokens alike), keep the state in float32 in the request's slot, and start from zero where a
row's first token is at position 0."""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import FixedState, Part, WeightDecl, param, register_part


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def _pad_rows(w: torch.Tensor, rows: int) -> torch.Tensor:
    if w.shape[0] == rows:
        return w.contiguous()
    return torch.cat((w, torch.zeros((rows - w.shape[0], w.shape[1]), dtype=w.dtype, device=w.device)), dim=0).contiguous()


def _pad_cols(w: torch.Tensor, cols: int) -> torch.Tensor:
    if w.shape[1] == cols:
        return w.contiguous()
    return torch.cat((w, torch.zeros((w.shape[0], cols - w.shape[1]), dtype=w.dtype, device=w.device)), dim=1).contiguous()


@register_part("mixer", "decay_linear_attention")
class DecayLinearAttention(Part):
    """Linear attention with a learned decay per key channel and token:

        S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T (q_t * dk^-0.5),
        a_t = sigmoid(W_a2 (W_a1 x_t) + b_a)^(1/tau)      (a low-rank projection; float32 from z on)

    per head, S [dk, dv]; then o is RMS-normed per head over dv (weight shared by the heads), multiplied
    by silu(W_g x) and projected by W_o. One product makes q|k|v|g, a second the low-rank input of the
    decay, a third the decay's logits. Parameters: ``hidden``, ``heads``, ``key_dim``, ``value_dim``,
    ``tau``, ``decay_rank``, ``eps``, ``names`` (q, k, v, g, o, norm, a1, a2, a_bias -> tensor names)."""
    shape_static = True
    NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", g="g_proj.weight", o="o_proj.weight",
                 norm="o_norm.weight", a1="a_proj.0.weight", a2="a_proj.1.weight", a_bias="a_proj.1.bias")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.dk = param(spec, "key_dim", int)
        self.dv = param(spec, "value_dim", int)
        self.tau = param(spec, "tau", float)
        self.rank = param(spec, "decay_rank", int)
        self.eps = param(spec, "eps", float)
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        if self.tau <= 0:
            raise ValueError(f"tau must be positive, got {self.tau}")
        self.feature_width = self.heads * self.dv

    def cache_need(self):
        return FixedState((self.heads, self.dv, self.dk), torch.float32)

    def weights(self):
        n, h, dk, dv, w = self.names, self.heads, self.dk, self.dv, self.hidden
        return {n["q"]: WeightDecl((h * dk, w)), n["k"]: WeightDecl((h * dk, w)), n["v"]: WeightDecl((h * dv, w)),
                n["g"]: WeightDecl((h * dv, w)), n["o"]: WeightDecl((w, h * dv)),
                n["norm"]: WeightDecl((dv,), precision="float32", init="ones_normal"),
                n["a1"]: WeightDecl((self.rank, w)), n["a2"]: WeightDecl((h * dk, self.rank)),
                n["a_bias"]: WeightDecl((h * dk,), precision="float32")}

    def stacks(self):
        n = self.names
        return {"qkvg_proj.weight": (n["q"], n["k"], n["v"], n["g"])}

    def bind(self, tensors):
        n = self.names
        joined = self.joined(tensors, "qkvg_proj.weight", self.stacks()["qkvg_proj.weight"])
        self.w_in = _pad_rows(joined, _pad8(joined.shape[0]))
        self.w_a1 = _pad_rows(tensors[n["a1"]], _pad8(self.rank))  # a rank that is no multiple of 8: zero rows and columns
        self.w_a2 = _pad_cols(tensors[n["a2"]], _pad8(self.rank))
        self.w_a_bias = tensors[n["a_bias"]].contiguous()
        self.w_norm = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.decay_coef = torch.full((self.heads,), 1.0 / self.tau, dtype=torch.float32, device=self.w_o.device)

    def features(self, x: torch.Tensor, ctx, cache, out: torch.Tensor, scale: float = 1.0) -> None:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        h, dk, dv = self.heads, self.dk, self.dv
        proj = ops.linear(x, self.w_in, stream=ctx.stream, out=ctx.buffer("lin.in", (t, self.w_in.shape[0]), dt, dev))
        low = ops.linear(x, self.w_a1, stream=ctx.stream, out=ctx.buffer("lin.low", (t, self.w_a1.shape[0]), dt, dev))
        z = ops.linear(low, self.w_a2, stream=ctx.stream, out=ctx.buffer("lin.z", (t, h * dk), dt, dev))
        o = ctx.buffer("lin.o", (t, h, dv), torch.float32, dev)
        at_k, at_v, at_g = h * dk, 2 * h * dk, 2 * h * dk + h * dv
        # sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
        ops.decay_scan(o, cache.state, proj[:, :at_k], proj[:, at_k:at_v], proj[:, at_v:at_g], z, self.w_a_bias, self.decay_coef,
                       -1.0, None, ctx, h, dk, dv, dk ** -0.5, delta=False)
        ops.head_norm_gate(out, o, self.w_norm, proj[:, at_g:at_g + h * dv], self.eps, scale, "silu", stream=ctx.stream)

    def forward(self, x, ctx, cache):
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        feat = ctx.buffer("lin.feat", (t, self.feature_width), dt, dev)
        self.features(x, ctx, cache, feat)
        return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("lin.proj", (t, self.hidden), dt, dev))


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(Part):
    """The delta rule with a decay per head and key channel:

        S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
        g_t = exp(-exp(A_h) softplus(W_a2 (W_a1 x_t) + b_dt)),   beta_t = sigmoid(W_b x_t)

    per head, S [dk, dv], the read-out after the token's own write. q and k (``kv_heads`` heads of dk,
    head h reading q/k head h // (heads / kv_heads)) and v (heads of dv) each pass a short causal
    convolution over time per channel and SiLU; q and k are then divided by their Euclidean length
    (sqrt(sum x^2 + unit_eps)), q also multiplied by dk^-0.5. o is divided by its root mean square per
    head over dv, times a weight shared by the heads, times sigmoid(W_g2 (W_g1 x)); then W_o. The
    convolution's last taps - 1 inputs are state beside S. One product makes q|k|v|beta, a second both
    low-rank inputs, a third (block-diagonal) the decay's and the gate's logits.
    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``key_dim``, ``value_dim``, ``conv`` (taps),
    ``decay_rank``, ``gate_rank``, ``eps``, ``unit_eps``, ``names``."""
    shape_static = True
    NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", q_conv="q_conv.weight", k_conv="k_conv.weight",
                 v_conv="v_conv.weight", beta="b_proj.weight", a_log="A_log", norm="o_norm.weight", a1="a_proj.0.weight",
                 a2="a_proj.1.weight", dt_bias="dt_bias", g1="g_proj.0.weight", g2="g_proj.1.weight", o="o_proj.weight")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.groups = param(spec, "kv_heads", int)
        self.dk = param(spec, "key_dim", int)
        self.dv = param(spec, "value_dim", int)
        self.taps = param(spec, "conv", int)
        self.a_rank = param(spec, "decay_rank", int)
        self.g_rank = param(spec, "gate_rank", int)
        self.eps = param(spec, "eps", float)
        self.unit_eps = float(spec.get("unit_eps", 1e-6))
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} query/key heads")
        if self.taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {self.taps}")
        self.channels = 2 * self.groups * self.dk + self.heads * self.dv
        self.feature_width = self.heads * self.dv

    def cache_need(self):
        state = FixedState((self.heads, self.dv, self.dk), torch.float32)
        if self.taps == 1:
            return state
        return (state, FixedState((self.taps - 1, self.channels), self.env.dtype))

    def weights(self):
        n, h, g, dk, dv, w = self.names, self.heads, self.groups, self.dk, self.dv, self.hidden
        f32 = dict(precision="float32")
        return {n["q"]: WeightDecl((g * dk, w)), n["k"]: WeightDecl((g * dk, w)), n["v"]: WeightDecl((h * dv, w)),
                n["beta"]: WeightDecl((h, w)),
                n["q_conv"]: WeightDecl((g * dk, self.taps), **f32), n["k_conv"]: WeightDecl((g * dk, self.taps), **f32),
                n["v_conv"]: WeightDecl((h * dv, self.taps), **f32),
                n["a_log"]: WeightDecl((h,), **f32), n["dt_bias"]: WeightDecl((h * dk,), **f32),
                n["norm"]: WeightDecl((dv,), init="ones_normal", **f32),
                n["a1"]: WeightDecl((self.a_rank, w)), n["a2"]: WeightDecl((h * dk, self.a_rank)),
                n["g1"]: WeightDecl((self.g_rank, w)), n["g2"]: WeightDecl((h * dv, self.g_rank)),
                n["o"]: WeightDecl((w, h * dv))}

    def stacks(self):
        n = self.names
        return {"qkvb_proj.weight": (n["q"], n["k"], n["v"], n["beta"]),
                "qkv_conv.weight": (n["q_conv"], n["k_conv"], n["v_conv"])}

    def bind(self, tensors):
        n, st = self.names, self.stacks()
        joined = self.joined(tensors, "qkvb_proj.weight", st["qkvb_proj.weight"])
        self.w_in = _pad_rows(joined, _pad8(joined.shape[0]))
        self.w_conv = self.joined(tensors, "qkv_conv.weight", st["qkv_conv.weight"])
        ra, rg = _pad8(self.a_rank), _pad8(self.g_rank)
        a1, g1 = _pad_rows(tensors[n["a1"]], ra), _pad_rows(tensors[n["g1"]], rg)
        self.w_low = torch.cat((a1, g1), dim=0).contiguous()  # [ra + rg, hidden]
        a2, g2 = _pad_cols(tensors[n["a2"]], ra), _pad_cols(tensors[n["g2"]], rg)
        # [decay logits | gate logits] = [a1 x | g1 x] times a block-diagonal matrix: the zero blocks add exact zeros
        up = torch.zeros((a2.shape[0] + g2.shape[0], ra + rg), dtype=a2.dtype, device=a2.device)
        up[:a2.shape[0], :ra] = a2
        up[a2.shape[0]:, ra:] = g2
        self.w_up = up
        self.w_dt_bias = tensors[n["dt_bias"]].contiguous()
        self.w_norm = tensors[n["norm"]].contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.decay_coef = torch.exp(tensors[n["a_log"]].float()).contiguous()

    def features(self, x: torch.Tensor, ctx, cache, out: torch.Tensor, scale: float = 1.0) -> None:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        h, g, dk, dv, c = self.heads, self.groups, self.dk, self.dv, self.channels
        state, conv = (cache if isinstance(cache, tuple) else (cache, None))
        proj = ops.linear(x, self.w_in, stream=ctx.stream, out=ctx.buffer("delta.in", (t, self.w_in.shape[0]), dt, dev))
        low = ops.linear(x, self.w_low, stream=ctx.stream, out=ctx.buffer("delta.low", (t, self.w_low.shape[0]), dt, dev))
        zg = ops.linear(low, self.w_up, stream=ctx.stream, out=ctx.buffer("delta.zg", (t, self.w_up.shape[0]), dt, dev))
        qkv = ctx.buffer("delta.qkv", (t, c), torch.float32, dev)
        conv_state = conv.state if conv is not None else ctx.buffer("delta.noconv", (1, 0, c), dt, dev)
        ops.conv_silu_unit(qkv, proj[:, :c], conv_state, self.w_conv, ctx, 2 * g, dk, h, dv, self.unit_eps)
        if conv is not None:
            ops.conv_state_update(conv_state, proj[:, :c], ctx, self.taps)
        o = ctx.buffer("delta.o", (t, h, dv), torch.float32, dev)
        ops.decay_scan(o, state.state, qkv[:, :g * dk], qkv[:, g * dk:2 * g * dk], qkv[:, 2 * g * dk:], zg[:, :h * dk],
                       self.w_dt_bias, self.decay_coef, 1.0, proj[:, c:c + h], ctx, h, dk, dv, dk ** -0.5, delta=True)
        ops.head_norm_gate(out, o, self.w_norm, zg[:, h * dk:h * dk + h * dv], self.eps, scale, "sigmoid", stream=ctx.stream)

    def forward(self, x, ctx, cache):
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        feat = ctx.buffer("delta.feat", (t, self.feature_width), dt, dev)
        self.features(x, ctx, cache, feat)
        return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("delta.proj", (t, self.hidden), dt, dev))


def _conv_unit(channels: int) -> int:
    """How many channels one warp of the convolution kernel takes: the largest divisor of ``channels`` up to 128."""
    for u in range(min(channels, 128), 0, -1):
        if channels % u == 0:
            return u
    return 1


@register_part("mixer", "mamba2")
class SelectiveStateSpace(Part):
    """A selective state-space layer in its dual (linear-attention) form: per head a matrix state S [state, head_dim],

        dt_t = softplus(raw_t + dt_bias_h),   a_t = exp(-exp(A_log_h) dt_t)          (float32)
        S_t = a_t S_(t-1) + dt_t B_t x_t^T,   y_t = S_t^T C_t + D_h x_t

    with one decay for the whole head, B and C shared by the heads of a group (head h reads group
    h // (heads / groups)). One product makes [z | x | B | C | raw dt]; x, B and C pass a short causal convolution per
    channel (with a bias) and SiLU; y of all heads times silu(z), then divided by its root mean square in
    ``norm_groups`` equal parts, times a weight, then the output projection. The recurrence is the decay rule of
    ``csrc/recurrence.cu`` with B as keys, C as queries and x (times dt per token and head) as values. The state and
    everything that enters it besides the convolution's output are float32; the convolution's last taps - 1 inputs
    are state beside S.
    Parameters: ``hidden``, ``heads``, ``head_dim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``, ``eps``,
    ``names`` (input, conv, conv_bias, dt_bias, a_log, skip, norm, o -> tensor names)."""
    shape_static = True
    NAMES = dict(input="in_proj.weight", conv="conv1d.weight", conv_bias="conv1d.bias", dt_bias="dt_bias", a_log="A_log",
                 skip="D", norm="norm.weight", o="out_proj.weight")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.dv = param(spec, "head_dim", int)
        self.n = param(spec, "state", int)
        self.groups = param(spec, "groups", int)
        self.taps = param(spec, "conv", int)
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = param(spec, "eps", float)
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.dv
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels do not split into {self.norm_groups} equal parts")
        if self.taps < 1:
            raise ValueError(f"the convolution needs at least one tap, got {self.taps}")
        self.channels = self.inner + 2 * self.groups * self.n  # what passes the convolution: x | B | C
        self.proj_rows = 2 * self.inner + 2 * self.groups * self.n + self.heads
        self.feature_width = self.inner

    def cache_need(self):
        state = FixedState((self.heads, self.dv, self.n), torch.float32)
        if self.taps == 1:
            return state
        return (state, FixedState((self.taps - 1, self.channels), self.env.dtype))

    def weights(self):
        n, f32 = self.names, dict(precision="float32")
        return {n["input"]: WeightDecl((self.proj_rows, self.hidden)),
                n["conv"]: WeightDecl((self.channels, self.taps), **f32), n["conv_bias"]: WeightDecl((self.channels,), **f32),
                n["dt_bias"]: WeightDecl((self.heads,), **f32), n["a_log"]: WeightDecl((self.heads,), **f32),
                n["skip"]: WeightDecl((self.heads,), init="ones_normal", **f32),
                n["norm"]: WeightDecl((self.inner,), init="ones_normal", **f32),
                n["o"]: WeightDecl((self.hidden, self.inner))}

    def bind(self, tensors):
        n = self.names
        self.w_in = _pad_rows(tensors[n["input"]], _pad8(self.proj_rows))
        self.w_conv = tensors[n["conv"]].float().contiguous()
        self.w_conv_bias = tensors[n["conv_bias"]].float().contiguous()
        self.w_dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.decay_coef = torch.exp(tensors[n["a_log"]].float()).contiguous()
        self.w_skip = tensors[n["skip"]].float().contiguous()
        self.w_norm = tensors[n["norm"]].float().contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def features(self, x: torch.Tensor, ctx, cache, out: torch.Tensor, scale: float = 1.0) -> None:
        if scale != 1.0:
            raise NotImplementedError("mamba2 hands its features on unscaled")
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        h, g, n, dv, c, inner = self.heads, self.groups, self.n, self.dv, self.channels, self.inner
        state, conv = (cache if isinstance(cache, tuple) else (cache, None))
        proj = ops.linear(x, self.w_in, stream=ctx.stream, out=ctx.buffer("ssm.in", (t, self.w_in.shape[0]), dt, dev))
        xbc_in = proj[:, inner:inner + c]
        xbc = ctx.buffer("ssm.xbc", (t, c), torch.float32, dev)
        conv_state = conv.state if conv is not None else ctx.buffer("ssm.noconv", (1, 0, c), dt, dev)
        unit = _conv_unit(c)
        ops.conv_silu_unit(xbc, xbc_in, conv_state, self.w_conv, ctx, 0, 1, c // unit, unit, 0.0, bias=self.w_conv_bias)
        if conv is not None:
            ops.conv_state_update(conv_state, xbc_in, ctx, self.taps)
        steps = ctx.buffer("ssm.dt", (2, t, h), torch.float32, dev)  # step sizes, then decays
        ops.ssm_step_decay(steps, proj[:, inner + c:inner + c + h], self.w_dt_bias, self.decay_coef, stream=ctx.stream)
        o = ctx.buffer("ssm.o", (t, h, dv), torch.float32, dev)
        xs, bs, cs = xbc[:, :inner], xbc[:, inner:inner + g * n], xbc[:, inner + g * n:]
        ops.decay_scan(o, state.state, cs, bs, xs, steps[1], None, self.decay_coef, 1.0, None, ctx, h, n, dv, 1.0, delta=False,
                       head_decay=True, v_scale=steps[0])
        ops.gated_group_norm(out, o.view(t, inner), xs, self.w_skip, proj[:, :inner], self.w_norm, self.norm_groups, dv, self.eps,
                             stream=ctx.stream)

    def forward(self, x, ctx, cache):
        t, dt, dev = x.shape[0], self.env.dtype, self.w_o.device
        feat = ctx.buffer("ssm.feat", (t, self.feature_width), dt, dev)
        self.features(x, ctx, cache, feat)
        return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("ssm.proj", (t, self.hidden), dt, dev))
