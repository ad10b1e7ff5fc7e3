"""Dense gated feed-forward."""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Part, WeightDecl, param, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    """down(act(gate(x)) * up(x)), no biases, act = SiLU (miniserve/model/qwen3.py:128-131). The gate and
    up matrices are stacked at load so that one product makes both
    (miniserve/model/fused.py:41-95 does the same). Parameters: ``hidden``, ``intermediate``; optional ``activation``
    (``silu``, the default, or ``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))) and ``names`` (gate / up /
    down -> tensor names)."""
    shape_static = True
    NAMES = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"swiglu knows the activations 'silu' and 'gelu_tanh', not {self.activation!r}")
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}

    def weights(self):
        n = self.names
        return {
            n["gate"]: WeightDecl((self.inter, self.hidden)),
            n["up"]: WeightDecl((self.inter, self.hidden)),
            n["down"]: WeightDecl((self.hidden, self.inter)),
        }

    def _stack(self):
        n = self.names
        return "gate_up_proj.weight", (n["gate"], n["up"])

    def stacks(self):
        return dict([self._stack()])

    def bind(self, tensors):
        self.w_gate_up = self.joined(tensors, *self._stack())
        self.w_down = tensors[self.names["down"]].contiguous()

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
        if dt == torch.bfloat16 and self.activation == "silu":
            # one kernel with the activation in its epilogue where there is one (decode steps, wide prompt steps)
            fused = ops.silu_mul_is_fused(x, self.w_gate_up, act)
            scratch = None if fused else ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev)
            ops.linear_silu_mul(x, self.w_gate_up, act, scratch=scratch, stream=ctx.stream)
        else:
            gate_up = ops.linear(x, self.w_gate_up, stream=ctx.stream, out=ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev))
            if self.activation == "silu":
                ops.silu_mul(act, gate_up, stream=ctx.stream)
            else:
                ops.act_mul(act, gate_up, self.activation, stream=ctx.stream)
        return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))


@register_part("feed_forward", "clamped_glu")
class ClampedGLU(Part):
    """down(g * sigmoid(alpha g) * (u + up_shift)) with g = min(gate(x), limit) and u = clamp(up(x), -limit, limit); every
    projection may have a bias. The gate and up matrices are stacked as in ``swiglu``; their biases are added, and the
    clamps and the activation computed, in float32 by one kernel behind the product. Parameters: ``hidden``,
    ``intermediate``, ``limit`` (absent: no clamps), optional ``alpha`` (1.702), ``up_shift`` (1.0), ``bias`` (True), ``names``
    (gate / up / down and gate_bias / up_bias / down_bias -> tensor names)."""
    shape_static = True
    NAMES = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight", gate_bias="gate_proj.bias",
                 up_bias="up_proj.bias", down_bias="down_proj.bias")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)
        self.limit = float(spec["limit"]) if spec.get("limit") is not None else -1.0  # negative: no clamps
        self.alpha = float(spec.get("alpha", 1.702))
        self.up_shift = float(spec.get("up_shift", 1.0))
        self.bias = bool(spec.params.get("bias", True))
        if spec.get("limit") is not None and self.limit < 0:
            raise ValueError(f"clamped_glu: limit={self.limit} must not be negative")
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}

    def weights(self):
        n = self.names
        w = {n["gate"]: WeightDecl((self.inter, self.hidden)), n["up"]: WeightDecl((self.inter, self.hidden)),
             n["down"]: WeightDecl((self.hidden, self.inter))}
        if self.bias:
            w.update({n["gate_bias"]: WeightDecl((self.inter,), precision="float32"), n["up_bias"]: WeightDecl((self.inter,), precision="float32"),
                      n["down_bias"]: WeightDecl((self.hidden,), precision="float32")})
        return w

    def _stack(self):
        n = self.names
        return "gate_up_proj.weight", (n["gate"], n["up"])

    def stacks(self):
        return dict([self._stack()])

    def bind(self, tensors):
        n = self.names
        self.w_gate_up = self.joined(tensors, *self._stack())
        self.w_down = tensors[n["down"]].contiguous()
        self.w_in_bias = torch.cat([tensors[n["gate_bias"]].float(), tensors[n["up_bias"]].float()]).contiguous() if self.bias else None
        self.w_out_bias = tensors[n["down_bias"]].float().contiguous() if self.bias else None

    @property
    def output_bias(self) -> torch.Tensor | None:
        """The down projection's bias (float32), for a caller that adds it together with something else
        (``forward(..., with_bias=False)``)."""
        return self.w_out_bias

    def forward(self, x, ctx, with_bias: bool = True) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        gate_up = ops.linear(x, self.w_gate_up, stream=ctx.stream, out=ctx.buffer("mlp.gate_up", (t, 2 * self.inter), dt, dev))
        act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
        ops.clamped_glu(act, gate_up, self.w_in_bias, self.limit, self.alpha, self.up_shift, stream=ctx.stream)
        out = ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))
        if with_bias and self.w_out_bias is not None:
            ops.sum_bias(out, out, None, self.w_out_bias, stream=ctx.stream)
        return out


@register_part("feed_forward", "dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))), no gate and no biases. Parameters: ``hidden``, ``intermediate``, ``activation``
    (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); ``relu_squared``: max(z, 0)^2), ``names``
    (up / down -> tensor names). ``features`` stops before the down projection, for a block that joins it with
    another part's output projection."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)
        self.activation = spec.get("activation", "gelu_tanh")
        if self.activation not in ("gelu_tanh", "relu_squared"):
            raise ValueError(f"dense_mlp knows the activations 'gelu_tanh' and 'relu_squared', not {self.activation!r}")
        self.feature_width = self.inter
        names = dict(spec.get("names") or {})
        self.names = {"up": names.get("up", "up_proj.weight"), "down": names.get("down", "down_proj.weight")}

    def weights(self):
        return {self.names["up"]: WeightDecl((self.inter, self.hidden)),
                self.names["down"]: WeightDecl((self.hidden, self.inter))}

    def bind(self, tensors):
        self.w_up = tensors[self.names["up"]].contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def features(self, x, ctx, out: torch.Tensor) -> None:
        """``out`` [T, intermediate] (a view whose rows may be part of wider ones) = act(up(x))."""
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        up = ops.linear(x, self.w_up, stream=ctx.stream, out=ctx.buffer("mlp.up", (t, self.inter), dt, dev))
        if self.activation == "relu_squared":
            ops.relu_squared(out, up, stream=ctx.stream)
        else:
            ops.gelu_tanh(up, up, stream=ctx.stream)
            out.copy_(up)

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        if self.activation == "relu_squared":
            act = ctx.buffer("mlp.act", (t, self.inter), dt, dev)
            self.features(x, ctx, act)
            return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))
        # the activation in the product's epilogue where there is such a kernel (decode steps)
        act = ops.linear_gelu_tanh(x, self.w_up, ctx.buffer("mlp.act", (t, self.inter), dt, dev), stream=ctx.stream)
        return ops.linear(act, self.w_down, stream=ctx.stream, out=ctx.buffer("mlp.down", (t, self.hidden), dt, dev))


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """A mixture of gated feed-forwards of which every token uses ``top``:

        z = W_router x (float32),  s = softmax(z),  choice score c = s + correction
        y = sum over the top c of  weight_scale * s_e * expert_e(x),   expert_e(x) = W_down[e] (act(W_gate[e] x) * (W_up[e] x))

    The router's outputs form ``group_count`` equal groups of neighbours; a group's score is the largest c in it and only
    outputs of the ``group_keep`` best groups can be chosen. The last ``identity`` router outputs are identity experts:
    they have no tensors and their output is x itself (times the weight). Weights use s without the correction and are
    not renormalised unless ``renormalize``. The router (its product, softmax and choice) is float32; its matrix and the
    correction stay float32. The experts' matrices are stacked at load ([E, 2 I, hidden]: an expert's gate rows, then its
    up rows; [E, hidden, I]) and one launch makes every expert's product over the step's (token, choice) pairs sorted by
    expert; the plan of that sort lives on the device, so the part's launches follow from the number of tokens alone.

    Parameters: ``hidden``, ``intermediate``, ``experts``, ``top``; optional ``identity`` (0), ``group_count`` (1),
    ``group_keep`` (1), ``weight_scale`` (1.0), ``renormalize`` (False), ``correction`` (True: a tensor of that name is
    added to the scores for the choice), ``activation`` (``silu`` or ``gelu_tanh``), ``score`` (``softmax``), ``names``
    (router, correction, gate, up, down -> tensor names; ``expert``: the prefix of expert e with ``{}`` for e).

    ``router_bias`` (True: a tensor [outputs] of that name is added to the logits themselves; with ``renormalize`` and no
    correction the weights are then the softmax over the chosen logits alone). ``shared`` (an intermediate size): one
    more gated feed-forward of the experts' form (a ``swiglu`` part under the prefix ``shared``) that every token uses;
    its output is added times sigmoid(w_sg . x), one number per token (tensor ``shared_gate`` [1, hidden], float32,
    computed by the router's kernel from the same input), or unweighted with ``shared_gated`` False."""
    shape_static = True
    NAMES = dict(router="router.weight", correction="router.correction", expert="experts.{}.", gate="gate_proj.weight",
                 up="up_proj.weight", down="down_proj.weight", router_bias="router.bias", shared="shared.", shared_gate="shared.gate")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.inter = param(spec, "intermediate", int)
        self.experts = param(spec, "experts", int)
        self.identity = int(spec.get("identity", 0) or 0)
        self.top = param(spec, "top", int)
        self.group_count = int(spec.get("group_count", 1) or 1)
        self.group_keep = int(spec.get("group_keep", 1) or 1)
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        self.renormalize = bool(spec.get("renormalize", False))
        self.has_correction = bool(spec.params.get("correction", True))
        self.activation = spec.get("activation", "silu")
        if self.activation not in ops.experts.ACTIVATIONS:
            raise ValueError(f"routed_experts knows the activations {sorted(ops.experts.ACTIVATIONS)}, not {self.activation!r}")
        if spec.get("score", "softmax") != "softmax":
            raise NotImplementedError(f"routed_experts scores by softmax, not {spec.get('score')!r}")
        self.outputs = self.experts + self.identity  # what the router chooses among
        if self.experts < 1 or not 1 <= self.top <= self.outputs:
            raise ValueError(f"routed_experts: top={self.top} of {self.experts} experts and {self.identity} identity experts")
        if (self.group_count < 1 or self.outputs % self.group_count or not 1 <= self.group_keep <= self.group_count
                or self.group_keep * (self.outputs // self.group_count) < self.top):
            raise ValueError(f"routed_experts: {self.outputs} router outputs in {self.group_count} groups of which {self.group_keep} are "
                             f"kept cannot give {self.top} choices")
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        self.has_router_bias = bool(spec.get("router_bias", False))
        self.shared_inter = int(spec.get("shared") or 0)
        self.shared_gated = bool(spec.params.get("shared_gated", True)) and self.shared_inter > 0
        self.shared = None
        if self.shared_inter:
            n = self.names
            self.shared = SwiGLU(PartSpec("swiglu", dict(hidden=self.hidden, intermediate=self.shared_inter, activation=self.activation,
                                                         names=dict(gate=n["gate"], up=n["up"], down=n["down"]))), env)
        self.w_router_bias = self.w_shared_gate = None

    def sub_parts(self):
        return {self.names["shared"]: self.shared} if self.shared is not None else {}

    def _expert(self, e: int, which: str) -> str:
        return self.names["expert"].format(e) + self.names[which]

    def weights(self):
        n = self.names
        w = {n["router"]: WeightDecl((self.outputs, self.hidden), precision="float32")}
        if self.has_correction:
            w[n["correction"]] = WeightDecl((self.outputs,), precision="float32")
        if self.has_router_bias:
            w[n["router_bias"]] = WeightDecl((self.outputs,), precision="float32")
        if self.shared_gated:
            w[n["shared_gate"]] = WeightDecl((1, self.hidden), precision="float32")
        for e in range(self.experts):
            w[self._expert(e, "gate")] = WeightDecl((self.inter, self.hidden))
            w[self._expert(e, "up")] = WeightDecl((self.inter, self.hidden))
            w[self._expert(e, "down")] = WeightDecl((self.hidden, self.inter))
        return w

    def stacks(self):
        return {"experts.gate_up": tuple(self._expert(e, k) for e in range(self.experts) for k in ("gate", "up")),
                "experts.down": tuple(self._expert(e, "down") for e in range(self.experts))}

    def bind(self, tensors):
        n, st = self.names, self.stacks()
        self.w_router = tensors[n["router"]].float().contiguous()
        self.w_correction = tensors[n["correction"]].float().contiguous() if self.has_correction else None
        self.w_router_bias = tensors[n["router_bias"]].float().contiguous() if self.has_router_bias else None
        self.w_shared_gate = tensors[n["shared_gate"]].float().reshape(-1).contiguous() if self.shared_gated else None
        self.w_gate_up = self.joined(tensors, "experts.gate_up", st["experts.gate_up"]).view(self.experts, 2 * self.inter, self.hidden)
        self.w_down = self.joined(tensors, "experts.down", st["experts.down"]).view(self.experts, self.hidden, self.inter)

    def route(self, x, ctx):
        """(idx [T, top] int32, wgt [T, top] float32): every token's chosen router outputs and their weights."""
        t, dev = x.shape[0], self.w_down.device
        idx = ctx.buffer("moe.idx", (t, self.top), torch.int32, dev)
        wgt = ctx.buffer("moe.wgt", (t, self.top), torch.float32, dev)
        gate = ctx.buffer("moe.shared_gate", (t,), torch.float32, dev) if self.shared_gated else None
        ops.experts.expert_route(idx, wgt, x, self.w_router, self.w_correction, self.top, self.group_count, self.group_keep,
                                 self.weight_scale, self.renormalize, stream=ctx.stream, logit_bias=self.w_router_bias,
                                 gate_w=self.w_shared_gate, gate_out=gate)
        return idx, wgt

    def forward(self, x, ctx) -> torch.Tensor:
        t, dt, dev = x.shape[0], self.env.dtype, self.w_down.device
        slots, i32 = t * self.top, torch.int32
        idx, wgt = self.route(x, ctx)
        pos = ctx.buffer("moe.pos", (slots,), i32, dev)
        perm = ctx.buffer("moe.perm", (slots,), i32, dev)
        offsets = ctx.buffer("moe.offsets", (self.experts + 1,), i32, dev)
        # bfloat16 with SiLU: both products on the tcgen05 kernel, over the tokens' inputs gathered into sorted order
        tc = ops.experts.tc_experts_ok(dt, self.hidden, self.inter, self.activation) and x.stride(0) % 8 == 0
        tile_rows = ops.experts.TC_TILE_ROWS if tc else ops.experts.TILE_ROWS
        tiles = ctx.buffer("moe.tiles", (ops.experts.expert_max_tiles(slots, self.experts, tile_rows), 2), i32, dev)
        meta = ctx.buffer("moe.meta", (2,), i32, dev)
        ops.experts.expert_plan(pos, perm, offsets, tiles, meta, idx, self.experts, stream=ctx.stream, tile_rows=tile_rows)
        act = ctx.buffer("moe.act", (slots, self.inter), dt, dev)
        y = ctx.buffer("moe.y", (slots, self.hidden), torch.float32, dev)
        if tc:
            xs = ctx.buffer("moe.xs", (slots, self.hidden), dt, dev)
            ops.experts.expert_gather(xs, x, perm, meta, self.top, stream=ctx.stream)
            ops.experts.expert_products_tc(act, xs, self.w_gate_up, tiles, meta, offsets, True, stream=ctx.stream)
            ops.experts.expert_products_tc(y, act, self.w_down, tiles, meta, offsets, False, stream=ctx.stream)
        else:
            ops.experts.expert_gate_up(act, x, self.w_gate_up, perm, self.top, tiles, meta, offsets, self.activation, stream=ctx.stream)
            ops.experts.expert_down(y, act, self.w_down, tiles, meta, offsets, stream=ctx.stream)
        out = ctx.buffer("moe.out", (t, self.hidden), dt, dev)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        gate = ctx.buffer("moe.shared_gate", (t,), torch.float32, dev) if self.shared_gated else None  # written by the router's kernel
        ops.experts.expert_combine(out, y, x, idx, wgt, pos, self.experts, stream=ctx.stream, shared=shared, shared_gate=gate)
        return out
