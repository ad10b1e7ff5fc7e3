"""Arrangements of mixer, feed-forward and norms into one layer."""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import LayerSpec, PartSpec
from .base import BuildEnv, FixedState, Part, ResidualStream, WeightDecl, build_part, register_part


def _norm(norm, stream: ResidualStream, ctx):
    """A block's first norm over the stream as the block before left it (its addend and the addend's factor)."""
    if stream.pending_scale != 1.0:
        return norm.forward(stream.total, stream.pending, ctx, delta_scale=stream.pending_scale)
    return norm.forward(stream.total, stream.pending, ctx)


@register_part("block", "prenorm")
class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += feed_forward(norm2(h)) (miniserve/model/qwen3.py:212-216).
    The adds are fused into the norm that follows them, so the block hands its last addend
    on as ``pending``. Parameters: ``names`` maps mixer / feed_forward / norm1 / norm2 to their
    tensor-name prefixes inside the layer. A layer without a feed-forward (``LayerSpec.feed_forward`` None)
    has neither it nor norm2, and hands the mixer's output on as the pending addend."""
    shape_static = True

    def __init__(self, spec, env: BuildEnv, layer: LayerSpec | None = None):
        super().__init__(spec, env)
        if layer is None:
            raise ValueError("a block is built from its LayerSpec (use build_block)")
        names = dict(spec.get("names") or {})
        self.has_ff = layer.feed_forward is not None
        self.names = {k: names[k] for k in ("mixer", "norm1") + (("feed_forward", "norm2") if self.has_ff else ())}
        self.mixer = build_part("mixer", layer.mixer, env)
        self.norm1 = build_part("norm", layer.norms["norm1"], env)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, env) if self.has_ff else None
        self.norm2 = build_part("norm", layer.norms["norm2"], env) if self.has_ff else None

    def sub_parts(self):
        out = {self.names["mixer"]: self.mixer, self.names["norm1"]: self.norm1}
        if self.has_ff:
            out.update({self.names["feed_forward"]: self.feed_forward, self.names["norm2"]: self.norm2})
        return out

    def forward(self, stream: ResidualStream, ctx, cache) -> ResidualStream:
        total = stream.total
        x = _norm(self.norm1, stream, ctx)
        a = self.mixer.forward(x, ctx, cache)
        if not self.has_ff:
            return ResidualStream(total, a)
        x = self.norm2.forward(total, a, ctx)
        return ResidualStream(total, self.feed_forward.forward(x, ctx))

@register_part("block", "parallel_residual")
class ParallelResidualBlock(Part):
    """h = norm1(x); x += residual_mult * (mixer(h) + feed_forward(h)): one norm, both sublayers read its output.
    When both can stop before their output projections (``features``, ``feature_width`` and ``w_o`` / ``w_down``),
    they write their features side by side into one row and ONE product with the two output matrices joined along
    their inputs makes the sum; otherwise the two outputs are added. The sum is handed on as the pending addend
    with ``residual_mult`` as its factor, so the multiplication and the add happen in float32 inside the next norm.
    The input side is joined likewise when the mixer says which tensor its input product uses (``input_weight``,
    ``input_rows``) and gates per channel, and the feed-forward's activation is squared ReLU: ONE product with the
    mixer's input matrices and the up projection stacked makes q, k, v, gate and up (or q, latent, gate and up),
    and one kernel applies the gate and the activation into the joint row. The parts' own copies of the joined
    matrices are dropped.
    Parameters: ``names`` (mixer / feed_forward / norm1 -> tensor-name prefixes), ``residual_mult``. A layer
    without a feed-forward adds the mixer's output alone."""
    shape_static = True

    def __init__(self, spec, env: BuildEnv, layer: LayerSpec | None = None):
        super().__init__(spec, env)
        if layer is None:
            raise ValueError("a block is built from its LayerSpec (use build_block)")
        names = dict(spec.get("names") or {})
        self.mult = float(spec.get("residual_mult", 1.0))
        self.has_ff = layer.feed_forward is not None
        self.names = {k: names[k] for k in ("mixer", "norm1") + (("feed_forward",) if self.has_ff else ())}
        self.mixer = build_part("mixer", layer.mixer, env)
        self.norm1 = build_part("norm", layer.norms["norm1"], env)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, env) if self.has_ff else None
        self.joint = self.has_ff and all(hasattr(p, "features") and hasattr(p, "feature_width") for p in (self.mixer, self.feed_forward))
        if self.joint and getattr(self.mixer, "general", True) is False:
            self.joint = False  # an attention on its own fused path has no such stop
        self.w_out = None
        self.w_in = None
        self.joint_in = False

    def sub_parts(self):
        out = {self.names["mixer"]: self.mixer, self.names["norm1"]: self.norm1}
        if self.has_ff:
            out[self.names["feed_forward"]] = self.feed_forward
        return out

    def bind_all(self, tensors, prefix: str = "") -> None:
        super().bind_all(tensors, prefix)
        if self.joint:
            w = torch.cat([self.mixer.w_o, self.feed_forward.w_down], dim=1)  # [hidden, mixer features + feed-forward features]
            if w.shape[1] % 8:  # the product wants rows of whole 16 bytes: zero columns, which meet zero features
                w = torch.cat((w, torch.zeros((w.shape[0], -w.shape[1] % 8), dtype=w.dtype, device=w.device)), dim=1)
            self.w_out = w.contiguous()
            mixer, ff = self.mixer, self.feed_forward
            name = getattr(mixer, "input_weight", None)
            self.joint_in = bool(name and getattr(mixer, "out_gate", "channel_sigmoid") == "channel_sigmoid"
                                 and getattr(ff, "activation", None) == "relu_squared")
            if self.joint_in:
                own = getattr(mixer, name)[:mixer.input_rows]
                w = torch.cat([own, ff.w_up], dim=0)  # [mixer's input rows + intermediate, hidden]
                if w.shape[0] % 8:  # rows of the product's output start on 16 bytes: a few zero rows at the end
                    w = torch.cat((w, torch.zeros((-w.shape[0] % 8, w.shape[1]), dtype=w.dtype, device=w.device)), dim=0)
                self.w_in = w.contiguous()
                setattr(mixer, name, None)  # the joined matrices live in this block now
                ff.w_up = None
            mixer.w_o = None
            ff.w_down = None

    def forward(self, stream: ResidualStream, ctx, cache) -> ResidualStream:
        total = stream.total
        x = _norm(self.norm1, stream, ctx)
        if not self.has_ff:
            return ResidualStream(total, self.mixer.forward(x, ctx, cache), self.mult)
        t, dt, dev = x.shape[0], self.env.dtype, x.device
        if self.joint:
            fa, fb = self.mixer.feature_width, self.feed_forward.feature_width
            feat = ctx.buffer("block.feat", (t, self.w_out.shape[1]), dt, dev)
            if self.joint_in:
                rows = self.mixer.input_rows
                proj = ops.linear(x, self.w_in, stream=ctx.stream, out=ctx.buffer("block.in", (t, self.w_in.shape[0]), dt, dev))
                vals, gate = self.mixer.features(x, ctx, cache, None, proj=proj[:, :rows], defer_gate=True)
                ops.gate_relu_squared(feat[:, :fa + fb], vals, gate, self.mixer.value_dim, proj[:, rows:rows + fb], stream=ctx.stream)
            else:
                self.mixer.features(x, ctx, cache, feat[:, :fa])
                self.feed_forward.features(x, ctx, feat[:, fa:fa + fb])
            if fa + fb < feat.shape[1]:
                feat[:, fa + fb:].zero_()
            y = ops.linear(feat, self.w_out, stream=ctx.stream, out=ctx.buffer("block.out", (t, self.w_out.shape[0]), dt, dev))
            return ResidualStream(total, y, self.mult)
        a = self.mixer.forward(x, ctx, cache)
        b = self.feed_forward.forward(x, ctx)
        y = ctx.buffer("block.out", tuple(a.shape), dt, dev)
        ops.axpby(y, a, b, 1.0, 1.0, stream=ctx.stream)
        return ResidualStream(total, y, self.mult)


class TokenShift(Part):
    """h_t <- h_t + (h_(t-1) - h_t) * mix, element by element, with h_(t-1) the previous token's h before the
    replacement and zeros before a sequence's first token. The last h of a portion is a request's state (one vector per
    run entry, in the run's dtype), so that the next portion or the next decoded token continues from it. ``mix`` is a
    float32 tensor [size]. Parameters: ``size``, ``name`` (the tensor's name)."""
    shape_static = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.name = spec.get("name", "shift")

    def weights(self):
        return {self.name: WeightDecl((self.size,), precision="float32")}

    def bind(self, tensors):
        self.w_mix = tensors[self.name].float().contiguous()

    def cache_need(self) -> FixedState:
        return FixedState((self.size,), self.env.dtype)

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        out = ctx.buffer("shift.out", tuple(h.shape), h.dtype, h.device)
        ops.token_shift(out, h, cache.state, self.w_mix, ctx)  # (and the portion's last h into the slot, by the CTA that read it)
        return out


@register_part("block", "parallel_dual_norm")
class ParallelDualNormBlock(Part):
    """x += mixer(shift(norm1(x))) + feed_forward(norm2(x)): both sublayers read the same x, each through a norm of its
    own; the sum is handed on as the pending addend, so the add happens in float32 inside the next norm. When both
    norms are layer norms they come out of one launch. ``token_shift`` (a name, or absent): what the mixer reads is
    first mixed with the previous token's (``TokenShift``); the block then needs a state vector per request beside the
    mixer's cache, and its cache view is the pair (shift state, mixer's view). A layer without a feed-forward has
    neither it nor norm2. Parameters: ``names`` (mixer / feed_forward / norm1 / norm2 -> tensor-name prefixes),
    ``token_shift``, ``hidden``."""
    shape_static = True

    def __init__(self, spec, env: BuildEnv, layer: LayerSpec | None = None):
        super().__init__(spec, env)
        if layer is None:
            raise ValueError("a block is built from its LayerSpec (use build_block)")
        names = dict(spec.get("names") or {})
        self.has_ff = layer.feed_forward is not None
        self.names = {k: names[k] for k in ("mixer", "norm1") + (("feed_forward", "norm2") if self.has_ff else ())}
        self.mixer = build_part("mixer", layer.mixer, env)
        self.norm1 = build_part("norm", layer.norms["norm1"], env)
        self.feed_forward = build_part("feed_forward", layer.feed_forward, env) if self.has_ff else None
        self.norm2 = build_part("norm", layer.norms["norm2"], env) if self.has_ff else None
        shift = spec.get("token_shift")
        self.shift = TokenShift(PartSpec("token_shift", dict(size=int(spec["hidden"]), name=shift)), env) if shift else None
        self.paired = self.has_ff and hasattr(self.norm1, "forward_pair") and type(self.norm1) is type(self.norm2)

    def sub_parts(self):
        out = {self.names["mixer"]: self.mixer, self.names["norm1"]: self.norm1}
        if self.has_ff:
            out.update({self.names["feed_forward"]: self.feed_forward, self.names["norm2"]: self.norm2})
        if self.shift is not None:
            out[""] = self.shift
        return out

    def cache_need(self):
        """The mixer's need, or with a token shift the pair (the shift's state, the mixer's need: None where the mixer
        reads another entry's cache)."""
        need = self.mixer.cache_need()
        return need if self.shift is None else (self.shift.cache_need(), need)

    def forward(self, stream: ResidualStream, ctx, cache) -> ResidualStream:
        total = stream.total
        if self.paired:
            h1, h2 = self.norm1.forward_pair(self.norm2, total, stream.pending, ctx, delta_scale=stream.pending_scale)
        else:
            h1 = _norm(self.norm1, stream, ctx)
            h2 = self.norm2.forward(total, None, ctx, role="norm.out2") if self.has_ff else None
        if self.shift is not None:
            shift_cache, cache = cache
            h1 = self.shift.forward(h1, ctx, shift_cache)
        a = self.mixer.forward(h1, ctx, cache)
        if not self.has_ff:
            return ResidualStream(total, a)
        # a bias on the feed-forward's output is added in the same kernel as the two sublayers' outputs
        bias = getattr(self.feed_forward, "output_bias", None)
        b = self.feed_forward.forward(h2, ctx, with_bias=False) if bias is not None else self.feed_forward.forward(h2, ctx)
        y = ctx.buffer("block.out", tuple(a.shape), self.env.dtype, a.device)
        ops.sum_bias(y, a, b, bias, stream=ctx.stream)
        return ResidualStream(total, y)


def build_block(layer: LayerSpec, env: BuildEnv) -> Part:
    from .base import _REGISTRY

    try:
        cls = _REGISTRY["block"][layer.block.kind]
    except KeyError:
        raise ValueError(f"no block arrangement named {layer.block.kind!r}; registered: {sorted(_REGISTRY['block'])}") from None
    return cls(layer.block, env, layer)
