"""Attention whose keys and values are made from one small vector per token, the only thing cached."""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import PagedKV, Part, WeightDecl, build_part, param, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """q = W_q x; c = rmsnorm(W_down x) * w_norm, a vector of ``latent`` numbers per token; head h has keys
    k_h = W_uk[h] c and values v_h = W_uv[h] c; causal softmax attention with scores (q_h . k_h) * scale, no
    position encoding; the concatenated heads times sigmoid(W_g x) element by element; output projection.

    Only c is cached, in pages of one "head" of size ``latent`` (rounded up to 16, zeros beyond) that serve as
    keys and as values (``PagedKV(values=False)``). The per-head matrices are folded onto the query side:
    q'_h = W_uk[h]^T q_h gives q_h . k_h = q'_h . c, so the framework's attention kernels run with every query
    head reading the one cached vector (keys and values alike), and the value of head h is W_uv[h] applied to
    attention's output over c. Two small products per head and step instead of keys and values of every head for
    every cached token. The norm of c is float32; its weight stays float32.

    Parameters: ``hidden``, ``heads``, ``head_dim``, ``value_dim``, ``latent``, ``scale``, ``eps``, ``names`` (q, down,
    norm, up_k, up_v, gate, o -> tensor names). ``features`` stops before the output projection.

    Optional parameters, each with its own constants, for designs that differ:
    ``q_latent`` (queries go through a latent of their own: c_q = rmsnorm(W_qdown x) * w_qnorm, q = W_q c_q; names
    q_down, q_norm); ``rotated_dim`` with ``position`` (a PartSpec of category ``position``: every query head has
    ``rotated_dim`` more channels behind its ``head_dim``, W_down has as many more rows, which are not normed and are
    one key part shared by all heads; both are rotated by position and their product adds to the score; the cache
    entry is [c | rotated key part], the query side [W_uk[h]^T q_h | rotated q_h]); ``window`` (a query sees itself
    and the window - 1 tokens before it; the cache gives older pages back); ``sink`` = ``"learned"`` (the softmax's
    denominator has one more term exp(sink_h), float32 per head, name ``sink``); ``out_gate`` = None (no gate and no
    gate tensor; default ``channel_sigmoid``)."""
    shape_static = True
    general = True
    input_weight = "w_in"  # the attribute that holds the input product's (stacked) matrix; its first ``input_rows`` rows are real
    NAMES = dict(q="q_proj.weight", down="kv_down_proj.weight", norm="kv_norm.weight", up_k="k_up_proj.weight",
                 up_v="v_up_proj.weight", gate="g_proj.weight", o="o_proj.weight", q_down="q_down_proj.weight",
                 q_norm="q_norm.weight", sink="sink")
    MAX_LATENT = 512  # the largest head size an attention kernel takes (the tensor-core kernels: 256; beyond, the row-wise kernel)

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.head_dim = param(spec, "head_dim", int)
        self.value_dim = param(spec, "value_dim", int)
        self.latent = param(spec, "latent", int)
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.eps = param(spec, "eps", float)
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        self.q_latent = int(spec.get("q_latent") or 0)
        self.rot = int(spec.get("rotated_dim") or 0)
        self.position = build_part("position", spec.get("position") or PartSpec("none"), env)
        if self.rot and (self.rot % 2 or self.position.kernel_table()[1] != self.rot):
            raise ValueError(f"latent_attention: the rotated part ({self.rot}) must be even and be what the position encoding rotates")
        self.window = int(spec.get("window") or 0) or None
        self.learned_sink = spec.get("sink") == "learned"
        if spec.get("sink") not in (None, False, "learned"):
            raise ValueError(f"latent_attention: sink must be 'learned' or absent, got {spec.get('sink')!r}")
        self.out_gate = spec.params.get("out_gate", "channel_sigmoid")
        if self.out_gate not in (None, "channel_sigmoid"):
            raise ValueError(f"latent_attention: out_gate must be 'channel_sigmoid' or None, got {self.out_gate!r}")
        self.extras = None
        self.cache_dim = -(-(self.latent + self.rot) // 16) * 16
        if self.cache_dim > self.MAX_LATENT:
            raise NotImplementedError(f"latent_attention: a latent of {self.latent} numbers is beyond the attention kernels' "
                                      f"largest head size ({self.MAX_LATENT})")
        self.feature_width = self.heads * self.value_dim

    def cache_need(self):
        return PagedKV(1, self.cache_dim, self.window, values=False)

    def weights(self):
        n, h = self.names, self.heads
        w = {n["q"]: WeightDecl((h * (self.head_dim + self.rot), self.q_latent or self.hidden)),
             n["down"]: WeightDecl((self.latent + self.rot, self.hidden)),
             n["norm"]: WeightDecl((self.latent,), precision="float32", init="ones_normal"),
             n["up_k"]: WeightDecl((h * self.head_dim, self.latent)),
             n["up_v"]: WeightDecl((h * self.value_dim, self.latent)),
             n["o"]: WeightDecl((self.hidden, h * self.value_dim))}
        if self.out_gate:
            w[n["gate"]] = WeightDecl((h * self.value_dim, self.hidden))
        if self.q_latent:
            w[n["q_down"]] = WeightDecl((self.q_latent, self.hidden))
            w[n["q_norm"]] = WeightDecl((self.q_latent,), precision="float32", init="ones_normal")
        if self.learned_sink:
            w[n["sink"]] = WeightDecl((h,), precision="float32")
        return w

    def _stack(self):
        """The input product's rows: the queries (or their latent), the keys' and values' latent with the rotated key
        part behind it, the gate."""
        n = self.names
        return "in_proj.weight", (n["q_down"] if self.q_latent else n["q"], n["down"]) + ((n["gate"],) if self.out_gate else ())

    def stacks(self):
        return dict([self._stack()])  # one product makes q, the latent before its norm, and the gate

    def bind(self, tensors):
        n, h, r, rc = self.names, self.heads, self.latent, self.cache_dim
        w_in = self.joined(tensors, *self._stack())
        self.input_rows = w_in.shape[0]  # rows of the input product that are this mixer's (before any padding)
        if w_in.shape[0] % 8:  # rows of the product's output start on 16 bytes: a few zero rows at the end
            w_in = torch.cat((w_in, torch.zeros((-w_in.shape[0] % 8, self.hidden), dtype=w_in.dtype, device=w_in.device)), dim=0)
        self.w_in = w_in.contiguous()
        self.w_norm = tensors[n["norm"]].float().contiguous()
        if self.q_latent:
            self.w_q_norm = tensors[n["q_norm"]].float().contiguous()
            self.w_q = tensors[n["q"]].contiguous()
        if self.learned_sink:
            self.w_sink = tensors[n["sink"]].float().contiguous()
            self.extras = ops.AttentionExtras(self.w_sink, 0.0, 0)
        uk = tensors[n["up_k"]].view(h, self.head_dim, r)
        uv = tensors[n["up_v"]].view(h, self.value_dim, r)
        # [heads, latent (padded), head_dim]: q' = W_uk[h]^T q; padded rows are zero, so q' is zero where the cache is
        self.w_uk_t = torch.zeros((h, rc, self.head_dim), dtype=uk.dtype, device=uk.device)
        self.w_uk_t[:, :r] = uk.transpose(1, 2)
        # [heads, value_dim, latent (padded)]
        self.w_uv = torch.zeros((h, self.value_dim, rc), dtype=uv.dtype, device=uv.device)
        self.w_uv[:, :, :r] = uv
        self.w_o = tensors[n["o"]].contiguous()

    def features(self, x: torch.Tensor, ctx, cache, out: torch.Tensor | None, scale: float = 1.0, proj: torch.Tensor | None = None,
                 defer_gate: bool = False):
        """``out`` [T, heads * value_dim] (a view whose rows may be part of wider ones) = scale * gate * attention.
        ``proj``: the q|latent|gate projection if the caller made it already (columns of a wider product).
        ``defer_gate``: nothing is written; the heads' values [T, heads, value_dim] and the gate's columns are
        returned for a caller that applies the gate together with something else."""
        t = x.shape[0]
        dt, dev = self.env.dtype, x.device
        h, dk, dv, r, rc = self.heads, self.head_dim, self.value_dim, self.latent, self.cache_dim
        if proj is None:
            proj = ops.linear(x, self.w_in, stream=ctx.stream, out=ctx.buffer("lat.in", (t, self.w_in.shape[0]), dt, dev))
        rot = self.rot
        at_c = self.q_latent or h * (dk + rot)
        at_g = at_c + r + rot
        if self.q_latent:
            cq = ctx.buffer("lat.cq", (t, self.q_latent), dt, dev)
            ops.row_rmsnorm(cq, proj[:, :at_c], self.w_q_norm, self.eps, stream=ctx.stream)
            qh = ops.linear(cq, self.w_q, stream=ctx.stream, out=ctx.buffer("lat.qh", (t, h * (dk + rot)), dt, dev)).view(t, h, dk + rot)
        else:
            qh = proj[:, :at_c].unflatten(1, (h, dk + rot))
        q = ctx.buffer("lat.q", (t, h, rc), dt, dev)
        ops.linear_heads(qh[:, :, :dk], self.w_uk_t, q, stream=ctx.stream)
        if rot:
            # after the per-head product (which wrote zeros there): the rotated parts behind the latent-sized part
            if not qh.is_contiguous():
                qh = ctx.buffer("lat.qh", (t, h, dk + rot), dt, dev).copy_(qh)
            ops.latent_rope_prepare(cache.k, proj[:, at_c:at_g], self.w_norm, self.eps, qh, dk, q, self.position.step_table(ctx),
                                    ctx.positions, ctx.row_of_token, ctx.page_indptr[cache.group], ctx.page_indices[cache.group],
                                    cache.page_size, ctx.status, stream=ctx.stream)
        else:
            ops.latent_prepare(cache.k, proj[:, at_c:at_g], self.w_norm, self.eps, ctx.positions, ctx.row_of_token,
                               ctx.page_indptr[cache.group], ctx.page_indices[cache.group], cache.page_size, ctx.status, stream=ctx.stream)
        att = ctx.buffer("lat.att", (t, h, rc), dt, dev)
        ops.attention(att, q, cache.k, cache.v, ctx, cache.group, self.scale, self.window, False, extras=self.extras)
        if not self.out_gate:
            if scale != 1.0:
                raise NotImplementedError("latent_attention without a gate hands its features on unscaled")
            if out.is_contiguous():  # the heads' values are the features themselves
                ops.linear_heads(att, self.w_uv, out.view(t, h, dv), stream=ctx.stream)
            else:
                val = ctx.buffer("lat.val", (t, h, dv), dt, dev)
                ops.linear_heads(att, self.w_uv, val, stream=ctx.stream)
                out.copy_(val.view(t, h * dv))
            return
        val = ctx.buffer("lat.val", (t, h, dv), dt, dev)
        ops.linear_heads(att, self.w_uv, val, stream=ctx.stream)
        if defer_gate:
            return val, proj[:, at_g:at_g + h * dv]
        ops.channel_gate(out, val, proj[:, at_g:at_g + h * dv], dv, scale, stream=ctx.stream)

    def forward(self, x: torch.Tensor, ctx, cache):
        t = x.shape[0]
        dt, dev = self.env.dtype, x.device
        feat = ctx.buffer("lat.feat", (t, self.feature_width), dt, dev)
        self.features(x, ctx, cache, feat)
        return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("lat.proj", (t, self.w_o.shape[0]), dt, dev))
