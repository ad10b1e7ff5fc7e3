"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import PagedKV, Part, WeightDecl, build_part, param, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """q/k/v projections (no bias), optional per-head RMSNorm of q and k over head_dim, position
    encoding, causal attention with query head h reading kv head h // (heads / kv_heads), output
    projection (miniserve/model/qwen3.py:110-126; scale d^-0.5 at :133-135).

    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``qk_norm`` (bool),
    ``qk_norm_eps``, ``position`` (a PartSpec of category ``position``), optional ``window``
    (a query sees only the last ``window`` keys), optional ``scale``, and ``kv_source``:
    ``own`` (default) or ``shared`` (the layer has no k/v projections and attends over the
    cache of the run entry named by ``RunEntry.cache_of``).

    Further optional parameters, for designs that are not Qwen3's: ``sink`` (the softmax's denominator
    has one more term of score 0, which carries no value: weights exp(s_j) / (1 + sum exp(s))),
    ``value_dim`` (a value size other than the key size ``head_dim``), ``out_gate`` = ``head_sigmoid``
    (head h's output is multiplied by sigmoid(W_g x)_h, one number per token and head, before the output
    projection), a position encoding that pairs adjacent channels (``rope_pairs``), and ``names`` (the
    tensors' names: q, k, v, o, q_norm, k_norm, gate). A gate, another value size or adjacent pairing
    take the general kernels: one product makes q|k|v|gate, ``ops.qkv_prepare`` norms and rotates in
    float32 and writes keys and values padded with zeros to one cache head size (a zero channel changes
    no score and no output), and ``ops.head_gate`` cuts, gates and scales attention's output.
    ``features`` stops before the output projection, for a mixer that joins several branches in one.

    More optional parameters: ``sink`` = ``"learned"`` (the sink's score is a tensor [heads], kept in float32, one
    number per head, neither scaled nor capped), ``softcap`` (scores become softcap * tanh(score / softcap) after
    the scale), ``chunk`` (a query at position p sees only keys from floor(p / chunk) * chunk on, blocks counted
    from position 0 of the sequence; the cache then gives back pages that lie a whole block behind), and
    ``out_gate`` = ``channel_sigmoid`` (attention's output is multiplied element by element by sigmoid(W_g x),
    W_g as wide as the concatenated heads). All of them take the general path.

    And: ``qk_norm`` = ``"unit"`` (q and k are divided by their root mean square over the head, no weight), ``qkv_bias``
    (q, k and v have biases, tensors ``q_bias`` / ``k_bias`` / ``v_bias`` of ``names``, added in float32 before the norm),
    ``head_temperature`` (a learned number per head, tensor ``temp``, multiplies the scaled scores: applied to the
    prepared queries), ``distance_bias`` (tensors ``r1`` and ``r2`` [heads]: r1_h ln(1 + r2_h (i - j)) is taken off the
    scaled score of query i and key j), ``keep_first`` (the first keys of a sequence stay visible behind the window;
    the cache then keeps every page) and ``cache_window`` (how far back the cache keeps keys when that is not the
    mixer's own reach: 0 for everything, for a mixer whose cache another mixer with a longer reach reads). With
    ``kv_source`` = ``shared`` these run on the general path too: the projection holds q (and the gate) alone."""
    shape_static = True
    input_weight = "w_qkv"  # the attribute that holds the input product's (stacked) matrix; its first ``input_rows`` rows are real
    NAMES = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", q_norm="q_norm.weight",
                 k_norm="k_norm.weight", gate="g_proj.weight", sink="sink", q_bias="q_proj.bias", k_bias="k_proj.bias",
                 v_bias="v_proj.bias", temp="temperature", r1="distance.r1", r2="distance.r2")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = param(spec, "hidden", int)
        self.heads = param(spec, "heads", int)
        self.kv_heads = param(spec, "kv_heads", int)
        self.head_dim = param(spec, "head_dim", int)
        self.unit_norm = spec.get("qk_norm") == "unit"  # a norm without weights
        self.qk_norm = bool(spec.get("qk_norm", False)) and not self.unit_norm
        self.qk_norm_eps = float(spec.get("qk_norm_eps", 0.0))
        self.window = spec.get("window")
        self.scale = float(spec.get("scale") or self.head_dim ** -0.5)
        self.kv_source = spec.get("kv_source", "own")
        if self.kv_source not in ("own", "shared"):
            raise ValueError(f"kv_source must be 'own' or 'shared', got {self.kv_source!r}")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are not a multiple of {self.kv_heads} kv heads")
        if self.window is not None and int(self.window) < 1:
            raise ValueError(f"window must be positive, got {self.window}")
        pos_spec = spec.get("position") or PartSpec("none")
        self.position = build_part("position", pos_spec, env)
        self.sink = bool(spec.get("sink", False))
        self.learned_sink = spec.get("sink") == "learned"
        self.softcap = float(spec.get("softcap") or 0.0)
        self.chunk = int(spec.get("chunk") or 0)
        if self.softcap < 0 or self.chunk < 0:
            raise ValueError(f"softcap={self.softcap} and chunk={self.chunk} must not be negative")
        self.value_dim = int(spec.get("value_dim") or self.head_dim)
        self.out_gate = spec.get("out_gate")
        if self.out_gate not in (None, "head_sigmoid", "channel_sigmoid"):
            raise ValueError(f"out_gate must be 'head_sigmoid', 'channel_sigmoid' or absent, got {self.out_gate!r}")
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.head_temperature = bool(spec.get("head_temperature", False))
        self.distance_bias = bool(spec.get("distance_bias", False))
        self.keep_first = int(spec.get("keep_first") or 0)
        self.cache_window = spec.get("cache_window")
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ValueError(f"keep_first={self.keep_first} needs a window that it reaches behind")
        self.names = {**self.NAMES, **dict(spec.get("names") or {})}
        self.adjacent = getattr(self.position, "pairing", "halves") == "adjacent"  # how the position encoding pairs channels
        self.general = bool(self.out_gate or self.value_dim != self.head_dim or self.adjacent or self.learned_sink or self.softcap
                            or self.chunk or getattr(self.position, "table_only", False) or self.unit_norm or self.qkv_bias
                            or self.head_temperature or self.distance_bias or self.keep_first or spec.get("general"))
        self.w_sink = None
        self.extras = None
        self.w_bias = self.w_temp = None
        # the general path keeps keys and values in one head size: the larger of the two, in steps of 16
        self.cache_dim = -(-max(self.head_dim, self.value_dim) // 16) * 16 if self.general else self.head_dim
        self.feature_width = self.heads * self.value_dim

    @property
    def gate_width(self) -> int:
        return self.heads * self.value_dim if self.out_gate == "channel_sigmoid" else (self.heads if self.out_gate else 0)

    @property
    def owns_cache(self) -> bool:
        return self.kv_source == "own"

    def cache_need(self):
        if not self.owns_cache:
            return None
        # keys a whole block behind the newest token are never seen again: the cache treats the block as a window
        reach = self._own_reach()
        if self.keep_first:
            reach = 0  # the kept first keys are read for as long as the request runs: no page is given back
        if self.cache_window is not None:
            reach = int(self.cache_window)
        return PagedKV(self.kv_heads, self.cache_dim, reach or None)

    def _own_reach(self) -> int:
        """How many keys back this mixer's own mask reaches (0: all of them)."""
        return min(int(self.window), self.chunk) if self.window and self.chunk else (int(self.window) if self.window else self.chunk)

    def weights(self):
        d, n = self.head_dim, self.names
        w = {n["q"]: WeightDecl((self.heads * d, self.hidden)),
             n["o"]: WeightDecl((self.hidden, self.heads * self.value_dim))}
        if self.owns_cache:
            w[n["k"]] = WeightDecl((self.kv_heads * d, self.hidden))
            w[n["v"]] = WeightDecl((self.kv_heads * self.value_dim, self.hidden))
        if self.out_gate:
            w[n["gate"]] = WeightDecl((self.gate_width, self.hidden))
        if self.learned_sink:
            w[n["sink"]] = WeightDecl((self.heads,), precision="float32")
        if self.qkv_bias:
            w[n["q_bias"]] = WeightDecl((self.heads * d,), precision="float32")
            if self.owns_cache:
                w[n["k_bias"]] = WeightDecl((self.kv_heads * d,), precision="float32")
                w[n["v_bias"]] = WeightDecl((self.kv_heads * self.value_dim,), precision="float32")
        if self.head_temperature:
            w[n["temp"]] = WeightDecl((self.heads,), precision="float32", init="ones_normal")
        if self.distance_bias:
            w[n["r1"]] = WeightDecl((self.heads,), precision="float32")
            w[n["r2"]] = WeightDecl((self.heads,), precision="float32", init="ones_normal")
        if self.qk_norm:
            # the general kernel takes the norm's weights in float32, the others in the run's dtype
            kind = dict(precision="float32") if self.general else {}
            w[n["q_norm"]] = WeightDecl((d,), init="ones_normal", **kind)
            if self.owns_cache:
                w[n["k_norm"]] = WeightDecl((d,), init="ones_normal", **kind)
        return w

    def _stack(self) -> tuple[str, tuple[str, ...]]:
        n = self.names
        kv = (n["k"], n["v"]) if self.owns_cache else ()
        return "qkv_proj.weight", (n["q"],) + kv + ((n["gate"],) if self.out_gate else ())

    def stacks(self):
        # one product makes q, k and v (miniserve/model/fused.py:41-95 joins the same rows), and the gate
        return dict([self._stack()]) if self.owns_cache or self.out_gate else {}

    def bind(self, tensors):
        n = self.names
        if self.owns_cache or self.out_gate:
            self.w_qkv = self.joined(tensors, *self._stack())
        else:
            self.w_qkv = tensors[n["q"]].contiguous()
        self.input_rows = self.w_qkv.shape[0]  # rows of the input product that are this mixer's (before any padding)
        if self.general and self.w_qkv.shape[0] % 8:
            # rows of the product's output start on 16 bytes: a few zero rows at the end
            pad = torch.zeros((-self.w_qkv.shape[0] % 8, self.hidden), dtype=self.w_qkv.dtype, device=self.w_qkv.device)
            self.w_qkv = torch.cat((self.w_qkv, pad), dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        self.w_q_norm = tensors[n["q_norm"]].contiguous() if self.qk_norm else None
        self.w_k_norm = tensors[n["k_norm"]].contiguous() if self.qk_norm and self.owns_cache else None
        self.w_sink = tensors[n["sink"]].float().contiguous() if self.learned_sink else None
        if self.qkv_bias:
            parts = (n["q_bias"], n["k_bias"], n["v_bias"]) if self.owns_cache else (n["q_bias"],)
            self.w_bias = torch.cat([tensors[p].float().reshape(-1) for p in parts]).contiguous()
        self.w_temp = tensors[n["temp"]].float().contiguous() if self.head_temperature else None
        r1 = tensors[n["r1"]].float().contiguous() if self.distance_bias else None
        r2 = tensors[n["r2"]].float().contiguous() if self.distance_bias else None
        if self.learned_sink or self.softcap or self.chunk or self.distance_bias or self.keep_first:
            self.extras = ops.AttentionExtras(self.w_sink, self.softcap, self.chunk, r1, r2, self.keep_first)

    @property
    def reach(self) -> int | None:
        """How far back the cache keeps keys for this mixer (what the kernels take as their window): the window, or the
        block of a mask by blocks (which then does the masking itself, inside that reach)."""
        return self._own_reach() or None

    def features(self, x: torch.Tensor, ctx, cache, out: torch.Tensor | None, scale: float = 1.0, proj: torch.Tensor | None = None,
                 defer_gate: bool = False, raw: bool = False):
        """The general path up to the output projection's input: ``out`` [T, heads * value_dim] (a view
        whose rows may be part of wider ones) = scale * gate * attention. ``proj``: the q|k|v|gate projection if
        the caller made it already (columns of a wider product, in this mixer's order). ``defer_gate`` (per-channel
        gates only): nothing is written; attention's output [T, heads, D] and the gate's columns are returned for a
        caller that applies the gate together with something else."""
        t = x.shape[0]
        dt, dev = self.env.dtype, x.device
        nq, nkv, dk, dv, dc = self.heads, self.kv_heads, self.head_dim, self.value_dim, self.cache_dim
        if proj is None:
            proj = ops.linear(x, self.w_qkv, stream=ctx.stream, out=ctx.buffer("attn.qkv", (t, self.w_qkv.shape[0]), dt, dev))
        at_k = nq * dk
        at_v, at_g = ((nq + nkv) * dk, (nq + nkv) * dk + nkv * dv) if self.owns_cache else (at_k, at_k)
        q = ctx.buffer("attn.q", (t, nq, dc), dt, dev)
        _, rotary_dim = self.position.kernel_table()
        own = self.owns_cache  # else the keys and values are another entry's, as its cache holds them
        ops.qkv_prepare(q, cache.k if own else None, cache.v if own else None, proj[:, :at_k], proj[:, at_k:at_v] if own else None,
                        proj[:, at_v:at_g] if own else None, self.w_q_norm, self.w_k_norm,
                        self.position.step_table(ctx), rotary_dim, self.adjacent, self.qk_norm_eps,
                        ctx.positions, ctx.row_of_token, ctx.page_indptr[cache.group], ctx.page_indices[cache.group],
                        cache.page_size, ctx.status, stream=ctx.stream, bias=self.w_bias, unit_norm=self.unit_norm, q_scale=self.w_temp)
        att = ctx.buffer("attn.out", (t, nq, dc), dt, dev)
        ops.attention(att, q, cache.k, cache.v, ctx, cache.group, self.scale, self.reach, self.sink, extras=self.extras)
        if raw:  # the caller takes attention's output [T, heads, D] itself (no gate, values as wide as the cache's heads)
            return att
        if self.out_gate == "channel_sigmoid":
            if defer_gate:
                return att, proj[:, at_g:at_g + nq * dv]
            ops.channel_gate(out, att, proj[:, at_g:at_g + nq * dv], dv, scale, stream=ctx.stream)
            return
        gate = proj[:, at_g:at_g + nq] if self.out_gate else None
        ops.head_gate(out, att, gate, dv, scale, stream=ctx.stream)

    def forward(self, x: torch.Tensor, ctx, cache):
        """Returns the mixer's addend to the residual stream: a tensor [T, hidden]."""
        t = x.shape[0]
        dt, dev = self.env.dtype, x.device
        if self.general:
            if not self.out_gate and self.value_dim == self.cache_dim:
                # nothing to cut and nothing to gate: attention's output is the output product's input as it stands
                feat = self.features(x, ctx, cache, None, raw=True).view(t, self.feature_width)
            else:
                feat = ctx.buffer("attn.feat", (t, self.feature_width), dt, dev)
                self.features(x, ctx, cache, feat)
            return ops.linear(feat, self.w_o, stream=ctx.stream, out=ctx.buffer("attn.proj", (t, self.w_o.shape[0]), dt, dev))
        q = ctx.buffer("attn.q", (t, self.heads, self.head_dim), dt, dev)
        inv_freq, rotary_dim = self.position.kernel_table()
        indptr, indices = ctx.page_indptr[cache.group], ctx.page_indices[cache.group]
        if (self.owns_cache
                and ops.qkv_fused_ok(x, self.w_qkv, self.heads, self.kv_heads, self.head_dim, rotary_dim if inv_freq is not None else 0,
                                     cache.k, self.w_q_norm, self.w_k_norm)):
            # prompt steps: norm, rotation and cache write in the product's epilogue
            tiled = None
            if inv_freq is not None:
                table = self.position.step_table(ctx)
                key = ("rope_table_tiled", table.data_ptr())
                tiled = ctx.step_cache.get(key)
                if tiled is None:  # once per step; every layer with the same table shares it
                    tiled = ctx.step_cache[key] = ops.rope_table_tiled(table, stream=ctx.stream)
            ops.qkv_norm_rope_kv(q, cache.k, cache.v, x, self.w_qkv, self.w_q_norm, self.w_k_norm, tiled, self.qk_norm_eps,
                                 ctx.positions, ctx.row_of_token, indptr, indices, cache.page_size, stream=ctx.stream)
        else:
            qkv = ops.linear(x, self.w_qkv, stream=ctx.stream, out=ctx.buffer("attn.qkv", (t, self.w_qkv.shape[0]), dt, dev))
            ops.qk_norm_rope_kv(
                q, cache.k if self.owns_cache else None, cache.v if self.owns_cache else None, qkv,
                self.w_q_norm, self.w_k_norm, inv_freq, rotary_dim, self.qk_norm_eps, ctx.positions,
                ctx.row_of_token, indptr, indices, cache.page_size, ctx.status, stream=ctx.stream,
                cos_sin=self.position.step_table(ctx))
        out = ctx.buffer("attn.out", (t, self.heads, self.head_dim), dt, dev)
        ops.attention(out, q, cache.k, cache.v, ctx, cache.group, self.scale, self.window, self.sink)
        return ops.linear(out.view(t, self.heads * self.head_dim), self.w_o, stream=ctx.stream,
                          out=ctx.buffer("attn.proj", (t, self.w_o.shape[0]), dt, dev))
