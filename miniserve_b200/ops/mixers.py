"""Python faces of the kernels in ``csrc/mixer_pointwise.cu`` and ``csrc/recurrence.cu``: Dynamic Tanh,
tanh-GELU, the general step between a q|k|v projection and attention, gates on attention's output, and
the linear-attention recurrences with what comes before and after them.

Several operands are column ranges of a wider row (one product makes q, k, v and gates side by side):
such an operand is passed as a 2-d view whose last stride is 1; its row stride goes to the kernel."""

from __future__ import annotations

import torch

from . import native


def _dt(dtype: torch.dtype) -> int:
    return {torch.float32: 0, torch.bfloat16: 1}[dtype]


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(stream) -> int:
    return torch.cuda.current_stream().cuda_stream if stream is None else stream


def _rows(t: torch.Tensor) -> int:
    """Row stride of a 2-d operand whose rows are contiguous."""
    assert t.is_cuda and t.dim() == 2 and (t.stride(1) == 1 or t.shape[1] == 1), "operand rows must be contiguous"
    return t.stride(0)


def _f32(*tensors) -> None:
    for t in tensors:
        assert t is None or (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous())


def add_dyt(out, residual, delta, weight, bias, alpha, rows=None, num_rows=None, write_residual=True, stream=None) -> None:
    """out[i] = tanh(alpha * (residual[r] + delta[r])) * weight + bias with r = rows[i] (or i); the sum
    is written back to ``residual`` when there is no gather. float32 arithmetic, float32 parameters."""
    _f32(residual, weight, bias, alpha)
    hidden = residual.shape[-1]
    n = out.shape[0] if num_rows is None else num_rows
    assert out.is_contiguous() and out.shape[-1] == hidden and weight.numel() == hidden and bias.numel() == hidden
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous())
    native.mixers_check(native.mixers().ms_add_dyt(
        _ptr(out), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(rows), n, hidden,
        int(write_residual and rows is None), _dt(out.dtype), _stream(stream)))


def gelu_tanh(out: torch.Tensor, x: torch.Tensor, stream=None) -> None:
    """out = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), in float32, rounded once (may be in place)."""
    assert out.is_contiguous() and x.is_contiguous() and out.dtype == x.dtype and out.numel() == x.numel()
    native.mixers_check(native.mixers().ms_gelu_tanh(_ptr(out), _ptr(x), x.numel(), _dt(x.dtype), _stream(stream)))


def scale_(x: torch.Tensor, s: float, stream=None) -> None:
    _f32(x)
    native.mixers_check(native.mixers().ms_scale_f32(_ptr(x), float(s), x.numel(), _stream(stream)))


def axpby(out: torch.Tensor, x: torch.Tensor, y: torch.Tensor, a: float, b: float, stream=None) -> None:
    assert out.is_contiguous() and x.is_contiguous() and y.is_contiguous() and x.dtype == y.dtype == out.dtype
    assert x.numel() == y.numel() == out.numel()
    native.mixers_check(native.mixers().ms_axpby(_ptr(out), _ptr(x), _ptr(y), float(a), float(b), x.numel(), _dt(x.dtype),
                                                  _stream(stream)))


def head_gate(out: torch.Tensor, attn: torch.Tensor, gate: torch.Tensor | None, value_dim: int, scale: float, stream=None) -> None:
    """out[t, h * dv + c] = scale * sigmoid(gate[t, h]) * attn[t, h, c] for c < dv; ``attn`` [T, heads, D],
    ``out`` and ``gate`` 2-d views of wider rows. Without ``gate`` only the scale and the cut to dv remain."""
    t, nq, d = attn.shape
    assert attn.is_contiguous() and out.shape == (t, nq * value_dim) and out.dtype == attn.dtype
    assert gate is None or (gate.shape == (t, nq) and gate.dtype == attn.dtype)
    native.mixers_check(native.mixers().ms_head_gate(
        _ptr(out), _rows(out), _ptr(attn), _ptr(gate), 0 if gate is None else _rows(gate), t, nq, d, value_dim, float(scale),
        _dt(attn.dtype), _stream(stream)))


def qkv_prepare(q_out, k_pool, v_pool, q, k, v, q_norm_w, k_norm_w, cos_sin, rotary_dim: int, adjacent: bool, eps: float,
                positions, row_of_token, page_indptr, page_indices, page_size: int, status, stream=None, bias=None,
                unit_norm: bool = False, q_scale=None) -> None:
    """Per-head RMS norm of q and k (float32 weights or None), rotation of the first ``rotary_dim`` channels
    (pairs (2i, 2i+1) if ``adjacent`` else (i, i + rotary_dim/2)) by the step's cos/sin table, q to
    ``q_out`` [T, nq, D] and k, v into their pages [pages, nkv, page_size, D], zero beyond their own
    sizes. ``q`` [T, nq*dk], ``k`` [T, nkv*dk], ``v`` [T, nkv*dv]: views into one projection's rows.
    ``bias``: float32 [nq*dk + nkv*dk + nkv*dv], the projections' biases in the order q, k, v, added first.
    ``unit_norm``: q and k are divided by their root mean square also without norm weights. ``q_scale``: float32 [nq],
    a factor per query head applied last. Without pools (``k_pool``, ``k`` and ``v`` None) only the queries are
    prepared (a mixer that reads another's keys and values); ``bias`` is then [nq*dk]."""
    t, nq, d = q_out.shape
    dk = q.shape[1] // nq
    _f32(q_norm_w, k_norm_w, cos_sin, bias, q_scale)
    assert cos_sin is None or cos_sin.shape == (t, rotary_dim)
    assert q_scale is None or q_scale.numel() == nq
    if k_pool is None:
        assert k is None and v is None and v_pool is None and q.shape == (t, nq * dk) and q.dtype == q_out.dtype
        assert bias is None or bias.numel() == nq * dk
        native.mixers_check(native.mixers().ms_qkv_prepare(
            _ptr(q_out), None, None, q.data_ptr(), _rows(q), 0, 0, 0, _ptr(q_norm_w), None, _ptr(cos_sin), _ptr(positions),
            _ptr(row_of_token), _ptr(page_indptr), _ptr(page_indices), t, nq, 1, dk, dk, d, rotary_dim if cos_sin is not None else 0,
            int(adjacent), float(eps), page_size, 0, _ptr(status), _dt(q.dtype), _stream(stream), _ptr(bias), _ptr(q_scale),
            int(unit_norm)))
        return
    nkv = k_pool.shape[1]
    dv = v.shape[1] // nkv
    assert k.shape == (t, nkv * dk) and q.shape == (t, nq * dk) and v.shape == (t, nkv * dv)
    assert k_pool.shape == v_pool.shape and k_pool.shape[2] == page_size and k_pool.shape[3] == d
    assert q.dtype == k.dtype == v.dtype == q_out.dtype == k_pool.dtype
    assert bias is None or bias.numel() == (nq + nkv) * dk + nkv * dv
    ld = _rows(q)
    assert _rows(k) == ld and _rows(v) == ld, "q, k and v must be columns of the same rows"
    item = q.element_size()
    base = min(q.data_ptr(), k.data_ptr(), v.data_ptr())
    offs = [(x.data_ptr() - base) // item for x in (q, k, v)]
    native.mixers_check(native.mixers().ms_qkv_prepare(
        _ptr(q_out), _ptr(k_pool), _ptr(v_pool), base, ld, offs[0], offs[1], offs[2], _ptr(q_norm_w), _ptr(k_norm_w),
        _ptr(cos_sin), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr), _ptr(page_indices), t, nq, nkv, dk, dv, d,
        rotary_dim if cos_sin is not None else 0, int(adjacent), float(eps), page_size, k_pool.shape[0], _ptr(status),
        _dt(q.dtype), _stream(stream), _ptr(bias), _ptr(q_scale), int(unit_norm)))


def add_layernorm(out, residual, delta, weight, bias, eps: float, rows=None, num_rows=None, write_residual=True, delta_scale: float = 1.0,
                  out2=None, weight2=None, bias2=None, stream=None) -> None:
    """out[i] = (h - mean(h)) / sqrt(mean((h - mean(h))^2) + eps) * weight + bias with h = residual[r] + delta_scale *
    delta[r], r = rows[i] (or i); h is written back to ``residual`` when there is no gather. ``out2`` with ``weight2``
    and ``bias2``: a second norm of the same rows (the statistics are computed once). float32 arithmetic and parameters."""
    _f32(residual, weight, bias, weight2, bias2)
    hidden = residual.shape[-1]
    n = out.shape[0] if num_rows is None else num_rows
    assert out.is_contiguous() and out.shape[-1] == hidden and weight.numel() == hidden and bias.numel() == hidden
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous())
    assert out2 is None or (out2.shape == out.shape and out2.dtype == out.dtype and out2.is_contiguous() and weight2.numel() == hidden
                            and bias2.numel() == hidden)
    native.mixers_check(native.mixers().ms_add_layernorm(
        _ptr(out), _ptr(out2), _ptr(residual), _ptr(delta), float(delta_scale), _ptr(weight), _ptr(bias), _ptr(weight2), _ptr(bias2),
        _ptr(rows), float(eps), n, hidden, int(write_residual and rows is None), _dt(out.dtype), _stream(stream)))


def token_shift(out, h, state, mix, ctx, update: bool = True) -> None:
    """out[t] = h[t] + (h[t - 1] - h[t]) * mix (float32 [width]); the token before a row's first one in this step is the
    row's slot of ``state`` [slots, width], or zeros where the row starts its sequence. ``out`` is not ``h``. With
    ``update`` the same launch leaves each row's last h of this step in its slot."""
    t, width = h.shape
    _f32(mix)
    assert out.shape == h.shape and out.dtype == h.dtype == state.dtype and out.is_contiguous() and h.is_contiguous()
    assert state.is_contiguous() and state.shape[1] == width and mix.numel() == width and out.data_ptr() != h.data_ptr()
    native.mixers_check(native.mixers().ms_token_shift(
        _ptr(out), _ptr(h), _ptr(state), _ptr(mix), _ptr(ctx.row_of_token), _ptr(ctx.cu_q), _ptr(ctx.q_start), _ptr(ctx.state_slot),
        t, width, int(update), _dt(h.dtype), ctx.stream))


def shift_state_update(state, h, ctx) -> None:
    """state[slot of row] = h[the row's last token of this step], for every row of the step."""
    assert h.is_contiguous() and state.is_contiguous() and state.dtype == h.dtype and state.shape[1] == h.shape[1]
    native.mixers_check(native.mixers().ms_shift_state_update(
        _ptr(state), _ptr(h), _ptr(ctx.cu_q), _ptr(ctx.state_slot), ctx.num_rows, h.shape[1], _dt(h.dtype), ctx.stream))


def clamped_glu(out, gate_up, bias, limit: float, alpha: float, shift: float, stream=None) -> None:
    """out[t, c] = g * sigmoid(alpha * g) * (u + shift), g = min(gate_up[t, c] + bias[c], limit), u = clamp(gate_up[t, I + c] +
    bias[I + c], -limit, limit); ``bias`` float32 [2 I] or None; a negative ``limit``: no clamps. float32 arithmetic, one rounding."""
    t, inter = out.shape
    _f32(bias)
    assert gate_up.shape == (t, 2 * inter) and gate_up.dtype == out.dtype and out.is_contiguous() and gate_up.is_contiguous()
    assert bias is None or bias.numel() == 2 * inter
    native.mixers_check(native.mixers().ms_clamped_glu(_ptr(out), _ptr(gate_up), _ptr(bias), t, inter, float(limit), float(alpha),
                                                       float(shift), _dt(out.dtype), _stream(stream)))


def sum_bias(out, a, b=None, vec=None, stream=None) -> None:
    """out = a (+ b) (+ vec on every row); a, b and out [rows, width] in the run's dtype (out may be a), vec float32 [width]."""
    rows, width = a.shape
    _f32(vec)
    assert out.shape == a.shape and out.dtype == a.dtype and out.is_contiguous() and a.is_contiguous()
    assert b is None or (b.shape == a.shape and b.dtype == a.dtype and b.is_contiguous())
    assert vec is None or vec.numel() == width
    native.mixers_check(native.mixers().ms_sum_bias(_ptr(out), _ptr(a), _ptr(b), _ptr(vec), rows, width, _dt(a.dtype), _stream(stream)))


def decay_scan(o_out, state, q, k, v, z, z_bias, decay_coef, z_sign: float, beta, ctx, heads: int, dk: int, dv: int,
               q_scale: float, delta: bool, head_decay: bool = False, v_scale=None) -> None:
    """The token-by-token recurrence of every row of the step (``csrc/recurrence.cu``), from each
    request's slot of ``state`` [slots, heads, dv, dk] float32 (zero where a row starts at position 0)
    and back into it; o_out [T, heads, dv] float32. q, k [T, groups*dk], v [T, heads*dv], z [T, heads*dk]
    and beta [T, heads] are 2-d views; z_bias [heads*dk], decay_coef [heads] float32.
    ``head_decay``: z [T, heads] float32 holds the decays themselves, one for all key channels of a head and token
    (z_bias, decay_coef and z_sign are not used). ``v_scale`` [T, heads] float32: v counts times it, per token and head."""
    t = o_out.shape[0]
    _f32(o_out, state, z_bias, decay_coef, v_scale)
    assert o_out.shape == (t, heads, dv) and state.shape[1:] == (heads, dv, dk)
    groups = q.shape[1] // dk
    assert q.shape == (t, groups * dk) and k.shape == q.shape and v.shape == (t, heads * dv)
    assert z.shape == (t, heads if head_decay else heads * dk) and (not head_decay or (z.dtype == torch.float32 and not delta))
    assert q.dtype == k.dtype == v.dtype and (beta is None or beta.dtype == z.dtype)
    assert v_scale is None or v_scale.shape == (t, heads)
    if not delta and not ctx.decode_only and t >= SEGMENT_MIN_TOKENS and SEGMENTS > 1:
        return _decay_scan_segmented(o_out, state, q, k, v, z, z_bias, decay_coef, z_sign, ctx, heads, dk, dv, q_scale, head_decay,
                                     v_scale)
    ready = int(head_decay)
    if not ctx.decode_only and not head_decay:
        # a prompt portion: exponentials and logarithms for all tokens at once, not inside the serial walk
        # (a decode step, one token a row, works them out while it stages the token)
        width = heads * dk + (heads if beta is not None else 0)
        pre = ctx.buffer("scan.decay", (t, width), torch.float32, o_out.device)
        native.recurrence_check(native.recurrence().ms_decay_from_logits(
            _ptr(pre), _ptr(z), _rows(z), _ptr(z_bias), _ptr(decay_coef), float(z_sign), _ptr(beta),
            0 if beta is None else _rows(beta), t, heads, dk, _dt(z.dtype), ctx.stream))
        z, beta, ready = pre[:, :heads * dk], (pre[:, heads * dk:] if beta is not None else None), 1
    native.recurrence_check(native.recurrence().ms_decay_scan(
        _ptr(o_out), _ptr(state), _ptr(q), _rows(q), _ptr(k), _rows(k), heads // groups, _ptr(v), _rows(v), _ptr(z), _rows(z),
        _ptr(z_bias), _ptr(decay_coef), float(z_sign), ready, _ptr(beta), 0 if beta is None else _rows(beta), _ptr(ctx.cu_q),
        _ptr(ctx.q_start), _ptr(ctx.state_slot), ctx.num_rows, heads, dk, dv, float(q_scale), int(delta), _dt(q.dtype),
        _dt(z.dtype), int(head_decay), _ptr(v_scale), ctx.stream))


def conv_silu_unit(out, x, conv_state, weight, ctx, unit_heads: int, dk: int, other_heads: int, dv: int, unit_eps: float,
                   bias=None) -> None:
    """out [T, C] float32 = SiLU(causal convolution over time of the C channels ``x`` [T, C], a view),
    the first ``unit_heads`` heads of dk channels then divided by sqrt(sum of squares + unit_eps).
    ``weight`` [C, taps] float32 (``bias`` [C] float32 is added if given); ``conv_state`` [slots, taps - 1, C] holds each
    request's last inputs."""
    t, c = out.shape
    taps = weight.shape[1]
    _f32(out, weight, bias)
    assert bias is None or bias.numel() == c
    assert x.shape == (t, c) and weight.shape[0] == c and conv_state.dtype == x.dtype and conv_state.is_contiguous()
    assert conv_state.shape[1:] == (max(taps - 1, 0), c)
    native.recurrence_check(native.recurrence().ms_conv_silu_unit(
        _ptr(out), _ptr(x), _rows(x), _ptr(conv_state), _ptr(weight), _ptr(ctx.row_of_token), _ptr(ctx.cu_q), _ptr(ctx.q_start),
        _ptr(ctx.state_slot), t, c, taps, unit_heads, dk, other_heads, dv, float(unit_eps), _dt(x.dtype), _ptr(bias), ctx.stream))


def conv_state_update(conv_state, x, ctx, taps: int) -> None:
    """Each row's slot of ``conv_state`` [slots, taps - 1, C] becomes the last taps - 1 inputs ``x`` [T, C]
    of its sequence after this step (older entries move up when the portion is shorter than that)."""
    assert conv_state.dtype == x.dtype and conv_state.is_contiguous()
    native.recurrence_check(native.recurrence().ms_conv_state_update(
        _ptr(conv_state), _ptr(x), _rows(x), _ptr(ctx.cu_q), _ptr(ctx.q_start), _ptr(ctx.state_slot), ctx.num_rows, x.shape[1],
        taps, _dt(x.dtype), ctx.stream))


# The decay rule is linear in the state with a diagonal factor, so the rows of a step with many tokens are cut into
# SEGMENTS pieces that are walked at the same time (``csrc/recurrence.cu``). Whether a step is cut follows from its
# number of tokens alone (what a captured graph is keyed by), never from how the tokens are shared among rows.
SEGMENTS = 8
SEGMENT_MIN_TOKENS = 512


def _decay_scan_segmented(o_out, state, q, k, v, z, z_bias, decay_coef, z_sign, ctx, heads, dk, dv, q_scale, head_decay=False,
                          v_scale=None) -> None:
    from types import SimpleNamespace

    t, dev, p, rows = o_out.shape[0], o_out.device, SEGMENTS, ctx.num_rows
    lib = native.recurrence()
    key = ("scan.segments", p)
    seg = ctx.step_cache.get(key) if hasattr(ctx, "step_cache") else None
    if seg is None:  # the same for every layer of the step
        ints = torch.empty(3 * rows * p + 1, dtype=torch.int32, device=dev)
        seg = (ints[:rows * p + 1], ints[rows * p + 1:2 * rows * p + 1], ints[2 * rows * p + 1:])
        native.recurrence_check(lib.ms_segment_setup(_ptr(seg[0]), _ptr(seg[1]), _ptr(seg[2]), _ptr(ctx.cu_q), rows, p, ctx.stream))
        if hasattr(ctx, "step_cache"):
            ctx.step_cache[key] = seg
    seg_cu, seg_zero, seg_slot = seg
    dkz = 1 if head_decay else dk
    if head_decay:
        decay = z
    else:
        decay = ctx.buffer("scan.decay", (t, heads * dk), torch.float32, dev)
        native.recurrence_check(lib.ms_decay_from_logits(_ptr(decay), _ptr(z), _rows(z), _ptr(z_bias), _ptr(decay_coef), float(z_sign),
                                                         None, 0, t, heads, dk, _dt(z.dtype), ctx.stream))
    ends = ctx.buffer("scan.ends", (rows * p, heads, dv, dk), torch.float32, dev)
    before = ctx.buffer("scan.before", (rows * p, heads, dv, dk), torch.float32, dev)
    cum = ctx.buffer("scan.cum", (t, heads * dkz), torch.float32, dev)
    pieces = SimpleNamespace(cu_q=seg_cu, q_start=seg_zero, state_slot=seg_slot, num_rows=rows * p, stream=ctx.stream)
    groups = q.shape[1] // dk
    native.recurrence_check(lib.ms_decay_scan(
        _ptr(o_out), _ptr(ends), _ptr(q), _rows(q), _ptr(k), _rows(k), heads // groups, _ptr(v), _rows(v), _ptr(decay), _rows(decay),
        _ptr(z_bias), _ptr(decay_coef), float(z_sign), 1, None, 0, _ptr(pieces.cu_q), _ptr(pieces.q_start), _ptr(pieces.state_slot),
        pieces.num_rows, heads, dk, dv, float(q_scale), 0, _dt(q.dtype), 0, int(head_decay), _ptr(v_scale), ctx.stream))
    native.recurrence_check(lib.ms_segment_finish(
        _ptr(o_out), _ptr(state), _ptr(ends), _ptr(before), _ptr(cum), _ptr(decay), _rows(decay), _ptr(q), _rows(q), heads // groups,
        _ptr(seg_cu), _ptr(ctx.q_start), _ptr(ctx.state_slot), rows, t, p, heads, dk, dv, float(q_scale), _dt(q.dtype), int(head_decay),
        ctx.stream), launches=3)


def ssm_step_decay(out, raw, bias, coef, stream=None) -> None:
    """out [2, T, H] float32: out[0] the step sizes softplus(raw[t, h] + bias[h]), out[1] the decays
    exp(-coef[h] * step size); ``raw`` [T, H] a view, bias and coef float32 [H]."""
    t, h = raw.shape
    _f32(out, bias, coef)
    assert out.shape == (2, t, h) and bias.numel() == h and coef.numel() == h
    native.recurrence_check(native.recurrence().ms_ssm_step_decay(_ptr(out), _ptr(raw), _rows(raw), _ptr(bias), _ptr(coef), t, h,
                                                                  _dt(raw.dtype), _stream(stream)))


def gated_group_norm(out, o, x, skip, gate, weight, parts: int, dv: int, eps: float, stream=None) -> None:
    """y = (o + skip[head] * x) * silu(gate) over the ``width`` channels of a token (head = channel // dv), then each of
    ``parts`` equal parts of y divided by its own root mean square, times ``weight`` [width]. ``o`` [T, width] float32;
    ``x`` [T, width] float32 (a view) and ``skip`` [heads] float32, or both None; ``out`` and ``gate`` 2-d views in the
    run's dtype. The gate comes before the norm."""
    t, width = o.shape
    _f32(o, weight, skip)
    assert out.shape == (t, width) and gate.shape == (t, width) and gate.dtype == out.dtype and weight.numel() == width
    assert (x is None) == (skip is None) and (x is None or (x.shape == (t, width) and x.dtype == torch.float32))
    native.recurrence_check(native.recurrence().ms_gated_group_norm(
        _ptr(out), _rows(out), _ptr(o), _ptr(x), 0 if x is None else _rows(x), _ptr(skip), _ptr(gate), _rows(gate), _ptr(weight), t,
        width, parts, dv, float(eps), _dt(out.dtype), _stream(stream)))


GATE_KINDS = {"silu": 0, "sigmoid": 1}


def head_norm_gate(out, o, weight, gate, eps: float, scale: float, gate_kind: str, stream=None) -> None:
    """out[t, h*dv + c] = scale * o[t, h, c] / sqrt(mean_c o^2 + eps) * weight[c] * act(gate[t, h*dv + c]);
    ``o`` [T, heads, dv] float32, ``out`` and ``gate`` 2-d views, act SiLU or sigmoid."""
    t, heads, dv = o.shape
    _f32(o, weight)
    assert out.shape == (t, heads * dv) and gate.shape == (t, heads * dv) and gate.dtype == out.dtype and weight.numel() == dv
    native.recurrence_check(native.recurrence().ms_head_norm_gate(
        _ptr(out), _rows(out), _ptr(o), _ptr(weight), _ptr(gate), _rows(gate), t, heads, dv, float(eps), float(scale),
        GATE_KINDS[gate_kind], _dt(out.dtype), _stream(stream)))


# ---------------------------------------------------------------- csrc/block_ops.cu

def add_rmsnorm_scaled(out, residual, delta, delta_scale: float, weight, weight_offset: float, eps: float, rows=None, num_rows=None,
                       write_residual=True, stream=None) -> None:
    """out[i] = h / sqrt(mean(h^2) + eps) * (weight_offset + weight) with h = residual[r] + delta_scale * delta[r],
    r = rows[i] (or i); h is written back to ``residual`` when there is no gather. float32 arithmetic, float32 weight."""
    _f32(residual, weight)
    hidden = residual.shape[-1]
    n = out.shape[0] if num_rows is None else num_rows
    assert out.is_contiguous() and out.shape[-1] == hidden and weight.numel() == hidden
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous())
    native.mixers_check(native.mixers().ms_add_rmsnorm_scaled(
        _ptr(out), _ptr(residual), _ptr(delta), float(delta_scale), _ptr(weight), float(weight_offset), _ptr(rows), float(eps), n,
        hidden, int(write_residual and rows is None), _dt(out.dtype), _stream(stream)))


def stream_concat(out, residual, delta, delta_scale: float, table, ids, first: bool = True, second: bool = True, stream=None) -> None:
    """out [T, 2W] in the run's dtype: columns 0..W-1 = residual + delta_scale * delta (float32 sum, rounded once),
    columns W..2W-1 = table[ids] (``first`` / ``second``: which half to write)."""
    _f32(residual)
    t, w = residual.shape
    assert out.is_contiguous() and out.shape == (t, 2 * w) and table.dtype == out.dtype and table.shape[1] == w and table.is_contiguous()
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == (t, w))
    assert ids.dtype == torch.int32 and ids.numel() >= t
    native.mixers_check(native.mixers().ms_stream_concat(
        _ptr(out), _ptr(residual), _ptr(delta), float(delta_scale), _ptr(table), _ptr(ids), table.shape[0], t, w, int(first),
        int(second), _dt(out.dtype), _stream(stream)))


def add_row_vector(x: torch.Tensor, vec: torch.Tensor, stream=None) -> None:
    """x [T, W] += vec [W], float32, in place."""
    _f32(x, vec)
    assert x.dim() == 2 and vec.numel() == x.shape[1]
    native.mixers_check(native.mixers().ms_add_row_vector(_ptr(x), _ptr(vec), x.shape[0], x.shape[1], _stream(stream)))


def relu_squared(out: torch.Tensor, x: torch.Tensor, stream=None) -> None:
    """out = max(x, 0)^2, in float32, rounded once; both 2-d views whose rows may be part of wider ones (may be in place)."""
    assert out.shape == x.shape and out.dtype == x.dtype
    native.mixers_check(native.mixers().ms_relu_squared(_ptr(out), _rows(out), _ptr(x), _rows(x), x.shape[0], x.shape[1],
                                                         _dt(x.dtype), _stream(stream)))


def channel_gate(out: torch.Tensor, attn: torch.Tensor, gate: torch.Tensor, value_dim: int, scale: float = 1.0, stream=None) -> None:
    """out[t, h * dv + c] = scale * sigmoid(gate[t, h * dv + c]) * attn[t, h, c] for c < dv; ``attn`` [T, heads, D],
    ``out`` and ``gate`` 2-d views of wider rows."""
    t, nq, d = attn.shape
    assert attn.is_contiguous() and out.shape == (t, nq * value_dim) and out.dtype == attn.dtype
    assert gate.shape == (t, nq * value_dim) and gate.dtype == attn.dtype
    native.mixers_check(native.mixers().ms_channel_gate(
        _ptr(out), _rows(out), _ptr(attn), _ptr(gate), _rows(gate), t, nq, d, value_dim, float(scale), _dt(attn.dtype), _stream(stream)))


def gate_relu_squared(out: torch.Tensor, attn: torch.Tensor, gate: torch.Tensor, value_dim: int, up: torch.Tensor, stream=None) -> None:
    """One launch for a row that holds a mixer's and a feed-forward's features side by side: out[t, :H*dv] as
    ``channel_gate`` (scale 1), out[t, H*dv:H*dv+I] = max(up[t], 0)^2. ``out``, ``gate`` and ``up`` are 2-d views of wider rows."""
    t, nq, d = attn.shape
    inter = up.shape[1]
    assert attn.is_contiguous() and out.shape == (t, nq * value_dim + inter) and out.dtype == attn.dtype == gate.dtype == up.dtype
    assert gate.shape == (t, nq * value_dim) and up.shape[0] == t
    native.mixers_check(native.mixers().ms_gate_relu_squared(
        _ptr(out), _rows(out), _ptr(attn), _ptr(gate), _rows(gate), _ptr(up), _rows(up), t, nq, d, value_dim, inter, _dt(attn.dtype),
        _stream(stream)))


def rope_table_scaled(positions: torch.Tensor, inv_freq: torch.Tensor, factor: float, num_tokens: int, rotary_dim: int,
                      stream=None) -> torch.Tensor:
    """float32 [T, rotary_dim]: factor * cos, then factor * sin, of position * inv_freq for every token of a step."""
    _f32(inv_freq)
    table = torch.empty((num_tokens, rotary_dim), dtype=torch.float32, device=inv_freq.device)
    native.mixers_check(native.mixers().ms_rope_table_scaled(_ptr(table), _ptr(positions), _ptr(inv_freq), float(factor), num_tokens,
                                                              rotary_dim, _stream(stream)))
    return table


def latent_prepare(pool, latent, weight, eps: float, positions, row_of_token, page_indptr, page_indices, page_size: int, status,
                   stream=None) -> None:
    """``latent`` [T, R] (a view into a projection's rows) over its root mean square, times the float32 ``weight`` [R],
    into each token's slot of ``pool`` [pages, 1, page_size, D], zero from R on."""
    _f32(weight)
    t, rank = latent.shape
    assert pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[2] == page_size and pool.shape[3] >= rank and pool.dtype == latent.dtype
    assert weight.numel() == rank
    native.mixers_check(native.mixers().ms_latent_prepare(
        _ptr(pool), _ptr(latent), _rows(latent), 0, _ptr(weight), float(eps), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr),
        _ptr(page_indices), t, rank, pool.shape[3], page_size, pool.shape[0], _ptr(status), _dt(latent.dtype), _stream(stream)))


def row_rmsnorm(out, x, weight, eps: float, stream=None) -> None:
    """out[t] = x[t] / sqrt(mean x[t]^2 + eps) * weight over the columns of 2-d views ``x`` and ``out`` (rows may be part
    of wider ones); float32 statistics, ``weight`` float32."""
    _f32(weight)
    t, n = x.shape
    assert out.shape == (t, n) and out.dtype == x.dtype and weight.numel() == n
    native.mixers_check(native.mixers().ms_row_rmsnorm(_ptr(out), _rows(out), _ptr(x), _rows(x), _ptr(weight), t, n, float(eps),
                                                       _dt(x.dtype), _stream(stream)))


def latent_rope_prepare(pool, kv, weight, eps: float, q, q_dim: int, q_out, cos_sin, positions, row_of_token, page_indptr, page_indices,
                        page_size: int, status, stream=None) -> None:
    """What latent attention with a rotated part caches and asks with. ``kv`` [T, R + rot] (a view into a projection's
    rows): its first R columns over their root mean square, times the float32 ``weight`` [R], and its last rot columns
    turned by the token's position (``cos_sin`` float32 [T, rot]: cosines of the pairs (i, i + rot / 2), then sines), go
    into the token's slot of ``pool`` [pages, 1, page_size, D] side by side, zeros behind. ``q`` [T, H, q_dim + rot]
    contiguous: every head's last rot channels, turned likewise, go to ``q_out`` [T, H, D] at columns R .. R + rot
    (zeros behind); the first R columns of ``q_out`` are the caller's."""
    _f32(weight, cos_sin)
    t, width = kv.shape
    rot = cos_sin.shape[1]
    rank = width - rot
    heads = q.shape[1]
    d = pool.shape[3]
    assert pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[2] == page_size and d >= width and pool.dtype == kv.dtype
    assert weight.numel() == rank and cos_sin.shape == (t, rot) and q.is_contiguous() and q.shape == (t, heads, q_dim + rot)
    assert q_out.is_contiguous() and q_out.shape == (t, heads, d) and q.dtype == kv.dtype == q_out.dtype
    native.mixers_check(native.mixers().ms_latent_rope_prepare(
        _ptr(pool), _ptr(kv), _rows(kv), _ptr(weight), float(eps), _ptr(q), heads * (q_dim + rot), heads, q_dim, _ptr(q_out),
        _ptr(cos_sin), _ptr(positions), _ptr(row_of_token), _ptr(page_indptr), _ptr(page_indices), t, rank, rot, d, page_size,
        pool.shape[0], _ptr(status), _dt(kv.dtype), _stream(stream)))


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def act_mul(out, gate_up, activation: str, stream=None) -> None:
    """out[t, c] = act(gate_up[t, c]) * gate_up[t, I + c], act SiLU or the tanh form of GELU, computed in float32."""
    t, inter = out.shape
    assert out.is_contiguous() and gate_up.is_contiguous() and gate_up.shape == (t, 2 * inter) and gate_up.dtype == out.dtype
    native.mixers_check(native.mixers().ms_act_mul(_ptr(out), _ptr(gate_up), t, inter, ACTIVATIONS[activation], _dt(out.dtype),
                                                   _stream(stream)))
