"""Python faces of the kernels in ``csrc/routed_experts.cu``: a router's choice, the plan that sorts a step's
(token, choice) pairs by expert, the experts' products over the sorted rows, and the weighted sum."""

from __future__ import annotations

import os

import torch

from . import native
from .mixers import _dt, _f32, _ptr, _rows, _stream

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}
TILE_ROWS = 64       # sorted rows per tile of the float32 and mma.sync products
TC_TILE_ROWS = 128   # of the products on the tcgen05 tensor cores
TC_EXPERTS = os.environ.get("MINISERVE_TC_EXPERTS", "1") != "0"  # bfloat16 experts on the tcgen05 kernel where it takes the shape


def tc_experts_ok(dtype, hidden: int, inter: int, activation: str) -> bool:
    """Whether the experts' products of this shape run on the tcgen05 kernel (``csrc/gemm_tc.cu``, the grouped form):
    bfloat16, SiLU (the kernel's fused epilogue), rows that are multiples of 16 bytes."""
    return TC_EXPERTS and dtype == torch.bfloat16 and activation == "silu" and hidden % 8 == 0 and inter % 8 == 0


def expert_route(idx, wgt, x, router, correction, top: int, group_count: int, group_keep: int, weight_scale: float,
                 renormalize: bool, stream=None, logit_bias=None, gate_w=None, gate_out=None) -> None:
    """idx [T, top] int32 and wgt [T, top] float32: each token's chosen router outputs and their weights.
    Logits ``x router^T`` in float32 (``router`` [R, K] float32), scores their softmax, choice scores the scores plus
    ``correction`` [R] (float32, or None); the R outputs form ``group_count`` equal groups of neighbours of which the
    ``group_keep`` with the largest choice score in them can be chosen from; weights are the chosen scores (without
    the correction) times ``weight_scale``, divided by their sum if ``renormalize`` (which makes them the softmax over
    the chosen logits alone). Ties go to the lower index. ``logit_bias`` [R] float32 is added to the logits themselves.
    ``gate_w`` [K] float32 with ``gate_out`` [T] float32: gate_out[t] = sigmoid(x[t] . gate_w), from the same staged input."""
    t, k = x.shape
    r = router.shape[0]
    _f32(router, correction, wgt, logit_bias, gate_w, gate_out)
    assert (gate_w is None) == (gate_out is None) and (gate_w is None or (gate_w.numel() == k and gate_out.numel() >= t))
    assert logit_bias is None or logit_bias.numel() == r
    assert router.shape == (r, k) and idx.shape == (t, top) and wgt.shape == (t, top) and idx.dtype == torch.int32
    assert idx.is_contiguous() and (correction is None or correction.numel() == r)
    native.experts_check(native.experts().ms_expert_route(
        _ptr(idx), _ptr(wgt), _ptr(x), _rows(x), _ptr(router), _ptr(correction), t, k, r, top, group_count, group_keep,
        float(weight_scale), int(renormalize), _dt(x.dtype), _stream(stream), _ptr(logit_bias), _ptr(gate_w), _ptr(gate_out)))


def expert_max_tiles(slots: int, experts: int, tile_rows: int = TILE_ROWS) -> int:
    """The most tiles of ``tile_rows`` sorted rows a step of ``slots`` (token, choice) pairs over ``experts`` experts can have."""
    return int(native.experts().ms_expert_max_tiles_of(slots, experts, tile_rows))


def expert_plan(pos, perm, offsets, tiles, meta, idx, experts: int, stream=None, tile_rows: int = TILE_ROWS) -> None:
    """Sorts the slots of ``idx`` [T, top] by expert, on the device: ``pos`` [T * top] the sorted row of a slot (-1: the
    slot's choice is not one of the ``experts`` experts with tensors), ``perm`` [T * top] the slot of a sorted row,
    ``offsets`` [experts + 1], ``tiles`` [max_tiles, 2] = (expert, first row), ``meta`` [2] = (tiles, sorted rows)."""
    slots = idx.numel()
    for a in (pos, perm, offsets, tiles, meta, idx):
        assert a.dtype == torch.int32 and a.is_contiguous() and a.is_cuda
    assert pos.numel() == slots and perm.numel() == slots and offsets.numel() == experts + 1 and meta.numel() >= 2
    assert tiles.numel() >= 2 * expert_max_tiles(slots, experts, tile_rows)
    native.experts_check(native.experts().ms_expert_plan_of(_ptr(pos), _ptr(perm), _ptr(offsets), _ptr(tiles), _ptr(meta), _ptr(idx),
                                                            slots, experts, tile_rows, _stream(stream)))


def expert_gather(xs, x, perm, meta, top: int, stream=None) -> None:
    """xs [T * top, K] bfloat16, row r = x[perm[r] // top] for the plan's sorted rows (the rows behind them stay as they are)."""
    slots, k = xs.shape
    assert x.shape[1] == k and xs.is_contiguous() and xs.dtype == x.dtype == torch.bfloat16
    native.experts_check(native.experts().ms_expert_gather(_ptr(xs), _ptr(x), _rows(x), _ptr(perm), _ptr(meta), top, slots, k,
                                                           _stream(stream)))


def expert_products_tc(out, a, w, tiles, meta, offsets, gated: bool, stream=None) -> None:
    """The experts' products over sorted rows on the tcgen05 tensor cores (tiles of ``TC_TILE_ROWS`` rows).
    ``gated``: out [S, I] bfloat16 = silu(a W_gate[e]^T) * (a W_up[e]^T) with ``w`` [E, 2 I, K]; else out [S, N] float32 =
    a W[e]^T with ``w`` [E, N, K]. ``a`` [S, K] bfloat16 in sorted order."""
    from . import device_status

    slots, n = out.shape
    e, w_rows, k = w.shape
    assert a.shape == (slots, k) and a.is_contiguous() and w.is_contiguous() and out.is_contiguous()
    assert a.dtype == w.dtype == torch.bfloat16 and w_rows == (2 * n if gated else n)
    assert out.dtype == (torch.bfloat16 if gated else torch.float32)
    lib = native.gemm_tc()
    native.kernel_check(lib.ms_gemm_tc_experts_bf16(_ptr(out), _ptr(a), _ptr(w), slots, n, k, e, int(gated), _ptr(tiles), _ptr(meta),
                                                    _ptr(offsets), expert_max_tiles(slots, e, TC_TILE_ROWS),
                                                    _ptr(device_status(a.device)), _stream(stream)),
                        lib=lib, errfn="ms_gemm_tc_last_error")


def expert_gate_up(out, x, w_gate_up, perm, top: int, tiles, meta, offsets, activation: str, stream=None) -> None:
    """out [T * top, I] (the run's dtype), row r = act(W_gate[e] h) * (W_up[e] h) with h = x[perm[r] // top] and e the
    expert whose sorted rows hold r; ``w_gate_up`` [E, 2 I, K]: an expert's gate rows, then its up rows."""
    slots, inter = out.shape
    e, two_i, k = w_gate_up.shape
    assert two_i == 2 * inter and x.shape[1] == k and out.is_contiguous() and w_gate_up.is_contiguous()
    assert out.dtype == x.dtype == w_gate_up.dtype
    native.experts_check(native.experts().ms_expert_gemm(
        _ptr(out), _ptr(x), _rows(x), _ptr(perm), top, _ptr(w_gate_up), _ptr(tiles), _ptr(meta), _ptr(offsets),
        expert_max_tiles(slots, e), inter, k, 1, ACTIVATIONS[activation], _dt(x.dtype), _stream(stream)))


def expert_down(out, act, w_down, tiles, meta, offsets, stream=None) -> None:
    """out [T * top, H] float32, row r = W_down[e] act[r] over the sorted rows; ``w_down`` [E, H, I]."""
    slots, hidden = out.shape
    e, h, inter = w_down.shape
    _f32(out)
    assert h == hidden and act.shape == (slots, inter) and act.is_contiguous() and w_down.is_contiguous() and act.dtype == w_down.dtype
    native.experts_check(native.experts().ms_expert_gemm(
        _ptr(out), _ptr(act), inter, None, 1, _ptr(w_down), _ptr(tiles), _ptr(meta), _ptr(offsets),
        expert_max_tiles(slots, e), hidden, inter, 0, 0, _dt(act.dtype), _stream(stream)))


def expert_combine(out, y, x, idx, wgt, pos, experts: int, stream=None, shared=None, shared_gate=None) -> None:
    """out[t] = sum over the token's choices, in their order, of wgt * (y[pos] for an expert with tensors, x[t] for a
    router output from ``experts`` on: an identity expert); float32 sum, one rounding. ``shared`` [T, H] (the run's
    dtype): the output of an expert that every token uses, added times ``shared_gate`` [T] float32 (or once)."""
    t, hidden = out.shape
    top = idx.shape[1]
    _f32(y, wgt)
    assert out.is_contiguous() and x.shape == (t, hidden) and x.dtype == out.dtype and y.shape[1] == hidden
    assert shared is None or (shared.shape == (t, hidden) and shared.dtype == out.dtype and shared.is_contiguous())
    _f32(shared_gate)
    native.experts_check(native.experts().ms_expert_combine(
        _ptr(out), _ptr(y), _ptr(x), _rows(x), _ptr(idx), _ptr(wgt), _ptr(pos), t, hidden, top, experts, _dt(out.dtype),
        _stream(stream), _ptr(shared), _ptr(shared_gate)))
