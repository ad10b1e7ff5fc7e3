"""Rofozen without a GPU: configuration -> parts and run order, declared tensors against a statement of the
checkpoint format, cache needs, refused configurations, and the oracle's functions against other statements
of the same formulas."""

import math

import pytest
import torch

from miniserve_b200.config.registry import resolve
from miniserve_b200.parts import FixedState, PagedKV
from miniserve_b200.parts.decoder import DecoderModel
from tests import rofozen_util as rx
from tests.plain import rofozen_plain as plain


# --------------------------------------------------------------------------- configuration
@pytest.mark.parametrize("make", [rx.config_a, rx.config_b, rx.config_c])
def test_declared_tensors_are_the_checkpoint_format(make):
    raw = make()
    _, cfg, spec = resolve(raw)
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    decls = {k: tuple(v.shape) for k, v in model.weight_decls().items()}
    assert decls == rx.tensor_shapes(raw)
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]


def test_borrowed_tensors_become_a_run_order_with_caches_of_their_own():
    _, _, spec = resolve(rx.config_a())
    assert [e.layer for e in spec.run_order] == [0, 1, 2, 1] and len(spec.layers) == 3
    model = DecoderModel(spec, torch.float32, "cpu")
    assert [c.owner for c in model.entry_caches] == [0, 1, 2, 3]
    _, _, spec_c = resolve(rx.config_c())  # a chain: layer 2 borrows from layer 1, which borrows from layer 0
    assert [e.layer for e in spec_c.run_order] == [0, 0, 0, 1, 2]


def test_cache_needs_follow_the_mixers():
    _, _, spec = resolve(rx.config_a())
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    needs = [c.need for c in model.entry_caches]
    # a state [heads, vdim, state] in 32-bit and the convolution's last taps - 1 inputs over x | B | C
    assert needs[0] == (FixedState((4, 16, 8), torch.float32), FixedState((2, 4 * 16 + 2 * 2 * 8), torch.bfloat16))
    # the latent (24) and the rotated key part (8) in one entry of 32 numbers, one pool, bounded by the window
    assert needs[1] == PagedKV(1, 32, 20, values=False) == needs[3]
    _, _, spec_c = resolve(rx.config_c())
    last = DecoderModel(spec_c, torch.bfloat16, "cpu").entry_caches[4].need
    assert last == FixedState((4, 64, 16), torch.float32)  # one tap: nothing of the convolution is state


@pytest.mark.parametrize("change, error", [
    (lambda r: r["layers"][0].update(type="attention"), NotImplementedError),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), NotImplementedError),
    (lambda r: r["layers"][0]["mixer"].update(groups=3), ValueError),
    (lambda r: r["layers"][0]["mixer"].update(norm_groups=5), ValueError),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=6), ValueError),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(size=0), ValueError),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), ValueError),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=3), ValueError),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=5), ValueError),  # one group of four cannot give five
    (lambda r: r["layers"][3].update(weights_of=0), ValueError),  # a latent layer with a state-space layer's tensors
    (lambda r: r["layers"][3].update(weights_of=3), ValueError),
    (lambda r: r.pop("norm"), KeyError),
])
def test_refused_configurations(change, error):
    raw = rx.config_a()
    change(raw)
    with pytest.raises(error):
        resolve(raw)


# --------------------------------------------------------------------------- the oracle against other statements
def test_state_space_recurrence_equals_its_quadratic_form():
    """y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (C_t . B_s) x_s + D x_t, head by head."""
    torch.manual_seed(0)
    m = dict(heads=4, vdim=6, state=5, groups=2, conv=3, norm_groups=2)
    width, t = 20, 11
    inner, gn = 24, 10
    w = {"in": torch.randn(2 * inner + 2 * gn + 4, width) * 0.3, "conv": torch.randn(inner + 2 * gn, 3) * 0.5,
         "conv.b": torch.randn(inner + 2 * gn) * 0.1, "dt_bias": torch.randn(4), "A_log": torch.randn(4) * 0.5, "D": torch.randn(4),
         "norm": 1 + 0.1 * torch.randn(inner), "o": torch.eye(inner)}
    h = torch.randn(t, width)
    got = plain.mamba2(h, w, "", m, 1e-5, torch.float32)
    proj = (h.double() @ w["in"].double().T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:inner + inner + 2 * gn], proj[:, -4:]
    pad = torch.cat((torch.zeros(2, xbc.shape[1], dtype=torch.float64), xbc))
    conv = sum(pad[j:j + t] * w["conv"].double()[:, j] for j in range(3)) + w["conv.b"].double()
    xbc = conv * torch.sigmoid(conv)
    x, b, c = xbc[:, :inner].view(t, 4, 6), xbc[:, inner:inner + gn].view(t, 2, 5), xbc[:, inner + gn:].view(t, 2, 5)
    dt = torch.log1p(torch.exp(dt + w["dt_bias"].double()))
    la = -torch.exp(w["A_log"].double()) * dt  # log of the decay
    y = torch.zeros(t, 4, 6, dtype=torch.float64)
    for hd in range(4):
        g = hd // 2
        cum = torch.cumsum(la[:, hd], 0)
        for i in range(t):
            for s in range(i + 1):
                y[i, hd] += math.exp(cum[i] - cum[s]) * dt[s, hd] * (c[i, g] @ b[s, g]) * x[s, hd]
            y[i, hd] += w["D"].double()[hd] * x[i, hd]
    y = y.reshape(t, inner) * (z * torch.sigmoid(z))
    y = y.view(t, 2, inner // 2)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-5)).reshape(t, inner) * w["norm"].double()
    assert (got.double() - y).abs().max() < 1e-4
    assert (plain.mamba2_fast(h, w, "", m, 1e-5, torch.float32) - got).abs().max() < 1e-5


def test_rescaled_frequencies():
    f, mag = plain.yarn_frequencies(16, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5})
    base = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f[0] == pytest.approx(base[0].item())  # the fastest pair keeps its frequency
    assert f[-1] == pytest.approx(base[-1].item() / 4.0)  # the slowest is divided by the factor
    assert all(base[i] / 4.0 - 1e-12 <= f[i] <= base[i] + 1e-12 for i in range(8))
    g, one = plain.yarn_frequencies(16, 10000.0, None)
    assert one == 1.0 and (torch.as_tensor(g) == base).all()


def test_the_sink_is_a_key_without_a_value_and_the_window_counts_the_token_itself():
    torch.manual_seed(1)
    m = dict(heads=2, dim=4, rot_dim=2, vdim=3, kv_rank=5, q_rank=4, scale=0.7, rot={"base": 10.0, "dims": 2}, mask={"size": 3})
    width, t = 8, 7
    w = {"dq": torch.randn(4, width), "dq.norm": torch.ones(4), "uq": torch.randn(12, 4), "dkv": torch.randn(7, width),
         "dkv.norm": torch.ones(5), "uk": torch.randn(8, 5), "uv": torch.randn(6, 5), "sink": torch.tensor([0.5, -1.0]), "o": torch.eye(6)}
    h = torch.randn(t, width)
    got = plain.latent_attention(h, w, "", m, 1e-5, torch.float32).view(t, 2, 3)
    cq = plain.rms_norm(h @ w["dq"].T, w["dq.norm"], 1e-5)
    q = (cq @ w["uq"].T).view(t, 2, 6)
    kv = h @ w["dkv"].T
    c = plain.rms_norm(kv[:, :5], w["dkv.norm"], 1e-5)
    pos = torch.arange(t)
    kr = plain.rotate(kv[:, 5:], pos, 2, 10.0, None)
    qr = plain.rotate(q[..., 4:], pos, 2, 10.0, None)
    k, v = (c @ w["uk"].T).view(t, 2, 4), (c @ w["uv"].T).view(t, 2, 3)
    for i in range(t):
        for hd in range(2):
            js = [j for j in range(t) if 0 <= i - j < 3]  # itself and the two before it
            sc = torch.stack([(q[i, hd, :4] @ k[j, hd] + qr[i, hd] @ kr[j]) * 0.7 for j in js])
            e = torch.exp(sc)
            out = sum(e[n] * v[j, hd] for n, j in enumerate(js)) / (e.sum() + math.exp(w["sink"][hd]))
            assert (got[i, hd] - out).abs().max() < 1e-5


def test_the_router_chooses_within_the_best_groups_and_weighs_without_the_correction():
    torch.manual_seed(2)
    width, t = 10, 40
    router = {"experts": 7, "identity": 2, "scale": 0.7, "top": 4, "groups": {"count": 3, "keep": 2}}
    w = {"router": torch.randn(9, width), "correction": torch.randn(9) * 0.3}
    h = torch.randn(t, width)
    chosen, weights = plain.route(h, w, "", router, torch.float32)
    s = torch.softmax(h @ w["router"].T, -1)
    c = s + w["correction"]
    for i in range(t):
        groups = sorted(range(3), key=lambda g: -max(c[i, 3 * g:3 * g + 3]))[:2]
        allowed = [e for e in range(9) if e // 3 in groups]
        best = sorted(allowed, key=lambda e: -c[i, e])[:4]
        assert sorted(chosen[i].tolist()) == sorted(best)
        for e, g in zip(chosen[i].tolist(), weights[i].tolist()):
            assert g == pytest.approx(0.7 * s[i, e].item(), rel=1e-5)


def test_an_identity_expert_hands_the_input_on():
    torch.manual_seed(3)
    width = 6
    mlp = {"expert": {"ff": 4}, "kind": "moe", "router": {"experts": 1, "identity": 1, "scale": 2.0, "top": 1}}
    w = {"router": torch.tensor([[0.0] * width, [0.0] * width]), "correction": torch.tensor([-1.0, 1.0]),  # the correction decides
         "e0.gate": torch.randn(4, width), "e0.up": torch.randn(4, width), "e0.down": torch.randn(width, 4)}
    h = torch.randn(3, width)
    assert (plain.moe_ff(h, w, "", mlp, torch.float32) - 2.0 * 0.5 * h).abs().max() < 1e-6  # s = 1/2 for both, times the scale
