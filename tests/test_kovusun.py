"""Kovusun without a GPU: configuration -> parts, run order and cache needs; declared tensors against a statement of
the checkpoint format; and the plain form's own properties (the oracle of the GPU tests must itself be right about
windows, kept keys, the sink, the shift and the router)."""

import math

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.cache.manager import group_needs
from miniserve_b200.config import KovusunConfig, resolve
from miniserve_b200.parts import DecoderModel, FixedState, PagedKV
from tests import kovusun_util as kx
from tests.plain import kovusun_plain as plain


@pytest.mark.parametrize("make", [kx.config_a, kx.config_b, kx.config_c])
def test_declared_tensors_are_the_checkpoint_format(make):
    raw = make()
    arch, cfg, spec = resolve(raw)
    assert arch.name == "Kovusun" and isinstance(cfg, KovusunConfig)
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    declared = {k: tuple(v.shape) for k, v in model.weight_decls().items()}
    assert declared == kx.tensor_shapes(raw)
    keep32 = {k for k, v in model.weight_decls().items() if v.precision == "float32"}
    for name in declared:  # norms, routers, sinks, temperatures, distance numbers, shift weights and biases stay 32-bit
        leaf = name.rsplit(".", 1)[-1]
        small = len(declared[name]) == 1 or leaf in ("router", "sg")
        assert (name in keep32) == small, name


def test_run_order_caches_and_shared_keys():
    raw = kx.config_a()
    _, cfg, spec = resolve(raw)
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    assert [e.cache_of for e in spec.run_order] == [None, None, 0, None]
    needs = [ec.need for ec in model.entry_caches]
    w = raw["width"]
    # every layer keeps its shift state; the reader of layer 0 has no pages of its own, and layer 0 keeps keys for the
    # longer of the two windows; kept first keys mean that no page is given back
    assert needs[0] == (FixedState((w,), torch.bfloat16), PagedKV(2, 16, 21))
    assert needs[1] == (FixedState((w,), torch.bfloat16), PagedKV(1, 32, None))
    assert needs[2] == (FixedState((w,), torch.bfloat16), None) and model.entry_caches[2].shares == 0
    assert needs[3] == (FixedState((w,), torch.bfloat16), PagedKV(2, 32, 12))
    groups, states = group_needs(model.entry_caches)
    assert len(groups) == 3 and len(states) == 4
    cache = CacheManager(model.entry_caches, 8, 16, 3, device=None)
    views = cache.entry_views
    assert views[2][1].group == views[0][1].group and views[2][0] is not views[0][0]
    assert model.layers[2].mixer.reach == 21 and model.layers[0].mixer.reach == 13


def test_a_reader_may_read_a_layer_of_another_kind_and_a_spare_norm_is_tolerated():
    raw = kx.config([kx.sink_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=12), kx.biased_layer(window=20, kv_from=0)])
    _, _, spec = resolve(raw)
    model = DecoderModel(spec, torch.float32, "cpu")
    assert model.entry_caches[1].shares == 0 and model.entry_caches[0].need[1] == PagedKV(2, 16, 20)
    assert set(spec.optional_tensors) == {"l0.norm2", "l0.norm2.b", "l1.norm2", "l1.norm2.b"}  # neither layer has a feed-forward


def test_a_reader_of_keys_with_kept_first_keys_keeps_every_page():
    own = kx.rotary_layer(window=9, keep_first=0)
    reader = kx.rotary_layer(window=30, keep_first=4)
    reader["mixer"]["kv_from"] = 0
    _, _, spec = resolve(kx.config([own, reader]))
    model = DecoderModel(spec, torch.float32, "cpu")
    assert model.entry_caches[0].need[1].window is None


@pytest.mark.parametrize("change, error", [
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=2), ValueError),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=1), ValueError),  # a layer of other key and value sizes
    (lambda raw: raw["layers"][2]["mixer"].update(dim=32), ValueError),  # other sizes than the owner's
    (lambda raw: raw["layers"][0].update(type="attention_9"), NotImplementedError),
    (lambda raw: raw["layers"][0]["mlp"].update(kind="sparse"), NotImplementedError),
    (lambda raw: raw["layers"][1]["mixer"]["mask"].update(size=0), ValueError),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=9), ValueError),
])
def test_bad_configurations_are_refused(change, error):
    raw = kx.config_a()
    change(raw)
    with pytest.raises(error):
        resolve(raw)


def test_plain_masks():
    m = plain.visible(12, 4)
    assert m[7].nonzero().flatten().tolist() == [4, 5, 6, 7] and m[0].nonzero().flatten().tolist() == [0]
    m = plain.visible(12, 3, 2)
    assert m[9].nonzero().flatten().tolist() == [0, 1, 7, 8, 9] and m[1].nonzero().flatten().tolist() == [0, 1]
    assert plain.visible(5, 1).sum() == 5


def test_plain_sink_shift_router_and_distance():
    torch.manual_seed(3)
    q, k, v = torch.randn(6, 2, 8), torch.randn(6, 1, 8), torch.randn(6, 1, 4)
    mask = plain.visible(6, 6)
    free = plain.attend(q, k, v, 0.5, mask)
    sunk = plain.attend(q, k, v, 0.5, mask, sink=torch.tensor([30.0, -30.0]))
    assert sunk[:, 0].abs().max() < 1e-6 and torch.allclose(sunk[:, 1], free[:, 1], atol=1e-6)
    # a distance bias with r2 = 0 is none; a large r1 leaves each query its own key alone
    same = plain.attend(q, k, v, 0.5, mask, dist=(torch.ones(2), torch.zeros(2)))
    assert torch.allclose(same, free, atol=1e-6)
    near = plain.attend(q, k, v, 0.5, mask, dist=(torch.full((2,), 200.0), torch.ones(2)))
    assert torch.allclose(near, v.repeat_interleave(2, dim=1), atol=1e-5)
    h = torch.randn(5, 3)
    mix = torch.tensor([0.0, 1.0, 0.25])
    out = plain.token_shift(h, mix)
    assert torch.equal(out[:, 0], h[:, 0]) and torch.allclose(out[1:, 1], h[:-1, 1], atol=1e-6) and out[0, 1].abs() < 1e-6
    assert torch.allclose(out[2, 2], 0.75 * h[2, 2] + 0.25 * h[1, 2])
    w = {"router": torch.eye(4), "router.b": torch.tensor([0.0, 0.0, 5.0, 0.0])}
    idx, wgt = plain.route(w, "", {"router": {"experts": 4, "top": 2}}, torch.tensor([[3.0, 1.0, -1.0, 0.0]]), torch.float32)
    assert idx.tolist() == [[2, 0]] and torch.allclose(wgt, torch.softmax(torch.tensor([[4.0, 3.0]]), -1))


def test_plain_rotation_turns_adjacent_pairs_by_their_own_frequencies():
    x = torch.zeros(3, 1, 6)
    x[:, 0, 0] = 1.0
    x[:, 0, 2] = 1.0
    x[:, 0, 5] = 7.0
    out = plain.rotate_pairs(x, torch.tensor([0, 1, 5]), 4, 100.0)
    assert torch.allclose(out[1, 0, :2], torch.tensor([math.cos(1.0), math.sin(1.0)]), atol=1e-6)
    assert torch.allclose(out[2, 0, 2:4], torch.tensor([math.cos(0.5), math.sin(0.5)]), atol=1e-6)  # 100^(-2/4) = 0.1
    assert torch.equal(out[:, 0, 4:], x[:, 0, 4:]) and torch.equal(out[0], x[0])


def test_plain_dense_feed_forward_clamps():
    w = {"gate": torch.eye(2) * 10, "gate.b": torch.zeros(2), "up": torch.eye(2) * 10, "up.b": torch.zeros(2), "down": torch.eye(2),
         "down.b": torch.tensor([0.5, 0.0])}
    y = plain.dense_ff(w, "", {"limit": 2.0}, torch.tensor([[1.0, -1.0]]), torch.float32)
    g = torch.tensor([2.0, -10.0])
    want = g * torch.sigmoid(1.702 * g) * (torch.tensor([2.0, -2.0]) + 1.0) + torch.tensor([0.5, 0.0])
    assert torch.allclose(y[0], want, atol=1e-6)
