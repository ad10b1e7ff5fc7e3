"""Kovusun on the GPU against the plain implementation: each mechanism alone, whole prompts against
token-by-token decoding and portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots that are given back and used again, keys far away, at page borders and
just inside and just outside the window and the kept first keys (in prompts and in decoding), the first
tokens of a sequence, long decoding, sizes that are no round numbers, the trace runner and greedy
generation through the entry point."""

import random

import pytest
import torch

from miniserve_b200.cache.manager import KVEntryView, StateEntryView
from miniserve_b200.config import KovusunConfig, PartSpec
from miniserve_b200.parts import BuildEnv, build_part
from tests import kovusun_util as kx
from tests.kernel_util import PagedBatch, make_context
from tests.plain import kovusun_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
F32 = 1e-4  # logits in 32-bit: distance over their spread; the oracle sums its products in 64-bit, the engine in 32-bit
DTYPES = [torch.float32, torch.bfloat16]
HIDDEN = 48
EPS = 1e-5


def _ids(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def _close(got, want, dtype, scale=1.0):
    got, want = got.double().cpu(), want.double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs()
    allowed = tol * scale * max(1.0, want.abs().max().item())
    bad = (err.reshape(err.shape[0], -1).amax(dim=1) > allowed).nonzero().flatten().tolist()
    assert not bad, f"off by {err.max().item():.3e} (values up to {want.abs().max().item():.2f}); tokens {bad[:8]}"


def _bind(part, dtype, seed=0, std=0.3, change=None):
    """Random bfloat16-exact weights bound to the part; returns them as float32 on the CPU by name."""
    gen = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, decl in part.all_weights().items():
        t = torch.randn(decl.shape, generator=gen) * std
        if decl.init == "ones_normal":
            t = 1.0 + t / 2
        tensors[name] = t.to(torch.bfloat16).float()
    if change:
        change(tensors)
    tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    part.bind_all({k: v.to(device=DEV, dtype=torch.float32 if part.all_weights()[k].precision == "float32" else dtype)
                   for k, v in tensors.items()})
    return tensors


@pytest.fixture(autouse=True)
def _seeded():
    torch.manual_seed(1357)
    torch.cuda.manual_seed(1357)


def _ctx(rows, page=8, kv_heads=1, d=16, dtype=torch.float32, slots=None, share=None, seed=0):
    pb = PagedBatch(rows, page, kv_heads, d, dtype, seed=seed, share=share)
    ctx = make_context(pb)
    ctx.state_slot = torch.tensor(slots if slots is not None else list(range(len(rows))), dtype=torch.int32, device=DEV)
    return pb, ctx


def _x(n, dtype, std=1.0, width=HIDDEN):
    return (torch.randn(n, width, device=DEV) * std).to(dtype)


def _cpu(x):
    return x.float().cpu()


# --------------------------------------------------------------------------- layer norm, token shift
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 36, 250, 1024])
def test_layer_norm_alone_in_pairs_and_with_the_add(dtype, width):
    env = BuildEnv(dtype, DEV)
    a = build_part("norm", PartSpec("layernorm", dict(size=width, eps=EPS, names=dict(weight="", bias=".b"))), env)
    b = build_part("norm", PartSpec("layernorm", dict(size=width, eps=EPS, names=dict(weight="", bias=".b"))), env)
    wa, wb = _bind(a, dtype, 1), _bind(b, dtype, 2)
    _, ctx = _ctx([(0, 9)], dtype=dtype)
    res = torch.randn(9, width, device=DEV) * 3 + 1.5  # a mean far from zero: the variance is about the mean, not about zero
    delta = _x(9, dtype, 1.0, width)
    want = res.cpu() + _cpu(delta)
    total = res.clone()
    _close(a.forward(total, delta, ctx), plain.layer_norm(want, wa[""], wa[".b"], EPS), dtype)
    _close(total, want, torch.float32)
    total = res.clone()
    ya, yb = a.forward_pair(b, total, delta, ctx)
    _close(ya, plain.layer_norm(want, wa[""], wa[".b"], EPS), dtype)
    _close(yb, plain.layer_norm(want, wb[""], wb[".b"], EPS), dtype)
    _close(total, want, torch.float32)
    rows = torch.tensor([7, 2], dtype=torch.int32, device=DEV)
    got = a.forward(res.clone(), delta, ctx, rows=rows, num_rows=2, write_residual=False)
    _close(got[:2], plain.layer_norm(want[[7, 2]], wa[""], wa[".b"], EPS), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 37])
def test_token_shift_whole_in_portions_decoded_and_over_used_slots(dtype, width):
    from miniserve_b200.parts.block import TokenShift

    part = TokenShift(PartSpec("token_shift", dict(size=width, name="shift")), BuildEnv(dtype, DEV))
    w = _bind(part, dtype, change=lambda t: t["shift"].copy_(torch.rand(width)))
    n = 23
    h = _x(n, dtype, 1.0, width)
    want = plain.token_shift(_cpu(h), w["shift"])
    # slots hold NaN, as one that another request left would hold anything: a sequence's first token reads zeros
    view = StateEntryView(torch.full((5, width), float("nan"), dtype=dtype, device=DEV), (width,))
    _, ctx = _ctx([(0, n)], dtype=dtype, slots=[2])
    _close(part.forward(h, ctx, view), want, dtype)
    assert torch.equal(view.state[2], h[n - 1]) and view.state[1].isnan().all()
    for cuts in ([5, 2, 1, 1, 7, 2, 2, 3], [1] * n, [2] * 12):
        outs, at = [], 0
        for size in cuts:
            size = min(size, n - at)
            if size <= 0:
                break
            _, ctx = _ctx([(at, size)], dtype=dtype, slots=[4])
            outs.append(part.forward(h[at:at + size].contiguous(), ctx, view).clone())
            at += size
        _close(torch.cat(outs), want, dtype)
    # two unequal rows in one step: one continues from its slot, the other starts a sequence in a used slot
    _, ctx = _ctx([(0, 6)], dtype=dtype, slots=[0])
    part.forward(h[:6].contiguous(), ctx, view)
    _, ctx = _ctx([(6, 1), (0, 9)], dtype=dtype, slots=[0, 4])
    both = part.forward(torch.cat((h[6:7], h[:9])).contiguous(), ctx, view)
    _close(both[:1], want[6:7], dtype)
    _close(both[1:], want[:9], dtype)


# --------------------------------------------------------------------------- the three attention mixers
def _layer(kind, **kw):
    return dict(attention=kx.biased_layer, attention_2=kx.sink_layer, attention_3=kx.rotary_layer)[kind](**kw)


def _mixer(dtype, kind, **kw):
    from miniserve_b200.models.kovusun import _mixer as spec_of

    cfg = KovusunConfig.from_dict(kx.config([_layer(kind, **kw)], width=HIDDEN))
    return build_part("mixer", spec_of(cfg, 0, cfg.layers[0]), BuildEnv(dtype, DEV)), cfg.layers[0].mixer


def _tune(t):
    """Numbers that random tensors would leave mild: distance numbers that keep the logarithm's argument positive,
    temperatures away from one, sinks that take a visible share."""
    if "r2" in t:
        t["r2"].copy_(0.05 + torch.rand_like(t["r2"]) * 1.5)
        t["r1"].mul_(3.0)
    if "temp" in t:
        t["temp"].copy_(0.5 + torch.rand_like(t["temp"]) * 1.5)
    if "sink" in t:
        t["sink"].mul_(6.0)


def _ref(x, w, m, kind, start=0):
    pos = torch.arange(x.shape[0])
    return plain.attention_mixer(w, "", m, kind, _cpu(x), pos, EPS, torch.float32)[0]


def _portions(part, view, x, cuts, page, dtype, full):
    outs, at = [], 0
    for size in cuts:
        size = min(size, x.shape[0] - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], page, part.kv_heads, part.cache_dim, dtype, share=full)
        outs.append(part.forward(x[at:at + size].contiguous(), ctx, view).clone())
        at += size
    return torch.cat(outs)


MIXER_CASES = [
    ("attention", dict(heads=4, kv_heads=2, dim=16, vdim=16, window=20, scale=0.3), 16),
    ("attention", dict(heads=6, kv_heads=3, dim=12, vdim=12, window=5, scale=0.5), 8),
    ("attention", dict(heads=2, kv_heads=2, dim=64, vdim=64, window=33, scale=0.125), 16),
    ("attention_2", dict(heads=4, kv_heads=2, dim=16, vdim=24, window=12, scale=0.3), 8),
    ("attention_2", dict(heads=3, kv_heads=3, dim=20, vdim=12, window=1, scale=0.25), 4),
    ("attention_2", dict(heads=4, kv_heads=1, dim=64, vdim=40, window=44, scale=0.11), 16),
    ("attention_3", dict(heads=4, kv_heads=1, dim=24, vdim=16, window=9, keep_first=3, rot=8, scale=0.2), 8),
    ("attention_3", dict(heads=5, kv_heads=1, dim=12, vdim=20, window=5, keep_first=0, rot=12, base=37.0, scale=0.4), 8),
    ("attention_3", dict(heads=2, kv_heads=2, dim=16, vdim=16, window=7, keep_first=19, rot=4, base=1000.0, scale=0.3), 16),
    ("attention_3", dict(heads=2, kv_heads=1, dim=128, vdim=128, window=24, keep_first=16, rot=64, scale=0.09), 16),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind, sizes, page", MIXER_CASES)
def test_attention_mixers_whole_in_portions_and_decoded(dtype, kind, sizes, page):
    att, m = _mixer(dtype, kind, **sizes)
    w = _bind(att, dtype, change=_tune)
    n = 61
    x = _x(n, dtype, 2.0)
    ref = _ref(x, w, m, kind)
    pb, ctx = _ctx([(0, n)], page, att.kv_heads, att.cache_dim, dtype, seed=1)
    view = KVEntryView(0, pb.k_pool, pb.v_pool, page)
    out = att.forward(x, ctx, view)
    assert pb.status.item() == 0
    _close(out, ref, dtype, 3.0)
    # what the cache holds: keys after their norm or rotation, values as projected, zeros beyond their sizes
    k, v = plain.keys_values(w, "", m, kind, _cpu(x), torch.arange(n), EPS, torch.float32)
    _close(pb.read(0, pb.k_pool, n)[..., :m["dim"]], k, dtype, 2.0)
    _close(pb.read(0, pb.v_pool, n)[..., :m["vdim"]], v, dtype, 2.0)
    assert (pb.read(0, pb.k_pool, n)[..., m["dim"]:] == 0).all() and (pb.read(0, pb.v_pool, n)[..., m["vdim"]:] == 0).all()
    full, _ = _ctx([(0, n)], page, att.kv_heads, att.cache_dim, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.v_pool, page)
    _close(_portions(att, view, x, (page + 3, 2, 13, 2) + (1,) * n, page, dtype, full), ref, dtype, 3.0)
    # two unequal requests in one step (the second decodes a token behind what an earlier step left)
    swapped, _ = _ctx([(0, n), (0, 30)], page, att.kv_heads, att.cache_dim, dtype, seed=8)
    view = KVEntryView(0, swapped.k_pool, swapped.v_pool, page)
    _, warm = _ctx([(0, n - 1)], page, att.kv_heads, att.cache_dim, dtype, share=swapped)
    att.forward(x[:n - 1].contiguous(), warm, view)
    _, ctx = _ctx([(n - 1, 1), (0, 30)], page, att.kv_heads, att.cache_dim, dtype, share=swapped)
    both = att.forward(torch.cat((x[n - 1:], x[:30])).contiguous(), ctx, view)
    _close(both[:1], ref[n - 1:], dtype, 3.0)
    _close(both[1:], ref[:30], dtype, 3.0)


def _needle_for(att):
    """Every head's query matrix is minus the key matrix of its key/value head, and nothing else decides a score
    (no biases, no distance bias, one temperature, a gate half open): a query scores far below everything against its
    own token's key and far above everything against the key of a token whose input is minus its own."""
    def change(t):
        for name in ("q.b", "k.b", "v.b", "r1"):
            if name in t:
                t[name].zero_()
        if "temp" in t:
            t["temp"].fill_(1.0)
        if "sink" in t:
            t["sink"].fill_(-2.0)
        if "g" in t:
            t["g"].zero_()
        d, rep = att.head_dim, att.heads // att.kv_heads
        k = t["k"].view(att.kv_heads, d, -1)
        t["q"].copy_((-k).repeat_interleave(rep, dim=0).reshape(att.heads * d, -1))
    return change


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind, window, keep, n, page, dim", [case if len(case) == 6 else case + (32,) for case in [
    ("attention", 16, 0, 41, 8), ("attention", 20, 0, 75, 16), ("attention_2", 5, 0, 30, 8), ("attention_2", 64, 0, 200, 16),
    ("attention_2", 1, 0, 9, 4), ("attention", 512, 0, 700, 16), ("attention_3", 16, 4, 60, 8), ("attention_3", 20, 17, 90, 16),
    ("attention_3", 33, 1, 300, 16), ("attention_3", 1024, 3, 1900, 16), ("attention_3", 7, 0, 40, 8),
    # heads of 128: bfloat16 prompts run on the tcgen05 kernel (kept keys in a tile of their own, in the window's first
    # tile, and none), decoded tokens on the split-key kernel
    ("attention_3", 200, 5, 700, 16, 128), ("attention_3", 100, 130, 600, 16, 128), ("attention_3", 300, 2, 350, 32, 128),
    ("attention", 300, 0, 700, 16, 128), ("attention_2", 129, 0, 400, 16, 128)]])
def test_a_key_just_inside_and_just_outside_the_window_and_the_kept_keys(dtype, kind, window, keep, n, page, dim):
    """The last query and one earlier token are made so that this pair scores far above everything else. With the
    earlier token window - 1 places back its value must come back; one place further it must not, unless it is one of
    the kept first keys (the last kept one shows, the one behind it does not): in a prompt, for a token decoded alone
    and in a short portion. A window of one sees only the token itself."""
    sizes = dict(heads=4, kv_heads=2, dim=dim, vdim=dim, window=window, scale=0.5 if dim == 32 else 0.05)
    if kind == "attention_3":
        sizes.update(keep_first=keep, rot=4, base=10000.0)  # (a slow rotation of few channels: the needle survives the distance)
    att, m = _mixer(dtype, kind, **sizes)
    w = _bind(att, dtype, change=_needle_for(att))
    last = n - 1
    direction = _x(1, dtype, 3.0)[0]
    for needle in sorted({last - window + 1, last - window, last - window + 2, 0, keep - 1, keep}):
        if not 0 <= needle < last:
            continue
        x = _x(n, dtype, 0.1)
        x[last], x[needle] = direction, -direction
        ref = _ref(x, w, m, kind)
        blank = x.clone()
        blank[needle] = _x(1, dtype, 0.1)[0]
        shows = (ref[last] - _ref(blank, w, m, kind)[last]).abs().max().item()
        assert (shows > 0.05) == (last - needle < window or needle < keep), "the test's needle shows exactly when the mask lets it"
        full, _ = _ctx([(0, n)], page, att.kv_heads, att.cache_dim, dtype, seed=3)
        view = KVEntryView(0, full.k_pool, full.v_pool, page)
        _, ctx = _ctx([(0, n)], page, att.kv_heads, att.cache_dim, dtype, share=full)
        _close(att.forward(x, ctx, view), ref, dtype, 3.0)  # in a prompt
        _, ctx = _ctx([(last, 1)], page, att.kv_heads, att.cache_dim, dtype, share=full)
        _close(att.forward(x[last:].contiguous(), ctx, view), ref[last:], dtype, 3.0)  # decoded alone over the same pages
        if n > 3:
            _, ctx = _ctx([(n - 3, 3)], page, att.kv_heads, att.cache_dim, dtype, share=full)
            _close(att.forward(x[n - 3:].contiguous(), ctx, view), ref[n - 3:], dtype, 3.0)  # a short portion


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, n, window", [(16, 37, 40), (128, 300, 400), (128, 420, 150)])
def test_distance_bias_prefers_near_keys_by_head(dtype, dim, n, window):
    """All keys equal: the scores differ by the distance bias alone. A head with r1 > 0 weighs near keys more, one with
    r1 < 0 far keys, one with r1 = 0 all alike; the engine agrees with the plain form in a prompt and in decoding."""
    att, m = _mixer(dtype, "attention", heads=3, kv_heads=1, dim=dim, vdim=16, window=window, scale=0.3)

    def change(t):
        t["r1"].copy_(torch.tensor([6.0, -6.0, 0.0]))
        t["r2"].copy_(torch.tensor([0.5, 2.0, 1.0]))
        t["k"].zero_()  # the keys are their biases: the same at every position
    w = _bind(att, dtype, change=change)
    x = _x(n, dtype, 1.0)
    ref = _ref(x, w, m, "attention")
    full, ctx = _ctx([(0, n)], 16, 1, att.cache_dim, dtype, seed=4)
    view = KVEntryView(0, full.k_pool, full.v_pool, 16)
    _close(att.forward(x, ctx, view), ref, dtype, 3.0)
    _, ctx = _ctx([(n - 1, 1)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[n - 1:].contiguous(), ctx, view), ref[n - 1:], dtype, 3.0)
    _, ctx = _ctx([(n - 70, 70)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[n - 70:].contiguous(), ctx, view), ref[n - 70:], dtype, 3.0) if n > 70 else None
    first = max(0, n - window)  # the last query's first visible key
    v = (_cpu(x).double() @ w["v"].double().T + w["v.b"].double()).float()  # [n, 16]
    o = (ref[n - 1].double() @ torch.linalg.pinv(w["o"].double()).T).float().view(3, 16)
    assert (o[2] - v[first:].mean(0)).abs().max() < 1e-3, "without a bias every key weighs the same"
    assert (o[0] - v[n - 1]).norm() < 0.5 * (o[0] - v[first]).norm()
    third = (n - first) // 3
    assert (o[1] - v[first:first + third].mean(0)).norm() < (o[1] - v[n - third:].mean(0)).norm()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_reader_of_another_layers_keys_and_values(dtype):
    """The owner writes its keys and values; the reader brings queries, a longer window and distance numbers of its own."""
    raw = kx.config([kx.biased_layer(window=9), kx.biased_layer(window=26, kv_from=0)], width=HIDDEN)
    from miniserve_b200.models.kovusun import _mixer as spec_of

    cfg = KovusunConfig.from_dict(raw)
    env = BuildEnv(dtype, DEV)
    own, reader = (build_part("mixer", spec_of(cfg, i, cfg.layers[i]), env) for i in (0, 1))
    assert own.cache_need().window == 26 and reader.cache_need() is None and reader.reach == 26
    wo, wr = _bind(own, dtype, 1, change=_tune), _bind(reader, dtype, 2, change=_tune)
    n, page = 50, 8
    xo, xr = _x(n, dtype, 2.0), _x(n, dtype, 2.0)
    pos = torch.arange(n)
    ref_own, kv = plain.attention_mixer(wo, "", raw["layers"][0]["mixer"], "attention", _cpu(xo), pos, EPS, torch.float32)
    ref_reader, _ = plain.attention_mixer(wr, "", raw["layers"][1]["mixer"], "attention", _cpu(xr), pos, EPS, torch.float32, kv=kv)
    full, _ = _ctx([(0, n)], page, own.kv_heads, own.cache_dim, dtype, seed=5)
    view = KVEntryView(0, full.k_pool, full.v_pool, page)
    outs_o, outs_r, at = [], [], 0
    for size in (11, 2, 1, 20, 1, 1, 14):
        _, ctx = _ctx([(at, size)], page, own.kv_heads, own.cache_dim, dtype, share=full)
        outs_o.append(own.forward(xo[at:at + size].contiguous(), ctx, view).clone())
        outs_r.append(reader.forward(xr[at:at + size].contiguous(), ctx, view).clone())
        at += size
    _close(torch.cat(outs_o), ref_own, dtype, 3.0)
    _close(torch.cat(outs_r), ref_reader, dtype, 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_reader_of_a_layer_of_another_kind_and_a_zero_limit(dtype, tmp_path):
    """A layer with biases and a distance bias reads the keys and values of a layer with a sink and a gate (unit-normed
    keys without biases, as that layer's cache holds them); the checkpoint carries a second norm for a layer without a
    feed-forward; a dense feed-forward with a limit of zero (the gate never above zero, up always zero)."""
    raw = kx.config([kx.sink_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=12, mlp=kx.dense(40, limit=0.0)),
                     kx.biased_layer(heads=6, kv_heads=2, dim=16, vdim=16, window=20, kv_from=0)], width=40, vocab=53)

    def spare(w):
        w["l1.norm2"] = torch.ones(40, dtype=torch.bfloat16)
        w["l1.norm2.b"] = torch.zeros(40, dtype=torch.bfloat16)
    folder = kx.write_model(tmp_path / "m", raw, seed=31, change=spare)
    ids = _ids(70, 53, 6)
    run = kx.Runner(folder, dtype, max_tokens=128, page_size=8)
    model = dict(oracle=kx.oracle(folder), rounded=kx.oracle(folder, torch.bfloat16))
    _logits_close(model, dtype, run.feed("w", ids, [70]), ids, "whole")
    _logits_close(model, dtype, run.feed("c", ids, [9, 2, 30, 1, 1, 1, 5, 2]), ids, "in portions")
    assert run.cache.is_idle()


@pytest.mark.parametrize("seed", [5, 6, 7])
def test_pages_given_back_behind_a_window_are_not_weighed(seed, tmp_path):
    """Values of 128 channels under a window of 33: prompts' portions run on the tcgen05 kernel, whose first key tile
    reaches back over pages that the window has given back (NaN-filled here). A probability of zero times a NaN is a
    NaN, so those rows of V must not reach the product."""
    raw = kx.config([kx.biased_layer(heads=2, kv_heads=1, dim=32, vdim=128, window=33, mlp=kx.dense(48)),
                     kx.sink_layer(heads=2, kv_heads=2, dim=128, vdim=64, window=20, scale=0.09)], width=64, vocab=71)
    folder = kx.write_model(tmp_path / "m", raw, seed=seed)
    ids = _ids(230, 71, seed)
    run = kx.Runner(folder, "bfloat16", max_tokens=256, page_size=16)
    got = run.feed("c", ids, [64, 2, 37, 1, 1, 1, 50, 3, 1, 1, 40, 2])
    assert not torch.isnan(got).any(), f"NaN from position {int(torch.isnan(got).any(dim=1).nonzero()[0])} on"
    ok, report = kx.rounded_ok(got, kx.oracle(folder)(ids), kx.oracle(folder, torch.bfloat16)(ids))
    assert ok, report


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_takes_its_share_and_the_gate_closes_heads(dtype):
    att, m = _mixer(dtype, "attention_2", heads=2, kv_heads=1, dim=16, vdim=16, window=30, scale=0.3)

    def change(t):
        t["sink"].copy_(torch.tensor([25.0, -25.0]))  # head 0 is all sink, head 1 none of it
    w = _bind(att, dtype, change=change)
    n = 21
    x = _x(n, dtype, 1.0)
    ref = _ref(x, w, m, "attention_2")
    full, ctx = _ctx([(0, n)], 8, 1, att.cache_dim, dtype)
    view = KVEntryView(0, full.k_pool, full.v_pool, 8)
    feat = torch.zeros(n, att.feature_width, device=DEV, dtype=dtype)
    att.features(x, ctx, view, feat)
    assert _cpu(feat)[:, :16].abs().max() < 1e-3 and _cpu(feat)[:, 16:].abs().max() > 1e-2
    _, ctx = _ctx([(0, n)], 8, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x, ctx, view), ref, dtype, 3.0)


# --------------------------------------------------------------------------- feed-forwards
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, inter, limit", [(40, 72, 1.0), (36, 52, 0.5), (48, 80, 7.0)])
def test_clamped_gated_feed_forward_with_biases(dtype, hidden, inter, limit):
    from miniserve_b200.models.kovusun import _feed_forward as spec_of

    mlp = kx.dense(inter, limit)
    part = build_part("feed_forward", spec_of(hidden, mlp), BuildEnv(dtype, DEV))
    w = _bind(part, dtype, std=0.4)
    x = _x(19, dtype, 2.0, hidden)  # large enough that gate and up pass the limit on both sides
    _, ctx = _ctx([(0, 19)], dtype=dtype)
    ref = plain.dense_ff(w, "", mlp, _cpu(x), torch.float32)
    g = _cpu(x) @ w["gate"].T + w["gate.b"]
    u = _cpu(x) @ w["up"].T + w["up.b"]
    if limit <= 1.0:
        assert (g > limit).any() and (u > limit).any() and (u < -limit).any(), "the test's inputs reach the clamps"
    _close(part.forward(x, ctx), ref, dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, ff, experts, top, shared", [(48, 24, 6, 2, 40), (36, 20, 3, 1, 0), (64, 64, 8, 3, 96), (40, 12, 5, 5, 8),
                                                              (48, 16, 12, 3, 32)])
def test_router_experts_and_the_shared_expert(dtype, hidden, ff, experts, top, shared):
    from miniserve_b200.models.kovusun import _feed_forward as spec_of

    mlp = kx.moe(ff, experts, top, shared)
    part = build_part("feed_forward", spec_of(hidden, mlp), BuildEnv(dtype, DEV))

    def change(t):
        t["router"].mul_(4.0)
        t["router.b"].mul_(5.0)  # a bias that changes who is chosen

    w = _bind(part, dtype, std=0.3, change=change)
    for n in (33, 7, 1):  # (down to the few rows of a decode step)
        x = _x(n, dtype, 1.0, hidden)
        _, ctx = _ctx([(0, n)], dtype=dtype)
        idx, wgt = part.route(x, ctx)
        want_idx, want_wgt = plain.route(w, "", mlp, _cpu(x), torch.float32)
        no_bias = torch.topk(_cpu(x) @ w["router"].T, top, dim=-1).indices
        if top < experts and n == 33:
            assert (no_bias.sort(-1).values != want_idx.sort(-1).values).any(), "the test's bias changes a choice"
        assert torch.equal(idx.cpu().long(), want_idx)
        assert (wgt.cpu() - want_wgt).abs().max() < 1e-5 and (wgt.sum(-1) - 1).abs().max() < 1e-5
        _close(part.forward(x, ctx), plain.moe_ff(w, "", mlp, _cpu(x), torch.float32), dtype, 3.0)


# --------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=["a", "b", "c"])
def model(request, tmp_path_factory):
    raw = dict(a=kx.config_a, b=kx.config_b, c=kx.config_c)[request.param]()
    folder = kx.write_model(tmp_path_factory.mktemp("kovusun_" + request.param), raw, seed=dict(a=21, b=22, c=23)[request.param])
    return dict(folder=folder, raw=raw, oracle=kx.oracle(folder), rounded=kx.oracle(folder, torch.bfloat16),
                page=dict(a=16, b=8, c=32)[request.param])


def _logits_close(model, dtype, got, ids, what=""):
    """32-bit: within F32 of the oracle. bfloat16: as near as rounding allows, position by position."""
    want = model["oracle"](ids)
    if dtype == "float32":
        err = kx.rel_err(got, want)
        assert err < F32, f"{what}: {err:.2e}"
    else:
        ok, report = kx.rounded_ok(got, want, model["rounded"](ids))
        assert ok, f"{what}: {report}"


def test_layer_streams_in_float32(model):
    """The residual stream after every layer, against the oracle's."""
    from miniserve_b200.cache import CacheManager
    from miniserve_b200.engine.loader import load_model
    from miniserve_b200.engine.step import StepFunction, StepRow
    from miniserve_b200.parts import ResidualStream

    ids = _ids(29, model["raw"]["vocab"], 8)
    want = kx.layer_streams(model["folder"], ids)
    _, _, net = load_model(model["folder"], "float32", "cuda:0")
    cache = CacheManager(net.entry_caches, 8, 16, 2, dtype=net.dtype, device=net.device)
    ctx = StepFunction(net, cache).prepare([StepRow(cache.new_request(), ids, [0])])
    stream = ResidualStream(net.embedding.forward(ctx))
    for i, e in enumerate(net.spec.run_order):
        stream = net.layers[e.layer].forward(stream, ctx, cache.entry_views[i])
        x = stream.total.double().cpu()
        if stream.pending is not None:
            x = x + stream.pending_scale * stream.pending.double().cpu()
        assert (x - want[i].double()).abs().max() < 1e-4 * max(1.0, want[i].abs().max().item()), f"after layer {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(model, dtype):
    vocab = model["raw"]["vocab"]
    run = kx.Runner(model["folder"], dtype, max_tokens=256, page_size=model["page"])
    for n, seed in ((1, 1), (2, 2), (37, 3), (150, 4)):
        ids = _ids(n, vocab, seed)
        _logits_close(model, dtype, run.feed("w", ids, [n]), ids, f"{n} whole")
        if n > 2:
            # the last 110 one by one: every window passes over decoded tokens
            _logits_close(model, dtype, run.feed("d", ids, [n - min(n - 1, 110), 1]), ids, f"{n} decoded")
            _logits_close(model, dtype, run.feed("c", ids, [7, 2, 24, 3, model["page"], 2, 5, 31, 2, 1, 1, 2, 9]), ids, f"{n} in portions")
            _logits_close(model, dtype, run.feed("p", ids, [2]), ids, f"{n} two by two")
        assert run.cache.is_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, portions of some beside single tokens of others, a pool that holds only what is
    live and four state slots: every page and slot is used by several requests in turn (pages are filled with NaN
    when given back, and the layers with a window give pages back while a request runs)."""
    vocab = model["raw"]["vocab"]
    seqs = {f"r{i}": _ids(n, vocab, 20 + i) for i, n in enumerate([90, 5, 64, 33, 1, 120, 17, 48, 2, 75])}
    run = kx.Runner(model["folder"], dtype, max_tokens=4 * 128, page_size=model["page"], max_requests=4)
    rng = random.Random(5)
    waiting, live, at, got = list(seqs), [], {}, {k: [] for k in seqs}
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        entries, ended = [], []
        order = sorted(live, key=lambda r: at[r] == 0 or len(seqs[r]) - at[r] > 40)  # decoding rows first
        for rid in order:
            left = len(seqs[rid]) - at[rid]
            n = 1 if left <= 40 and at[rid] > 0 else min(left, rng.choice([2, 3, 16, 29, 50]))
            if rng.random() < 0.15 and len(order) > 1:
                continue  # left out of this step
            entries.append((rid, seqs[rid][at[rid]:at[rid] + n], "all"))
            at[rid] += n
            if at[rid] == len(seqs[rid]):
                ended.append(rid)
        if not entries:
            continue
        logits = run.step(entries, end=ended)
        i = 0
        for rid, toks, _ in entries:
            got[rid].append(logits[i:i + len(toks)])
            i += len(toks)
        live = [r for r in live if r not in ended]
    for rid in seqs:
        _logits_close(model, dtype, torch.cat(got[rid]), seqs[rid], rid)
    assert run.cache.is_idle()


def test_long_decoding_in_float32(model):
    ids = _ids(400, model["raw"]["vocab"], 9)
    run = kx.Runner(model["folder"], "float32", max_tokens=448, page_size=model["page"])
    assert kx.rel_err(run.feed("long", ids, [3, 1]), model["oracle"](ids)) < F32


def test_trace_runner_replays_a_schedule(model, tmp_path):
    from tests.trace_util import Trace, run_trace

    vocab = model["raw"]["vocab"]
    a, b = _ids(50, vocab, 31), _ids(21, vocab, 32)
    tr = Trace()
    tr.step([("a", a[:30], [0, 29])])
    tr.step([("a", a[30:31], [0]), ("b", b[:19], "last")])
    tr.step([("b", b[19:20], [0]), ("a", a[31:], "all")], end=["a"])
    tr.step([("b", b[20:], [0])], end=["b"])
    tr.step([("c", b, "last")], end=["c"])  # in the pages and the slot that were given back
    out = run_trace(model["folder"], "float32", tr, tmp_path / "out", page_size=model["page"], vocab=vocab)
    want = {"a": model["oracle"](a), "b": model["oracle"](b), "c": model["oracle"](b)}
    assert len(out) == 2 + 2 + 1 + 19 + 1 + 1
    for (rid, pos, _), logits in out.items():
        assert kx.rel_err(logits[None], want[rid][pos:pos + 1]) < F32, (rid, pos)


@pytest.mark.parametrize("dtype, cuda_graph", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_entry_point(model, dtype, cuda_graph):
    from miniserve_b200.engine import LLM, SamplingParams

    vocab = model["raw"]["vocab"]
    prompts = [_ids(n, vocab, 40 + n) for n in (5, 17, 33, 1, 9, 70)]
    llm = LLM(model["folder"], dtype=dtype, kv_pool_tokens=1024, page_size=model["page"], max_running=4,
              chunked_prefill_size=24, cuda_graph=cuda_graph)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=10))
    assert llm.engine.cache.is_idle()
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        every = model["oracle"](list(p) + list(o))  # causal: row i is what the oracle says after tokens 0..i
        moved = (model["rounded"](list(p) + list(o)) - every).abs().amax(dim=1) if dtype == "bfloat16" else None
        for i, t in enumerate(o):  # teacher-forced: each chosen token is the oracle's best, or within rounding of it
            at = len(p) + i - 1
            logits = every[at]
            slack = 1e-4 if dtype == "float32" else max(0.15, 3.0 * moved[at].item())
            assert (logits.max() - logits[t]).item() <= slack, (at + 1, t)
