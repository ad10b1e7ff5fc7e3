"""Rofozen on the GPU against the plain implementation: each mechanism alone, whole prompts against
token-by-token decoding and portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots that are given back and used again, keys far away, at page borders and
just inside and just outside the window (in prompts and in decoding), the first tokens of a sequence,
long decoding, sizes that are no round numbers, the trace runner and greedy generation through the
entry point."""

import random

import pytest
import torch

from miniserve_b200.cache.manager import KVEntryView, StateEntryView
from miniserve_b200.config import PartSpec
from miniserve_b200.parts import BuildEnv, ResidualStream, build_part
from tests import rofozen_util as rx
from tests.kernel_util import PagedBatch, make_context
from tests.plain import rofozen_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
F32 = 1e-4  # logits in 32-bit: distance over their spread (rel_err); the oracle sums its products in 64-bit, the engine in 32-bit, layer after layer
DTYPES = [torch.float32, torch.bfloat16]
HIDDEN = 48


def _ids(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def _close(got, want, dtype, scale=1.0, noise=None):
    """``noise`` [T]: what rounding alone costs the plain form at each token (its distance from itself computed one
    precision higher); a token may be four times that far on top of the tolerance."""
    got, want = got.double().cpu(), want.double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    err = (got - want).abs()
    allowed = torch.full((want.shape[0],), tol * scale * max(1.0, want.abs().max().item()), dtype=torch.float64)
    if noise is not None:
        allowed = allowed + 4.0 * noise.double()
    bad = (err.amax(dim=tuple(range(1, err.dim()))) > allowed).nonzero().flatten().tolist()
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
    torch.manual_seed(2468)
    torch.cuda.manual_seed(2468)


def _ctx(rows, page=8, kv_heads=1, d=16, dtype=torch.float32, slots=None, share=None, seed=0):
    pb = PagedBatch(rows, page, kv_heads, d, dtype, seed=seed, share=share)
    ctx = make_context(pb)
    ctx.state_slot = torch.tensor(slots if slots is not None else list(range(len(rows))), dtype=torch.int32, device=DEV)
    return pb, ctx


def _x(n, dtype, std=1.0):
    return (torch.randn(n, HIDDEN, device=DEV) * std).to(dtype)


def _cpu(x):
    return x.float().cpu()


# --------------------------------------------------------------------------- the state-space mixer
def _ssm(dtype, heads, vdim, state, groups, conv, norm_groups):
    from miniserve_b200.models.rofozen import _mamba2 as spec_of

    m = rx.ssm_layer(heads, vdim, state, groups, conv, norm_groups)["mixer"]
    return build_part("mixer", spec_of(HIDDEN, 1e-5, m), BuildEnv(dtype, DEV)), m


def _ssm_weights(t):
    t["A_log"].copy_(torch.linspace(-2.0, 0.5, t["A_log"].numel()))  # decays from slow to fast
    t["dt_bias"].sub_(0.5)


def _state_views(part):
    need = part.cache_need()
    needs = need if isinstance(need, tuple) else (need,)
    views = tuple(StateEntryView(torch.full((5, *nd.shape), float("nan"), dtype=nd.dtype, device=DEV), tuple(nd.shape)) for nd in needs)
    return views if isinstance(need, tuple) else views[0]


def _state_portions(part, views, x, cuts, slot, dtype):
    outs, at = [], 0
    for size in cuts:
        size = min(size, x.shape[0] - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], dtype=dtype, slots=[slot])
        outs.append(part.forward(x[at:at + size].contiguous(), ctx, views).clone())
        at += size
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, vdim, state, groups, conv, norm_groups", [
    (4, 16, 8, 2, 3, 2), (5, 12, 12, 1, 2, 5), (6, 8, 20, 3, 4, 3), (2, 64, 16, 2, 1, 1), (8, 32, 64, 8, 4, 4), (1, 40, 128, 1, 5, 2)])
def test_state_space_mixer_whole_in_portions_and_decoded(dtype, heads, vdim, state, groups, conv, norm_groups):
    part, m = _ssm(dtype, heads, vdim, state, groups, conv, norm_groups)
    w = _bind(part, dtype, change=_ssm_weights)
    n = 70
    x = _x(n, dtype)
    ref = plain.mamba2(_cpu(x), w, "", m, 1e-5, torch.float32)
    views = _state_views(part)
    _close(_state_portions(part, views, x, (n,), 1, dtype), ref, dtype, 3.0)
    # the same slot again (the state of the request before is still there); portions shorter than the convolution's
    # history, single tokens from the very first one, then portions down to two tokens, then token by token
    _close(_state_portions(part, views, x, (1, 1, 2, 1, 3, 2, 17, 2, 9) + (1,) * n, 1, dtype), ref, dtype, 3.0)
    # two requests of unequal length in one step, in other slots; then both go on, one decoding beside a portion
    _, ctx = _ctx([(0, 21), (0, n - 9)], dtype=dtype, slots=[4, 0])
    both = part.forward(torch.cat((x[:21], x[:n - 9])), ctx, views)
    _close(both[:21], ref[:21], dtype, 3.0)
    _close(both[21:], ref[:n - 9], dtype, 3.0)
    _, ctx = _ctx([(n - 9, 1), (21, 30)], dtype=dtype, slots=[0, 4])
    both = part.forward(torch.cat((x[n - 9:n - 8], x[21:51])), ctx, views)
    _close(both[:1], ref[n - 9:n - 8], dtype, 3.0)
    _close(both[1:], ref[21:51], dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, vdim, state, groups", [(2, 24, 16, 1), (4, 64, 64, 2)])
def test_state_space_mixer_over_a_long_portion_and_long_decoding(dtype, heads, vdim, state, groups):
    """A portion of 700 tokens (the scan may walk it in segments), behind an earlier portion, beside a short row,
    and 300 tokens decoded one by one from the state it left: the state keeps what it should for hundreds of steps."""
    part, m = _ssm(dtype, heads, vdim, state, groups, 4, 2)
    w = _bind(part, dtype, change=_ssm_weights)
    n = 1000
    x = _x(n, dtype)
    # Among a thousand tokens a few have a part of y with a tiny root mean square, where the norm amplifies rounding:
    # the truth is the plain form one precision higher, and the plain form at the run's precision says how far
    # rounding alone gets there.
    if dtype == torch.float32:
        ref = plain.mamba2_fast(_cpu(x), w, "", m, 1e-5, torch.float32, acc=torch.float64)
        noise = (plain.mamba2_fast(_cpu(x), w, "", m, 1e-5, torch.float32).double() - ref).abs().amax(dim=1)
    else:
        ref = plain.mamba2_fast(_cpu(x), w, "", m, 1e-5, torch.float32)
        noise = (plain.mamba2_fast(_cpu(x), w, "", m, 1e-5, dtype) - ref).abs().amax(dim=1)
    views = _state_views(part)
    _close(_state_portions(part, views, x[:700], (700,), 1, dtype), ref[:700], dtype, 3.0, noise[:700])
    _close(_state_portions(part, views, x, (37, 663) + (1,) * n, 2, dtype), ref, dtype, 3.0, noise)
    _, ctx = _ctx([(0, 5), (0, 690)], dtype=dtype, slots=[4, 0])
    both = part.forward(torch.cat((x[:5], x[:690])), ctx, views)
    _close(both[:5], ref[:5], dtype, 3.0, noise[:5])
    _close(both[5:], ref[:690], dtype, 3.0, noise[:690])


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_mixer_remembers_an_early_token_through_a_slow_head(dtype):
    """Head 0 hardly decays and head 1 forgets within a few tokens: a change of the first token's input must show in
    the last token's output through head 0's channels, and not through head 1's."""
    part, m = _ssm(dtype, 2, 16, 8, 1, 2, 2)

    def decays(t):
        t["A_log"].copy_(torch.tensor([-6.0, 2.0]))
        t["dt_bias"].fill_(1.0)

    w = _bind(part, dtype, change=decays)
    n = 90
    x = _x(n, dtype)
    other = x.clone()
    other[0] = _x(1, dtype, 3.0)[0]
    views = _state_views(part)
    feats = []
    for inp in (x, other):
        _, ctx = _ctx([(0, n - 1)], dtype=dtype, slots=[3])
        part.forward(inp[:n - 1].contiguous(), ctx, views)
        _, ctx = _ctx([(n - 1, 1)], dtype=dtype, slots=[3])
        f = torch.zeros(1, part.feature_width, device=DEV, dtype=dtype)
        part.features(inp[n - 1:].contiguous(), ctx, views, f)
        feats.append(f.float().cpu()[0])
    diff = (feats[0] - feats[1]).abs()
    assert diff[:16].max() > 1e-2 and diff[16:].max() < 1e-3
    _, ctx = _ctx([(0, n)], dtype=dtype, slots=[0])
    _close(part.forward(other, ctx, views), plain.mamba2(_cpu(other), w, "", m, 1e-5, torch.float32), dtype, 3.0)


# --------------------------------------------------------------------------- latent attention with a rotated key part
def _latent(dtype, heads, dim, rot, vdim, rank, q_rank, window, scale=0.3, scaling=True, base=50.0):
    from miniserve_b200.models.rofozen import _latent as spec_of

    m = rx.latent_layer(heads, dim, rot, vdim, rank, q_rank, window, base, scaling, scale)["mixer"]
    return build_part("mixer", spec_of(HIDDEN, 1e-5, m), BuildEnv(dtype, DEV)), m


def _latent_ref(x, w, m):
    return plain.latent_attention(_cpu(x), w, "", m, 1e-5, torch.float32)


def _kv_portions(part, view, x, cuts, page, dtype, full):
    outs, at = [], 0
    for size in cuts:
        size = min(size, x.shape[0] - at)
        if size <= 0:
            break
        _, ctx = _ctx([(at, size)], page, 1, part.cache_dim, dtype, share=full)
        outs.append(part.forward(x[at:at + size].contiguous(), ctx, view).clone())
        at += size
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot, vdim, rank, q_rank, window, page, scaling", [
    (3, 16, 8, 24, 24, 20, 20, 16, True), (5, 12, 4, 20, 28, 12, 5, 8, None), (2, 24, 16, 8, 40, 36, None, 16, True),
    (4, 48, 16, 64, 112, 64, 33, 16, True), (1, 64, 32, 8, 16, 8, 16, 4, True), (2, 16, 0, 24, 36, 16, 7, 8, None),
    (2, 16, 8, 24, 300, 40, 50, 16, True)])  # the last: a cache entry beyond the tensor-core kernels' head sizes
def test_latent_attention_whole_in_portions_and_decoded(dtype, heads, dim, rot, vdim, rank, q_rank, window, page, scaling):
    att, m = _latent(dtype, heads, dim, rot, vdim, rank, q_rank, window, scaling=scaling)
    w = _bind(att, dtype, change=lambda t: t["sink"].mul_(4.0))
    n = 61
    x = _x(n, dtype, 2.0)
    ref = _latent_ref(x, w, m)
    pb, ctx = _ctx([(0, n)], page, 1, att.cache_dim, dtype, seed=1)
    view = KVEntryView(0, pb.k_pool, pb.k_pool, page)
    out = att.forward(x, ctx, view)
    assert pb.status.item() == 0
    _close(out, ref, dtype, 3.0)
    # what the cache holds: the normed latent, then the rotated key part, zeros beyond
    stored = pb.read(0, pb.k_pool, n)[:, 0].float().cpu()
    kv = _cpu(x).double() @ w["dkv"].double().T
    _close(stored[:, :rank], plain.rms_norm(kv[:, :rank].float(), w["dkv.norm"], 1e-5), dtype, 2.0)
    if rot:
        _close(stored[:, rank:rank + rot], plain.rotate(kv[:, rank:].float(), torch.arange(n), rot, 50.0, m["rot"].get("scaling")), dtype, 4.0)
    assert (stored[:, rank + rot:] == 0).all()
    full, _ = _ctx([(0, n)], page, 1, att.cache_dim, dtype, seed=2)
    view = KVEntryView(0, full.k_pool, full.k_pool, page)
    _close(_kv_portions(att, view, x, (page + 3, 2, 13, 2) + (1,) * n, page, dtype, full), ref, dtype, 3.0)
    # two unequal requests in one step (the second decodes a token behind what an earlier step left)
    both_pb, _ = _ctx([(0, 30), (0, n)], page, 1, att.cache_dim, dtype, seed=7)
    view = KVEntryView(0, both_pb.k_pool, both_pb.k_pool, page)
    _, warm = _ctx([(0, 1), (0, n - 1)], page, 1, att.cache_dim, dtype, share=both_pb)
    att.forward(torch.cat((x[:1], x[:n - 1])).contiguous(), warm, view)
    _, ctx = _ctx([(0, 30), (n - 1, 1)], page, 1, att.cache_dim, dtype, share=both_pb)
    both = att.forward(torch.cat((x[:30], x[n - 1:])).contiguous(), ctx, view)
    _close(both[:30], ref[:30], dtype, 3.0)
    _close(both[30:], ref[n - 1:], dtype, 3.0)


def _needle(t):
    """Queries read the same latent as keys (one down projection and norm for both) and every head's query matrix
    is minus its key matrix: a query scores far below everything against its own token's key and far above
    everything against the key of a token whose input is minus its own. The rotated channels carry nothing."""
    rank = t["uk"].shape[1]
    t["dq"].copy_(t["dkv"][:rank])
    t["dq.norm"].copy_(t["dkv.norm"])
    heads = t["sink"].numel()
    dim = t["uk"].shape[0] // heads
    uq = t["uq"].view(heads, -1, rank)
    uq.zero_()
    uq[:, :dim] = -t["uk"].view(heads, dim, rank)
    t["sink"].fill_(-2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, n, page, rank", [(16, 41, 8, 24), (20, 75, 16, 24), (5, 30, 8, 40), (64, 200, 16, 112), (512, 700, 16, 48),
                                                   (1024, 1900, 16, 112), (1, 9, 4, 24)])
def test_a_key_just_inside_and_just_outside_the_window(dtype, window, n, page, rank):
    """The last query and one earlier token are made so that this pair scores far above everything else. With the
    earlier token window - 1 places back its value must come back; one place further it must not: in a prompt, for
    a token decoded alone and in a short portion. A window of one sees only the token itself."""
    heads, dim, vdim = 4, 32, 32
    # (scores grow with the latent's size; the scale keeps the softmax as sharp as at 24: far sharper and bfloat16's
    # rounding of the scores decides between two keys that nearly tie)
    att, m = _latent(dtype, heads, dim, 8, vdim, rank, rank, window, scale=min(1.0, 24.0 / rank))
    w = _bind(att, dtype, change=_needle)
    last = n - 1
    direction = _x(1, dtype, 3.0)[0]
    for needle in (last - window + 1, last - window, last - window + 2, 0):
        if not 0 <= needle < last:
            continue
        x = _x(n, dtype, 0.1)
        x[last], x[needle] = direction, -direction
        ref = _latent_ref(x, w, m)
        blank = x.clone()
        blank[needle] = _x(1, dtype, 0.1)[0]
        shows = (ref[last] - _latent_ref(blank, w, m)[last]).abs().max().item()
        assert (shows > 0.05) == (last - needle < window), "the test's needle shows exactly when it is inside the window"
        full, _ = _ctx([(0, n)], page, 1, att.cache_dim, dtype, seed=3)
        view = KVEntryView(0, full.k_pool, full.k_pool, page)
        _, ctx = _ctx([(0, n)], page, 1, att.cache_dim, dtype, share=full)
        _close(att.forward(x, ctx, view), ref, dtype, 3.0)  # in a prompt
        _, ctx = _ctx([(last, 1)], page, 1, att.cache_dim, dtype, share=full)
        _close(att.forward(x[last:].contiguous(), ctx, view), ref[last:], dtype, 3.0)  # decoded alone over the same pages
        if n > 3:
            _, ctx = _ctx([(n - 3, 3)], page, 1, att.cache_dim, dtype, share=full)
            _close(att.forward(x[n - 3:].contiguous(), ctx, view), ref[n - 3:], dtype, 3.0)  # a short portion


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n, rank", [(700, 48), (1900, 112)])
def test_latent_attention_without_a_window_finds_a_far_key_among_hundreds(dtype, n, rank):
    att, m = _latent(dtype, 4, 32, 8, 32, rank, rank, None, scale=min(1.0, 24.0 / rank))
    w = _bind(att, dtype, change=_needle)
    needle, last = 5, n - 1
    x = _x(n, dtype, 0.1)
    direction = _x(1, dtype, 3.0)[0]
    x[last], x[needle] = direction, -direction
    ref = _latent_ref(x, w, m)
    blank = x.clone()
    blank[needle] = _x(1, dtype, 0.1)[0]
    assert (ref[last] - _latent_ref(blank, w, m)[last]).abs().max() > 0.05, "the test's needle does not show"
    full, _ = _ctx([(0, n)], 16, 1, att.cache_dim, dtype, seed=3)
    view = KVEntryView(0, full.k_pool, full.k_pool, 16)
    _, ctx = _ctx([(0, last)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[:last].contiguous(), ctx, view), ref[:last], dtype, 3.0)
    _, ctx = _ctx([(last, 1)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[last:].contiguous(), ctx, view), ref[last:], dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotated_key_part_decides_by_distance(dtype):
    """Only the rotated channels carry a score: every token has the same rotated query and key before rotation, so
    the score depends on the distance alone (cos of distance times frequency, summed over the pairs) and the
    engine's weights over the keys must follow the oracle's, in a prompt and decoded, at positions of a thousand."""
    heads, dim, rot, rank = 2, 16, 8, 24
    att, m = _latent(dtype, heads, dim, rot, 24, rank, rank, None, scale=2.0, base=10.0, scaling={"factor": 2.0, "fast": 4.0, "original": 32,
                                                                                                  "slow": 1.0})

    def only_rotated(t):
        uq = t["uq"].view(heads, dim + rot, -1)
        uq[:, :dim] = 0.0

    w = _bind(att, dtype, change=only_rotated)
    n = 1200
    x = _x(n, dtype)
    ref = _latent_ref(x, w, m)
    full, _ = _ctx([(0, n)], 16, 1, att.cache_dim, dtype, seed=4)
    view = KVEntryView(0, full.k_pool, full.k_pool, 16)
    _, ctx = _ctx([(0, n - 2)], 16, 1, att.cache_dim, dtype, share=full)
    _close(att.forward(x[:n - 2].contiguous(), ctx, view), ref[:n - 2], dtype, 3.0)
    for at in (n - 2, n - 1):
        _, ctx = _ctx([(at, 1)], 16, 1, att.cache_dim, dtype, share=full)
        _close(att.forward(x[at:at + 1].contiguous(), ctx, view), ref[at:at + 1], dtype, 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_takes_its_share(dtype):
    """A large sink empties the output of its head; a very negative one leaves the plain softmax. The first token of
    a sequence has one key and the sink: its weight is 1 / (1 + exp(sink - score))."""
    att, m = _latent(dtype, 2, 16, 8, 16, 24, 16, 6)

    def sinks(t):
        t["sink"].copy_(torch.tensor([9.0, -30.0]))
        t["o"].copy_(torch.eye(HIDDEN, 32))

    w = _bind(att, dtype, change=sinks)
    n = 20
    x = _x(n, dtype)
    ref = _latent_ref(x, w, m)
    pb, ctx = _ctx([(0, n)], 8, 1, att.cache_dim, dtype)
    out = att.forward(x, ctx, KVEntryView(0, pb.k_pool, pb.k_pool, 8))
    _close(out, ref, dtype, 3.0)
    assert out[:, :16].abs().max() < 0.2 * out[:, 16:32].abs().max()  # head 0 is drowned by its sink
    none = dict(w)
    none["sink"] = torch.tensor([-30.0, -30.0])
    assert (_latent_ref(x, none, m) - ref).abs().max() > 0.05


# --------------------------------------------------------------------------- feed-forward
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, inter", [(40, 72), (36, 52)])
def test_gated_feed_forward_with_tanh_gelu(dtype, hidden, inter):
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(hidden=hidden, intermediate=inter, activation="gelu_tanh",
                                                             names=dict(gate="gate", up="up", down="down"))), BuildEnv(dtype, DEV))
    w = _bind(ffn, dtype)
    x = (torch.randn(9, hidden, device=DEV) * 2).to(dtype)
    _, ctx = _ctx([(0, 9)], dtype=dtype)
    _close(ffn.forward(x, ctx), plain.dense_ff(_cpu(x), w, "", torch.float32), dtype, 3.0)


def _experts(dtype, hidden, ff, experts, identity, top, count, keep, scale):
    from miniserve_b200.models.rofozen import _feed_forward as spec_of

    mlp = rx.moe(ff, experts, identity, top, count, keep, scale)
    return build_part("feed_forward", spec_of(hidden, mlp), BuildEnv(dtype, DEV)), mlp


EXPERT_CASES = [(48, 24, 6, 2, 2, 2, 1, 1.5), (36, 20, 5, 0, 1, 0, 1, 1.0), (40, 28, 7, 2, 4, 3, 2, 0.7), (64, 64, 8, 0, 2, 4, 2, 2.5),
                (48, 16, 1, 1, 1, 0, 1, 1.0), (48, 40, 12, 4, 6, 4, 2, 1.0), (56, 24, 3, 0, 3, 0, 1, 1.0), (128, 136, 30, 2, 8, 8, 3, 1.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, ff, experts, identity, top, count, keep, scale", EXPERT_CASES)
def test_router_and_experts(dtype, hidden, ff, experts, identity, top, count, keep, scale):
    ffn, mlp = _experts(dtype, hidden, ff, experts, identity, top, count, keep, scale)

    def sharpen(t):
        t["router"].mul_(1.5)
        t["correction"].mul_(0.3)  # of the size of the scores: it changes choices, and some choice scores are negative

    w = _bind(ffn, dtype, change=sharpen)
    for n in (1, 2, 77, 300):
        x = (torch.randn(n, hidden, device=DEV)).to(dtype)
        _, ctx = _ctx([(0, n)], dtype=dtype)
        idx, wgt = ffn.route(x, ctx)
        chosen, weights = plain.route(_cpu(x), w, "", mlp["router"], torch.float32)
        order_g, order_w = idx.long().cpu().sort(-1), chosen.sort(-1)
        assert (order_g.values == order_w.values).all()
        assert torch.allclose(wgt.cpu().gather(1, order_g.indices), weights.gather(1, order_w.indices), rtol=1e-4, atol=1e-6)
        want = plain.moe_ff(_cpu(x), w, "", mlp, torch.float32)
        _close(ffn.forward(x, ctx), want, dtype, 3.0)
        if dtype == torch.bfloat16:  # the products on the older tensor-core path too (what shapes off the tcgen05 kernel's take)
            from miniserve_b200.ops import experts as xo

            held, xo.TC_EXPERTS = xo.TC_EXPERTS, False
            try:
                _close(ffn.forward(x, ctx), want, dtype, 3.0)
            finally:
                xo.TC_EXPERTS = held


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_correction_chooses_but_does_not_weigh_and_groups_shut_experts_out(dtype):
    """Router rows of zero give every output the same score 1/R: the correction alone decides. The largest
    correction sits in group 1 and the next two in group 0; with one group kept both choices come from group 1,
    although group 0 holds the second and third best. A negative correction everywhere keeps choice scores below
    zero: an output that is shut out counts as minus infinity, not as zero."""
    hidden = 48
    ffn, mlp = _experts(dtype, hidden, 24, 4, 2, 2, 2, 1, 3.0)

    def fixed(t):
        t["router"].zero_()
        t["correction"].copy_(torch.tensor([-0.5, -0.4, -0.9, -0.8, -0.3, -0.95]))

    w = _bind(ffn, dtype, change=fixed)
    x = torch.randn(5, hidden, device=DEV).to(dtype)
    _, ctx = _ctx([(0, 5)], dtype=dtype)
    idx, wgt = ffn.route(x, ctx)
    assert (idx.long().cpu().sort(-1).values == torch.tensor([3, 4])).all()  # an expert and an identity expert of group 1
    assert torch.allclose(wgt.cpu(), torch.full((5, 2), 3.0 / 6.0), rtol=1e-5)
    _close(ffn.forward(x, ctx), plain.moe_ff(_cpu(x), w, "", mlp, torch.float32), dtype, 3.0)


# --------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module", params=["a", "b", "c"])
def model(request, tmp_path_factory):
    raw = dict(a=rx.config_a, b=rx.config_b, c=rx.config_c)[request.param]()
    folder = rx.write_model(tmp_path_factory.mktemp("rofozen_" + request.param), raw, seed=dict(a=11, b=12, c=13)[request.param])
    return dict(folder=folder, raw=raw, oracle=rx.oracle(folder), rounded=rx.oracle(folder, torch.bfloat16),
                page=dict(a=16, b=8, c=32)[request.param])


def _logits_close(model, dtype, got, ids, what=""):
    """32-bit: within F32 of the oracle. bfloat16: as near as rounding allows, position by position (``rx.rounded_ok``)."""
    want = model["oracle"](ids)
    if dtype == "float32":
        err = rx.rel_err(got, want)
        assert err < F32, f"{what}: {err:.2e}"
    else:
        ok, report = rx.rounded_ok(got, want, model["rounded"](ids))
        assert ok, f"{what}: {report}"


def test_layer_streams_in_float32(model):
    """The residual stream after every layer run, against the oracle's (a layer that runs again counts each time)."""
    from miniserve_b200.cache import CacheManager
    from miniserve_b200.engine.loader import load_model
    from miniserve_b200.engine.step import StepFunction, StepRow

    ids = _ids(29, model["raw"]["vocab"], 8)
    want = rx.layer_streams(model["folder"], ids)
    _, _, net = load_model(model["folder"], "float32", "cuda:0")
    cache = CacheManager(net.entry_caches, 8, 16, 2, dtype=net.dtype, device=net.device)
    ctx = StepFunction(net, cache).prepare([StepRow(cache.new_request(), ids, [0])])
    stream = ResidualStream(net.embedding.forward(ctx))
    for i, e in enumerate(net.spec.run_order):
        stream = net.layers[e.layer].forward(stream, ctx, cache.entry_views[i])
        x = stream.total.double().cpu()
        if stream.pending is not None:
            x = x + stream.pending_scale * stream.pending.double().cpu()
        assert (x - want[i].double()).abs().max() < 1e-4 * max(1.0, want[i].abs().max().item()), f"after run {i} (layer {e.layer})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(model, dtype):
    vocab = model["raw"]["vocab"]
    run = rx.Runner(model["folder"], dtype, max_tokens=256, page_size=model["page"])
    for n, seed in ((1, 1), (2, 2), (37, 3), (150, 4)):
        ids = _ids(n, vocab, seed)
        _logits_close(model, dtype, run.feed("w", ids, [n]), ids, f"{n} whole")
        if n > 2:
            # the last 110 one by one: the window passes over decoded tokens
            _logits_close(model, dtype, run.feed("d", ids, [n - min(n - 1, 110), 1]), ids, f"{n} decoded")
            _logits_close(model, dtype, run.feed("c", ids, [7, 2, 24, 3, model["page"], 2, 5, 31, 2, 1, 1, 2, 9]), ids, f"{n} in portions")
        assert run.cache.is_idle()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, portions of some beside single tokens of others, a pool that holds only what is
    live and four state slots: every page and slot is used by several requests in turn (both are filled with NaN
    when given back, and the layers with a window give pages back while a request runs)."""
    vocab = model["raw"]["vocab"]
    seqs = {f"r{i}": _ids(n, vocab, 20 + i) for i, n in enumerate([90, 5, 64, 33, 1, 120, 17, 48, 2, 75])}
    run = rx.Runner(model["folder"], dtype, max_tokens=4 * 128, page_size=model["page"], max_requests=4)
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
    run = rx.Runner(model["folder"], "float32", max_tokens=448, page_size=model["page"])
    assert rx.rel_err(run.feed("long", ids, [3, 1]), model["oracle"](ids)) < F32


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
        assert rx.rel_err(logits[None], want[rid][pos:pos + 1]) < F32, (rid, pos)


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
        # bfloat16: how far rounding alone moves the oracle's own logits at each position
        moved = (model["rounded"](list(p) + list(o)) - every).abs().amax(dim=1) if dtype == "bfloat16" else None
        for i, t in enumerate(o):  # teacher-forced: each chosen token is the oracle's best, or within rounding of it
            at = len(p) + i - 1
            logits = every[at]
            slack = 1e-4 if dtype == "float32" else max(0.15, 3.0 * moved[at].item())
            assert (logits.max() - logits[t]).item() <= slack, (at + 1, t)
