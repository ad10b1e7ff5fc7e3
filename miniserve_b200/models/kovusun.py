"""The Kovusun decoder as data: its configuration mapped onto parts.

Every layer adds ``mixer(shift(norm1(x))) + ff(norm2(x))`` to the stream: two layer norms (weight and bias) of the same
x, and a token shift (a per-channel mix with the previous token's normed input, carried as per-request state) in front
of the mixer. Three attention mixers over grouped heads with a sliding window: ``attention`` (biases on q, k and v; q
and k divided by their root mean square; a logarithmic distance bias per head; optionally reading an earlier layer's
keys and values), ``attention_2`` (the same unit norm, no positions, a learned sink per head in the softmax's
denominator, a sigmoid gate per head and token) and ``attention_3`` (rotation of adjacent channel pairs, a learned
temperature per head, the sequence's first keys kept visible behind the window). Feed-forward: dense and gated, with
biases and clamps, or a mixture of SiLU-gated experts (a router with a bias, weights by a softmax over the chosen
logits) beside a shared expert weighed by a sigmoid gate per token, or none. Tensor names are the checkpoint's:
``embed``, ``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.kovusun import KovusunConfig, KovusunLayer
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

_NAMES = dict(q="q", k="k", v="v", o="o", gate="g", sink="sink", q_bias="q.b", k_bias="k.b", v_bias="v.b", temp="temp", r1="r1", r2="r2")


def _cache_window(cfg: KovusunConfig, index: int) -> int | None:
    """How far back layer ``index`` must keep keys: its own reach unless a layer that reads its cache reaches further
    (0: everything). None: the mixer's own reach."""
    readers = [layer for layer in cfg.layers if layer.kv_from == index]
    if not readers:
        return None
    reaches = [0 if layer.keep_first else layer.window for layer in (cfg.layers[index], *readers)]
    return 0 if 0 in reaches else max(reaches)


def _mixer(cfg: KovusunConfig, index: int, layer: KovusunLayer) -> PartSpec:
    c = layer.mixer
    p = dict(hidden=cfg.width, heads=int(c["heads"]), kv_heads=int(c["kv_heads"]), head_dim=int(c["dim"]), value_dim=int(c["vdim"]),
             scale=float(c["scale"]), window=layer.window, qk_norm_eps=cfg.eps, names=_NAMES, general=True,
             kv_source="own" if layer.kv_from is None else "shared")
    window = _cache_window(cfg, index)
    if window is not None:
        p["cache_window"] = window
    if layer.type == "attention":
        p.update(qk_norm="unit", qkv_bias=True, distance_bias=True)
    elif layer.type == "attention_2":
        p.update(qk_norm="unit", sink="learned", out_gate="head_sigmoid")
    else:
        rot = c.get("rot")
        if rot is not None and int(rot["dims"]) > 0:
            p["position"] = PartSpec("rope_pairs", dict(head_dim=int(c["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"])))
        p.update(head_temperature=True, keep_first=layer.keep_first)
    return PartSpec("gqa_attention", p)


def _feed_forward(width: int, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("clamped_glu", dict(
            hidden=width, intermediate=int(mlp["ff"]), limit=float(mlp["limit"]) if mlp.get("limit") is not None else None, alpha=1.702,
            up_shift=1.0, bias=True,
            names=dict(gate="gate", up="up", down="down", gate_bias="gate.b", up_bias="up.b", down_bias="down.b")))
    r = mlp["router"]
    shared = mlp.get("shared")
    return PartSpec("routed_experts", dict(
        hidden=width, intermediate=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), score="softmax",
        renormalize=True, correction=False, router_bias=True, activation="silu", shared=int(shared["ff"]) if shared else 0,
        names=dict(router="router", router_bias="router.b", expert="e{}.", gate="gate", up="up", down="down", shared="shared.",
                   shared_gate="shared.sg")))


def kovusun_model_spec(cfg: KovusunConfig) -> ModelSpec:
    norm = PartSpec("layernorm", dict(size=cfg.width, eps=cfg.eps, names=dict(weight="", bias=".b")))
    layers: list[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        ffn = _feed_forward(cfg.width, layer.mlp)
        names = dict(mixer="mix.", norm1="norm1")
        norms = dict(norm1=norm)
        if ffn is not None:
            names.update(feed_forward="mlp.", norm2="norm2")
            norms["norm2"] = norm
        block = PartSpec("parallel_dual_norm", dict(names=names, token_shift="shift", hidden=cfg.width))
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, mixer=_mixer(cfg, i, layer), feed_forward=ffn, norms=norms))
    run_order = tuple(RunEntry(i, cache_of=layer.kv_from) for i, layer in enumerate(cfg.layers))
    # a layer without a feed-forward has nothing for a second norm to feed: a checkpoint may carry its tensors all the same
    spare = tuple(f"l{i}.norm2{suffix}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for suffix in ("", ".b"))
    return ModelSpec(
        architecture="Kovusun", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, name="embed")),
        layers=tuple(layers), run_order=run_order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", dict(vocab=cfg.vocab, hidden=cfg.width, tied=False, name="head")), optional_tensors=spare)


KOVUSUN = register_architecture(Architecture("Kovusun", KovusunConfig.from_dict, kovusun_model_spec), replace=True)
