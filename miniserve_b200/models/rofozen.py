"""The Rofozen decoder as data: its configuration mapped onto parts.

Pre-norm layers with RMS norms; two kinds of mixer, ``mamba2`` (a selective state-space layer in its dual form: a
scalar decay per head and token, inputs through a short causal convolution, a gate before a norm in groups) and
``latent_attention`` (queries through a normed latent; keys and values of all heads made from one small normed
vector per token, with one rotated key part shared by the heads beside it, the only things cached; rescaled rotary
frequencies; a sliding window; a learned sink per head); a gated dense feed-forward with tanh-GELU, a mixture of
SiLU-gated experts with a corrected, group-limited choice and identity experts, or none; a layer may run with
another layer's tensors and a cache of its own. Tensor names are the checkpoint's: ``embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.rofozen import RofozenConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mamba2(width: int, eps: float, c) -> PartSpec:
    return PartSpec("mamba2", dict(
        hidden=width, heads=int(c["heads"]), head_dim=int(c["vdim"]), state=int(c["state"]), groups=int(c["groups"]),
        conv=int(c["conv"]), norm_groups=int(c["norm_groups"]), eps=eps,
        names=dict(input="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", skip="D", norm="norm", o="o")))


def _latent(width: int, eps: float, c) -> PartSpec:
    rd = int(c.get("rot_dim", 0))
    position = PartSpec("none")
    if rd:
        rot = c["rot"]
        # without rescaling: a factor of one leaves every frequency and the factor on cos and sin as they are
        scaling = rot.get("scaling") or {"factor": 1.0, "original": 1.0, "fast": 1.0, "slow": 1.0}
        position = PartSpec("rope_yarn", dict(head_dim=rd, theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                                              factor=float(scaling["factor"]), original=float(scaling["original"]),
                                              fast=float(scaling["fast"]), slow=float(scaling["slow"])))
    mask = c.get("mask")
    return PartSpec("latent_attention", dict(
        hidden=width, heads=int(c["heads"]), head_dim=int(c["dim"]), value_dim=int(c["vdim"]), latent=int(c["kv_rank"]),
        q_latent=int(c["q_rank"]), rotated_dim=rd, position=position, window=int(mask["size"]) if mask else None,
        sink="learned", out_gate=None, scale=float(c["scale"]), eps=eps,
        names=dict(q_down="dq", q_norm="dq.norm", q="uq", down="dkv", norm="dkv.norm", up_k="uk", up_v="uv", sink="sink", o="o")))


def _feed_forward(width: int, mlp) -> PartSpec | None:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden=width, intermediate=int(mlp["ff"]), activation="gelu_tanh",
                                       names=dict(gate="gate", up="up", down="down")))
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("routed_experts", dict(
        hidden=width, intermediate=int(mlp["expert"]["ff"]), experts=int(r["experts"]), identity=int(r.get("identity", 0)),
        top=int(r["top"]), group_count=int(groups["count"]), group_keep=int(groups["keep"]), weight_scale=float(r.get("scale", 1.0)),
        score="softmax", renormalize=False, activation="silu",
        names=dict(router="router", correction="correction", expert="e{}.", gate="gate", up="up", down="down")))


def rofozen_model_spec(cfg: RofozenConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.eps, name=""))
    layers: list[LayerSpec] = []
    index_of: dict[int, int] = {}  # config layer -> index among the layers that have tensors
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        mixer = _mamba2(cfg.width, cfg.eps, layer.mixer) if layer.type == "mamba2" else _latent(cfg.width, cfg.eps, layer.mixer)
        ffn = _feed_forward(cfg.width, layer.mlp)
        names = dict(mixer="mix.", norm1="norm1")
        norms = dict(norm1=norm)
        if ffn is not None:
            names.update(feed_forward="mlp.", norm2="norm2")
            norms["norm2"] = norm
        index_of[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm", dict(names=names)), mixer=mixer, feed_forward=ffn,
                                norms=norms))
    run_order = tuple(RunEntry(index_of[layer.weights_of if layer.weights_of is not None else i])
                      for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        architecture="Rofozen", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=cfg.width, name="embed")),
        layers=tuple(layers), run_order=run_order, final_norm=norm, final_norm_prefix="final.norm",
        head=PartSpec("linear_head", dict(vocab=cfg.vocab, hidden=cfg.width, tied=False, name="head")))


ROFOZEN = register_architecture(Architecture("Rofozen", RofozenConfig.from_dict, rofozen_model_spec), replace=True)
