"""Named config.json contents for the random-weights mode and the benchmark.

The reference names models by size and pins checkpoints to download
(miniserve/model/weights.py:24-39); there is no network here, so a preset is just the
config.json of that size. These are data for ``--random PRESET``; no kernel or part
reads a size from this file.
"""

from __future__ import annotations


def _qwen3(hidden, inter, vocab, layers, heads, kv_heads, head_dim, theta, eps, tied, max_pos) -> dict:
    return dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
        hidden_size=hidden, intermediate_size=inter, vocab_size=vocab, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
        rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tied, max_position_embeddings=max_pos,
    )


def _fekulix(width, vocab, ff, pattern, left, right, delta) -> dict:
    """A Fekulix config.json: ``pattern`` is a string of P (parallel layer) and D (channel_delta layer); a
    layer written in lower case runs with the tensors of the first layer of its kind."""
    first = {"P": pattern.index("P") if "P" in pattern else None, "D": pattern.index("D") if "D" in pattern else None}
    layers = []
    for ch in pattern:
        kind = ch.upper()
        entry = ({"type": "parallel", "mixer": {"left": dict(left), "left_scale": 1.0, "right": dict(right), "right_scale": 0.5}}
                 if kind == "P" else {"type": "channel_delta", "mixer": dict(delta)})
        entry["mlp"] = {"kind": "dense", "ff": ff}
        if ch.islower():
            entry["weights_of"] = first[kind]
        layers.append(entry)
    return dict(architecture="Fekulix", width=width, vocab=vocab, logit_scale=1.0, norm={"eps": 1e-6}, layers=layers)


def _mugipel(width, vocab, ff, pattern, attention, latent, loop, mult) -> dict:
    """A Mugipel config.json: ``pattern`` is a string of A (attention layer) and L (latent-attention layer);
    ``loop`` = (start, stop, times) or None."""
    layers = [{"type": "attention" if ch == "A" else "latent_attention", "mixer": dict(attention if ch == "A" else latent),
               "mlp": {"kind": "dense", "ff": ff}} for ch in pattern]
    raw = dict(architecture="Mugipel", width=width, vocab=vocab, norm={"eps": 1e-5}, residual_mult=mult, layers=layers)
    if loop:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


def _kovusun(width, vocab, ff, heads, kv_heads, dim, window) -> dict:
    """A Kovusun config.json of four layers: attention with a distance bias, rotary attention with kept first keys,
    attention that reads the first layer's keys and values, attention with a sink and a gate; dense and routed
    feed-forwards in turn."""
    base = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": dim ** -0.5, "vdim": dim}
    dense = {"ff": ff, "kind": "dense", "limit": 4.0}
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 6, "top": 2}, "shared": {"ff": ff // 2}}
    layers = []
    for i, kind in enumerate(("attention", "attention_3", "attention", "attention_2")):
        mixer = {k: (dict(v) if isinstance(v, dict) else v) for k, v in base.items()}
        if kind == "attention_3":
            mixer["mask"]["keep_first"] = 2
            mixer["rot"] = {"base": 10000.0, "dims": dim // 2}
        if i == 2:
            mixer["kv_from"] = 0
        layers.append({"type": kind, "mixer": mixer, "mlp": dict(moe if i % 2 else dense)})
    return dict(architecture="Kovusun", width=width, vocab=vocab, norm={"eps": 1e-5}, layers=layers)


PRESETS: dict[str, dict] = {
    "kovusun-tiny": _kovusun(96, 503, 160, 6, 2, 32, 48),
    "mugipel-tiny": _mugipel(
        96, 503, 160, "ALAL",
        attention={"dim": 32, "heads": 6, "kv_heads": 2, "mask": {"size": 64}, "scale": 32 ** -0.5, "softcap": 30.0, "vdim": 32,
                   "rot": {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 16.0, "original": 256, "slow": 1.0}}},
        latent={"dim": 16, "heads": 6, "kv_rank": 48, "scale": 0.25, "vdim": 16}, loop=(2, 4, 2), mult=0.6),
    "fekulix-tiny": _fekulix(
        96, 503, 160, "PDpd",
        left={"dim": 32, "heads": 6, "kv_heads": 2, "rot": {"base": 10000.0, "dims": 16}, "scale": 32 ** -0.5, "vdim": 16},
        right={"dim": 16, "heads": 3, "tau": 8.0, "vdim": 32, "decay_rank": 8},
        delta={"conv": 3, "dim": 24, "heads": 4, "kv_heads": 2, "vdim": 24, "decay_rank": 8, "gate_rank": 16}),
    "tiny-a": _qwen3(64, 128, 256, 2, 4, 2, 16, 10000.0, 1e-6, True, 128),
    "tiny-b": _qwen3(96, 224, 503, 3, 6, 1, 32, 1000000.0, 1e-5, False, 256),
    "0.6b": _qwen3(1024, 3072, 151936, 28, 16, 8, 128, 1000000.0, 1e-6, True, 40960),
    "1.7b": _qwen3(2048, 6144, 151936, 28, 16, 8, 128, 1000000.0, 1e-6, True, 40960),
    "8b": _qwen3(4096, 12288, 151936, 36, 32, 8, 128, 1000000.0, 1e-6, False, 40960),
    "32b": _qwen3(5120, 25600, 151936, 64, 64, 8, 128, 1000000.0, 1e-6, False, 40960),
}


def preset(name: str) -> dict:
    try:
        return dict(PRESETS[name.lower()])
    except KeyError:
        raise ValueError(f"unknown preset {name!r}; expected one of {sorted(PRESETS)}") from None
