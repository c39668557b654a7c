"""Kikelorn as data: its configuration turned into a ``ModelSpec``.

Every layer is an out-norm block: each sublayer reads the residual stream itself through a causal
convolution over time, its result is gated by a sigmoid of a linear map of the residual stream,
normed, multiplied by ``residual_mult`` and added.  The mixer is one of three parts: the attention
part in the variant "convolutions on q, k and v, RMS norm over the whole q and the whole k
projection, rotate-half rotation of the first ``rot.dims`` values, value heads of their own size, a
chunked mask, values mixed with those of the first mixing layer, a gate per head"; the latent
attention part in the variant "query latent, rotation of adjacent pairs with YaRN frequencies, a
gate per output value"; the minGRU part.  The feed-forward is the dense part with biases and the
tanh GELU.  The head is the embedding table (without the embedding's scale).

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``, ``norm2``, ``canon1``, ``canon2``,
``rg1``, ``rg1.b``, ``rg2``, ``rg2.b``; ``l<i>.mix.*`` (attention: ``q, k, v, q.norm, k.norm, q.conv, k.conv, v.conv,
vmix, g, o``; latent attention: ``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o``; minGRU: ``z, z.b, x, x.b,
g, o``); ``l<i>.mlp.{up, up.b, down, down.b}``; matrices are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

from ..config.kikelorn import KikelornAttention, KikelornConfig, KikelornLatent
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec


def _rotary(rot, pairing: str):
    if rot is None:
        return None
    params = {"theta": rot.base, "rot_dim": rot.dims, "pairing": pairing}
    if rot.scaling is not None:
        params["scaling"] = rot.scaling_dict()
    return PartSpec("rotary", params)


def kikelorn_spec(cfg: KikelornConfig) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.width, "eps": cfg.eps})
    layers, unused = [], []
    mixing_seen = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        names = {"norm1.weight": p + "norm1", "conv1": p + "canon1", "gate1_proj": p + "rg1", "gate1_proj.bias": p + "rg1.b"}
        q = p + "mix."
        if isinstance(m, KikelornAttention):
            v_mix = None
            if m.v_mix:
                v_mix = "mix" if mixing_seen else "source"
                mixing_seen = True
                names["mixer.v_mix"] = q + "vmix"
            else:       # a checkpoint may still carry the factor of a layer that does not mix
                unused.append(q + "vmix")
            mixer = PartSpec("attention", {
                "width": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
                "position": _rotary(m.rot, "half"), "qk_norm": "row", "eps": cfg.eps, "scale": m.scale, "chunk": m.chunk,
                "exact_weights": True, "conv_taps": m.conv, "v_mix": v_mix, "gate": "head"})
            names.update({"mixer.q_proj": q + "q", "mixer.k_proj": q + "k", "mixer.v_proj": q + "v",
                          "mixer.q_norm": q + "q.norm", "mixer.k_norm": q + "k.norm", "mixer.q_proj.conv": q + "q.conv",
                          "mixer.k_proj.conv": q + "k.conv", "mixer.v_proj.conv": q + "v.conv", "mixer.g_proj": q + "g",
                          "mixer.o_proj": q + "o"})
        elif isinstance(m, KikelornLatent):
            mixer = PartSpec("latent_attention", {
                "width": cfg.width, "n_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
                "kv_rank": m.kv_rank, "q_rank": m.q_rank, "position": _rotary(m.rot, "adjacent"), "eps": cfg.eps,
                "scale": m.scale, "gate": "value"})
            names.update({"mixer.dq_proj": q + "dq", "mixer.dq_norm": q + "dq.norm", "mixer.uq_proj": q + "uq",
                          "mixer.dkv_proj": q + "dkv", "mixer.dkv_norm": q + "dkv.norm", "mixer.uk_proj": q + "uk",
                          "mixer.uv_proj": q + "uv", "mixer.g_proj": q + "g", "mixer.o_proj": q + "o"})
        else:
            mixer = PartSpec("min_gru", {"width": cfg.width, "inner": m.width, "candidate": "positive"})
            names.update({"mixer.z_proj": q + "z", "mixer.z_proj.bias": q + "z.b", "mixer.x_proj": q + "x",
                          "mixer.x_proj.bias": q + "x.b", "mixer.g_proj": q + "g", "mixer.o_proj": q + "o"})
        params = {"width": cfg.width, "norm1": norm, "mixer": mixer, "mult": cfg.residual_mult,
                  "conv_taps": cfg.canon_taps, "gate": True}
        if layer.mlp is not None:
            f = p + "mlp."
            params.update({"norm2": norm, "ffn": PartSpec("dense_mlp", {"width": cfg.width, "inner": layer.mlp.ff,
                                                                        "activation": "gelu_tanh", "bias": True})})
            names.update({"norm2.weight": p + "norm2", "conv2": p + "canon2", "gate2_proj": p + "rg2",
                          "gate2_proj.bias": p + "rg2.b", "ffn.up_proj": f + "up", "ffn.up_proj.bias": f + "up.b",
                          "ffn.down_proj": f + "down", "ffn.down_proj.bias": f + "down.b"})
        else:       # a checkpoint may still carry what stands around the feed-forward the layer does not have
            unused += [p + "norm2", p + "canon2", p + "rg2", p + "rg2.b"]
        layers.append(LayerSpec(block=PartSpec("outnorm", params), names=names))
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding_name="embed", layers=tuple(layers),
        schedule=tuple(RunSpec(layer=i) for i in range(len(layers))),
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name=None, ignored_names=tuple(unused),
        max_positions=cfg.max_positions, stop_ids=tuple(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale)


def describe(config: Dict[str, Any]) -> ModelSpec:
    return kikelorn_spec(KikelornConfig.from_dict(config))
