"""Munerax as data: its configuration turned into a ``ModelSpec``.

The embedded tokens (times the embedding's scale) get a hashed bigram embedding added (an input
part with the previous token as per-sequence state).  Every layer is a pre-norm block; its mixer is
the latent attention part with rotate-half rotation of the rotated part, a learned sink per head
and an output gate per head; a layer with ``kv_from`` has no down projection and its run reads the
cache of the named layer's run.  The feed-forward is the gated one with the tanh GELU, or the
routed part in the variant "sigmoid scores, no correction, a group counts by its two best scores,
weights times the router's scale, experts ``W_down relu(W_up h)^2``, a shared expert of the same form
added as it is".  The head is the embedding table (without the embedding's scale).

Tensor names: ``embed``, ``bigram``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q, dkv, dkv.norm, uk, uv, sink, g, o}``, ``l<i>.mlp.{gate, up, down}`` or
``l<i>.mlp.{router, e<j>.up, e<j>.down, shared.up, shared.down}``; matrices are ``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

from ..config.munerax import MuneraxConfig, MuneraxDense
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

GROUP_SCORE_TOP = 2     # a group of experts counts by the sum of its two best scores


def munerax_spec(cfg: MuneraxConfig) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.width, "eps": cfg.eps})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        own = m.kv_from is None
        position = None
        if m.rot_base is not None and m.rot_dims > 0:
            position = PartSpec("rotary", {"theta": m.rot_base, "rot_dim": m.rot_dims, "pairing": "half"})
        mixer = PartSpec("latent_attention", {
            "width": cfg.width, "n_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
            "kv_rank": m.kv_rank, "position": position, "eps": cfg.eps, "scale": m.scale, "own_kv": own,
            "sink": "learned", "gate": True})
        names = {"norm1.weight": p + "norm1", "mixer.q_proj": p + "mix.q", "mixer.uk_proj": p + "mix.uk",
                 "mixer.uv_proj": p + "mix.uv", "mixer.sink": p + "mix.sink", "mixer.g_proj": p + "mix.g",
                 "mixer.o_proj": p + "mix.o"}
        if own:
            names.update({"mixer.dkv_proj": p + "mix.dkv", "mixer.dkv_norm": p + "mix.dkv.norm"})
        params = {"norm1": norm, "mixer": mixer}
        f = layer.mlp
        if f is not None:
            q = p + "mlp."
            names["norm2.weight"] = p + "norm2"
            if isinstance(f, MuneraxDense):
                ffn = PartSpec("gated_mlp", {"width": cfg.width, "inner": f.ff, "activation": "gelu_tanh"})
                names.update({"ffn.gate_proj": q + "gate", "ffn.up_proj": q + "up", "ffn.down_proj": q + "down"})
            else:
                ffn = PartSpec("mixture_of_experts", {
                    "width": cfg.width, "n_experts": f.experts, "top": f.top, "inner": f.ff, "n_groups": f.groups,
                    "keep_groups": f.keep, "shared_inner": f.shared_ff, "correction": False, "weight_scale": f.scale,
                    "score": "sigmoid", "group_top": GROUP_SCORE_TOP, "expert": "relu_squared", "shared_gate": False})
                names["ffn.router"] = q + "router"
                for e in range(f.experts):
                    names[f"ffn.experts.{e}.up_proj"] = f"{q}e{e}.up"
                    names[f"ffn.experts.{e}.down_proj"] = f"{q}e{e}.down"
                if f.shared_ff is not None:
                    names.update({"ffn.shared.up_proj": q + "shared.up", "ffn.shared.down_proj": q + "shared.down"})
            params.update({"norm2": norm, "ffn": ffn})
        layers.append(LayerSpec(block=PartSpec("prenorm", params), names=names))
        schedule.append(RunSpec(layer=i, cache_of=m.kv_from))      # run i is layer i: every layer runs once, in order
    inputs = ()
    if cfg.bigram is not None:
        b = cfg.bigram
        inputs = ((PartSpec("hashed_bigram", {"width": cfg.width, "vocab": cfg.vocab, "buckets": b.buckets,
                                              "mul_prev": b.mul_prev, "mul_cur": b.mul_cur}), {"table": "bigram"}),)
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name=None,
        max_positions=cfg.max_positions, stop_ids=tuple(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale,
        input_parts=inputs)


def describe(config: Dict[str, Any]) -> ModelSpec:
    return munerax_spec(MuneraxConfig.from_dict(config))
