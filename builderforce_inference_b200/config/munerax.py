"""``MuneraxConfig``: the sizes and constants of a Munerax decoder, read from its config.json.

A Munerax model adds a hashed bigram embedding to the token embedding and is a stack of pre-norm
blocks whose mixer is latent attention (all heads' keys and values are made from one small cached
vector per token; a layer may borrow an earlier layer's cache) and whose feed-forward, where a
layer has one, is a dense gated one or a mixture of experts.  config.json carries:

    architecture            "Munerax"
    vocab, width            vocabulary size, residual width
    norm.eps                epsilon of every RMS norm
    embedding.scale         factor on the token embedding (default 1; the tied head does not take it)
    embedding.bigram        absent, or {buckets, mul_prev, mul_cur}
    layers[i].type          "latent_attention"
    layers[i].mixer         heads, dim, rot_dim, vdim, kv_rank, scale, rot.{base, dims},
                            kv_from (optional: the layer whose cache this one reads)
    layers[i].mlp           null, {kind: "dense", ff}, or
                            {kind: "moe", expert.ff, router.{experts, top, scale, groups.{count, keep}},
                             shared.ff (optional)}

Every value is checked here, so a bad folder fails by key before any weight is read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ConfigReader
from .datasun import _sub


@dataclass(frozen=True)
class MuneraxBigram:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class MuneraxLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: Optional[float]
    rot_dims: int
    kv_from: Optional[int]


@dataclass(frozen=True)
class MuneraxDense:
    ff: int


@dataclass(frozen=True)
class MuneraxMoE:
    experts: int
    top: int
    ff: int
    groups: int
    keep: int
    scale: float
    shared_ff: Optional[int]


@dataclass(frozen=True)
class MuneraxLayer:
    type: str
    mixer: MuneraxLatent
    mlp: Any                    # None, MuneraxDense or MuneraxMoE


def _latent(r: ConfigReader, index: int) -> MuneraxLatent:
    heads = r.integer("heads", minimum=1)
    dim = r.integer("dim", minimum=1)
    rot_dim = r.integer("rot_dim", default=0, minimum=0)
    rank = r.integer("kv_rank", minimum=1)
    if (rank + rot_dim) % 2 != 0 or rank + rot_dim > 1024 or rank > 512:
        raise ConfigError(f"{r.what}: kv_rank = {rank} must be at most 512, kv_rank + rot_dim = {rank + rot_dim} even and at most 1024")
    base, dims = None, 0
    rot = _sub(r, "rot", required=False)
    if rot is not None and rot_dim > 0:
        dims = rot.integer("dims", default=rot_dim, minimum=2)
        if dims % 2 != 0 or dims > rot_dim:
            raise ConfigError(f"{rot.what}: key 'dims' must be even and at most rot_dim {rot_dim}, got {dims}")
        base = rot.number("base", positive=True)
    src = r.integer("kv_from", default=None, minimum=0)
    if src is not None and src >= index:
        raise ConfigError(f"{r.what}: key 'kv_from' must name an earlier layer, got {src}")
    return MuneraxLatent(heads=heads, dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim", default=dim, minimum=1), kv_rank=rank,
                         scale=r.number("scale", default=(dim + rot_dim) ** -0.5, positive=True), rot_base=base,
                         rot_dims=dims, kv_from=src)


def _mlp(r: ConfigReader):
    kind = r.string("kind", default="dense")
    if kind == "dense":
        return MuneraxDense(ff=r.integer("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{r.what}: key 'kind' must be \"dense\" or \"moe\", got {kind!r}")
    router = _sub(r, "router")
    experts = router.integer("experts", minimum=1)
    top = router.integer("top", minimum=1)
    if top > experts:
        raise ConfigError(f"{router.what}: key 'top' {top} exceeds the {experts} experts")
    count = keep = 1
    groups = _sub(router, "groups", required=False)
    if groups is not None:
        count = groups.integer("count", default=1, minimum=1)
        keep = groups.integer("keep", default=count, minimum=1)
        if experts % count != 0 or keep > count:
            raise ConfigError(f"{groups.what}: {experts} experts in {count} groups, {keep} kept")
        if keep * (experts // count) < top:
            raise ConfigError(f"{groups.what}: {keep} groups of {experts // count} experts cannot give top {top}")
    shared = _sub(r, "shared", required=False)
    return MuneraxMoE(experts=experts, top=top, ff=_sub(r, "expert").integer("ff", minimum=1), groups=count, keep=keep,
                      scale=router.number("scale", default=1.0),
                      shared_ff=None if shared is None else shared.integer("ff", minimum=1))


@dataclass(frozen=True)
class MuneraxConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    bigram: Optional[MuneraxBigram]
    layers: Tuple[MuneraxLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...]

    @classmethod
    def from_dict(cls, data: Dict[str, Any], what: str = "config.json") -> "MuneraxConfig":
        r = ConfigReader(data, what)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        scale, bigram = 1.0, None
        emb = _sub(r, "embedding", required=False)
        if emb is not None:
            scale = emb.number("scale", default=1.0)
            b = _sub(emb, "bigram", required=False)
            if b is not None:
                bigram = MuneraxBigram(buckets=b.integer("buckets", minimum=1), mul_prev=b.integer("mul_prev", minimum=0),
                                       mul_cur=b.integer("mul_cur", minimum=0))
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{what}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = ConfigReader(entry, f"{what}: layers[{i}]")
            kind = lr.string("type")
            if kind != "latent_attention":
                raise ConfigError(f"{lr.what}: key 'type' must be \"latent_attention\", got {kind!r}")
            m = _latent(_sub(lr, "mixer"), i)
            if m.kv_from is not None:
                src = layers[m.kv_from].mixer
                if src.kv_from is not None:
                    raise ConfigError(f"{lr.what}: layer {m.kv_from}, whose cache it reads, keeps none of its own")
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                    raise ConfigError(f"{lr.what}: kv_rank, rot_dim and rotation must equal those of layer {m.kv_from}, "
                                      "whose cache it reads")
            mr = _sub(lr, "mlp", required=False)
            layers.append(MuneraxLayer(type=kind, mixer=m, mlp=None if mr is None else _mlp(mr)))
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, bigram=bigram, layers=tuple(layers),
                   max_positions=r.integer("max_positions", default=0, minimum=0),
                   eos_token_ids=tuple(r.int_or_list("eos_token_id")))
