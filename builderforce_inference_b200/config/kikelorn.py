"""``KikelornConfig``: the sizes and constants of a Kikelorn decoder, read from its config.json.

A Kikelorn model is a stack of blocks that norm each sublayer's OUTPUT (the sublayers read the
residual stream itself, through a short causal convolution over time, and their result passes a
sigmoid gate made from the residual stream before the norm).  The mixer of a layer is chunked
grouped-query attention with short convolutions on q, k and v, latent attention whose queries go
through a latent too, or a minGRU; the feed-forward, where a layer has one, is a dense one with
biases and the tanh GELU.  config.json carries:

    architecture            "Kikelorn"
    vocab, width            vocabulary size, residual width
    norm.eps                epsilon of every RMS norm
    embedding.scale         factor on the token embedding (default 1; the tied head does not take it)
    residual_mult           factor on every normed sublayer output as it is added (default 1)
    canon.taps              taps of the convolution in front of every sublayer
    layers[i].type          "attention" | "latent_attention" | "mingru"
    layers[i].mixer         attention: heads, kv_heads, dim, vdim, conv (taps), scale, mask.size,
                                       rot.{base, dims, scaling?}, v_mix
                            latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                       rot.{base, dims, scaling.{factor, original, fast, slow}?}
                            mingru: width
    layers[i].mlp           null or {kind: "dense", ff}

Every value is checked here, so a bad folder fails by key before any weight is read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ConfigReader
from .datasun import _sub

MAX_TAPS = 16       # the convolution kernels keep a token's taps in registers


@dataclass(frozen=True)
class KikelornRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]      # sorted (name, value) pairs of factor, original, fast, slow

    def scaling_dict(self) -> Optional[Dict[str, float]]:
        return None if self.scaling is None else dict(self.scaling)


@dataclass(frozen=True)
class KikelornAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                   # taps of the convolution on q, k and v (1: a factor per channel)
    scale: float
    chunk: int
    rot: Optional[KikelornRotation]
    v_mix: bool


@dataclass(frozen=True)
class KikelornLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Optional[KikelornRotation]


@dataclass(frozen=True)
class KikelornMinGRU:
    width: int


@dataclass(frozen=True)
class KikelornDense:
    ff: int


@dataclass(frozen=True)
class KikelornLayer:
    type: str
    mixer: Any                  # KikelornAttention, KikelornLatent or KikelornMinGRU
    mlp: Optional[KikelornDense]


def _rotation(r: ConfigReader, limit: int, default_dims: int) -> Optional[KikelornRotation]:
    rot = _sub(r, "rot", required=False)
    if rot is None or limit < 2:
        return None
    dims = rot.integer("dims", default=default_dims, minimum=2)
    if dims % 2 != 0 or dims > limit:
        raise ConfigError(f"{rot.what}: key 'dims' must be even and at most {limit}, got {dims}")
    base = rot.number("base", positive=True)
    scaling = None
    sc = _sub(rot, "scaling", required=False)
    if sc is not None:
        if not base > 1.0:
            raise ConfigError(f"{rot.what}: frequency scaling needs a base above 1, got {base}")
        scaling = tuple(sorted((k, sc.number(k, positive=True)) for k in ("factor", "original", "fast", "slow")))
    return KikelornRotation(base=base, dims=dims, scaling=scaling)


def _taps(r: ConfigReader, key: str) -> int:
    taps = r.integer(key, minimum=1)
    if taps > MAX_TAPS:
        raise ConfigError(f"{r.what}: key '{key}' must be at most {MAX_TAPS}, got {taps}")
    return taps


def _attention(r: ConfigReader) -> KikelornAttention:
    heads = r.integer("heads", minimum=1)
    kv_heads = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv_heads != 0:
        raise ConfigError(f"{r.what}: {heads} heads do not divide into {kv_heads} kv_heads")
    dim = r.integer("dim", minimum=2)
    if dim % 2 != 0 or dim > 512:
        raise ConfigError(f"{r.what}: key 'dim' must be even and at most 512, got {dim}")
    vdim = r.integer("vdim", default=dim, minimum=1)
    if vdim > 512:
        raise ConfigError(f"{r.what}: key 'vdim' must be at most 512, got {vdim}")
    mask = _sub(r, "mask")
    return KikelornAttention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=_taps(r, "conv"),
                             scale=r.number("scale", default=dim ** -0.5, positive=True),
                             chunk=mask.integer("size", minimum=1), rot=_rotation(r, dim, dim),
                             v_mix=r.boolean("v_mix", default=False))


def _latent(r: ConfigReader) -> KikelornLatent:
    heads = r.integer("heads", minimum=1)
    dim = r.integer("dim", minimum=1)
    rot_dim = r.integer("rot_dim", default=0, minimum=0)
    rank = r.integer("kv_rank", minimum=1)
    if (rank + rot_dim) % 2 != 0 or rank + rot_dim > 1024 or rank > 512:
        raise ConfigError(f"{r.what}: kv_rank = {rank} must be at most 512, kv_rank + rot_dim = {rank + rot_dim} even and at most 1024")
    return KikelornLatent(heads=heads, dim=dim, rot_dim=rot_dim, vdim=r.integer("vdim", default=dim, minimum=1), kv_rank=rank,
                          q_rank=r.integer("q_rank", minimum=1),
                          scale=r.number("scale", default=(dim + rot_dim) ** -0.5, positive=True),
                          rot=_rotation(r, rot_dim, rot_dim))


@dataclass(frozen=True)
class KikelornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    canon_taps: int
    layers: Tuple[KikelornLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...]

    @classmethod
    def from_dict(cls, data: Dict[str, Any], what: str = "config.json") -> "KikelornConfig":
        r = ConfigReader(data, what)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        emb = _sub(r, "embedding", required=False)
        scale = 1.0 if emb is None else emb.number("scale", default=1.0)
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{what}: key 'layers' must be a non-empty list")
        layers, mixing = [], None
        for i, entry in enumerate(raw_layers):
            lr = ConfigReader(entry, f"{what}: layers[{i}]")
            kind = lr.string("type")
            mr = _sub(lr, "mixer")
            if kind == "attention":
                m = _attention(mr)
                if m.v_mix:
                    if mixing is not None and (mixing.kv_heads, mixing.vdim) != (m.kv_heads, m.vdim):
                        raise ConfigError(f"{lr.what}: layers that mix values must agree on kv_heads and vdim")
                    mixing = mixing or m
            elif kind == "latent_attention":
                m = _latent(mr)
            elif kind == "mingru":
                m = KikelornMinGRU(width=mr.integer("width", minimum=1))
            else:
                raise ConfigError(f"{lr.what}: key 'type' must be \"attention\", \"latent_attention\" or \"mingru\", got {kind!r}")
            fr = _sub(lr, "mlp", required=False)
            mlp = None
            if fr is not None:
                ff_kind = fr.string("kind", default="dense")
                if ff_kind != "dense":
                    raise ConfigError(f"{fr.what}: key 'kind' must be \"dense\", got {ff_kind!r}")
                mlp = KikelornDense(ff=fr.integer("ff", minimum=1))
            layers.append(KikelornLayer(type=kind, mixer=m, mlp=mlp))
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale,
                   residual_mult=r.number("residual_mult", default=1.0), canon_taps=_taps(_sub(r, "canon"), "taps"),
                   layers=tuple(layers), max_positions=r.integer("max_positions", default=0, minimum=0),
                   eos_token_ids=tuple(r.int_or_list("eos_token_id")))
