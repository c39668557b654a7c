"""Shared by the Munerax tests: small configurations with sizes of their own, weights made here
(larger than the package's random fill, so that softmaxes are sharp, sinks matter and routers
decide), and model folders written from them."""
import json
import math
import os
import struct
import tempfile

import torch

F32, BF16 = torch.float32, torch.bfloat16


def lat(heads, dim, rot_dim, vdim, rank, scale, rot=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale, count=None, keep=None, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if count:
        m["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# odd sizes everywhere: head counts 1 to 4, a latent narrower and wider than a head, a rotated part
# that is turned whole and one of which only the first values turn, value heads narrower and wider
# than the keys, two layers with caches of their own and three that borrow (one from each, and one
# borrows what an earlier borrower already reads), a layer without feed-forward, dense layers first
# and last, a router with groups of two that keeps 2 of 3, one without groups and top 1, and a
# feed-forward without shared expert
MX_ODD = {"architecture": "Munerax", "vocab": 131, "width": 40, "norm": {"eps": 2e-5},
          "embedding": {"scale": 3.7, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 13}},
          "layers": [
              layer(lat(3, 10, 6, 12, 14, 0.21, (100.0, 6)), dense(24)),
              layer(lat(2, 8, 6, 5, 14, 0.3, (100.0, 6), kv_from=0), moe(6, 3, 20, 1.5, 3, 2, 12)),
              layer(lat(4, 16, 8, 16, 24, 0.17, (5e4, 4)), None),
              layer(lat(1, 12, 8, 30, 24, 0.25, (5e4, 4), kv_from=2), moe(5, 1, 16, 0.8)),
              layer(lat(3, 6, 6, 8, 14, 0.4, (100.0, 6), kv_from=0), dense(56))]}
# sizes nearer to a served model's: a cache row of 96 and of 160 values, heads of 48 + 32 and 64 + 32
MX_WIDE = {"architecture": "Munerax", "vocab": 300, "width": 128, "norm": {"eps": 1e-6},
           "embedding": {"scale": 11.3, "bigram": {"buckets": 211, "mul_prev": 29, "mul_cur": 3}},
           "layers": [
               layer(lat(5, 48, 32, 40, 64, 0.11, (1e6, 32)), moe(8, 2, 64, 2.5, 4, 2, 128)),
               layer(lat(8, 64, 32, 64, 128, 0.1, (1e4, 32)), dense(192)),
               layer(lat(4, 32, 32, 64, 64, 0.125, (1e6, 32), kv_from=0), moe(12, 3, 48, 1.0, 3, 2, 64))]}
CONFIGS = {"odd": MX_ODD, "wide": MX_WIDE}


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a Munerax model, from its config alone."""
    w = cfg["width"]
    out = {"embed": ((cfg["vocab"], w), "table"), "final.norm": ((w,), "norm")}
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        out["bigram"] = ((big["buckets"] + 1, w), "table")
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        a, d, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out[p + "norm1"] = ((w,), "norm")
        out.update({p + "mix.q": ((a * (d + rd), w), "matrix"), p + "mix.uk": ((a * d, r), "matrix"),
                    p + "mix.uv": ((a * dv, r), "matrix"), p + "mix.sink": ((a,), "sink"), p + "mix.g": ((a, w), "gate"),
                    p + "mix.o": ((w, a * dv), "matrix")})
        if "kv_from" not in m:
            out.update({p + "mix.dkv": ((r + rd, w), "matrix"), p + "mix.dkv.norm": ((r,), "norm")})
        f = lay.get("mlp")
        if f:
            q = p + "mlp."
            out[p + "norm2"] = ((w,), "norm")
            if f["kind"] == "dense":
                out.update({q + "gate": ((f["ff"], w), "matrix"), q + "up": ((f["ff"], w), "matrix"), q + "down": ((w, f["ff"]), "matrix")})
            else:
                out[q + "router"] = ((f["router"]["experts"], w), "router")
                ff = f["expert"]["ff"]
                for e in range(f["router"]["experts"]):
                    out.update({f"{q}e{e}.up": ((ff, w), "matrix"), f"{q}e{e}.down": ((w, ff), "matrix")})
                if f.get("shared"):
                    out.update({q + "shared.up": ((f["shared"]["ff"], w), "matrix"), q + "shared.down": ((w, f["shared"]["ff"]), "matrix")})
    return out


def make_weights(cfg, seed, dt, steady=False):
    """``steady``: milder matrices, for the bfloat16 models (a rounding error is amplified where
    softmaxes and gates are sharp)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g)
        if kind == "norm":
            t = 1.0 + 0.2 * t
        elif kind == "table":
            t = 0.7 * t
        elif kind == "sink":
            t = 1.5 * t
        elif kind == "gate":
            t = t * (2.0 / math.sqrt(shape[1]))
        elif kind == "router":
            t = t * (3.0 / math.sqrt(shape[1]))
        else:
            t = t * ((1.0 if steady else 1.6) / math.sqrt(shape[1]))
        out[name] = t.to(dt)
    return out


def write_folder(cfg, weights):
    folder = tempfile.mkdtemp(prefix="bfi_munerax_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != BF16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": {F32: "F32", BF16: "BF16"}[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder


_MODELS = {}


def model(name, dtype, seed=3):
    """(folder, config, float64 weights as stored) of a test model; the store is the run dtype's."""
    key = (name, dtype, seed)
    if key not in _MODELS:
        cfg = CONFIGS[name]
        w = make_weights(cfg, seed, F32 if dtype == "float32" else BF16, steady=dtype != "float32")
        _MODELS[key] = (write_folder(cfg, w), cfg, {k: v.to(torch.float64) for k, v in w.items()})
    return _MODELS[key]


def prompts(vocab, lengths, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def _divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def random_config(seed):
    """A configuration drawn from a seed: two to six layers, each with a cache of its own or
    borrowing an earlier owner's, sizes from lists that hold odd ones and values that make other
    sizes equal or 1, rotation over the whole rotated part, a part of it or none, routers with and
    without groups (also groups of one expert), layers with a dense, a routed or no feed-forward,
    with and without a shared expert, with and without the bigram table."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 96, 160, 256])
    layers, owners = [], []
    for i in range(rng.randint(2, 6)):
        heads, dim, vdim = rng.choice([1, 2, 3, 4, 6, 8]), rng.choice([4, 8, 16, 24, 32, 64]), rng.choice([4, 8, 16, 32, 40, 64])
        if owners and rng.random() < 0.5:
            src = rng.choice(owners)
            sm = layers[src]["mixer"]
            mixer = lat(heads, dim, sm["rot_dim"], vdim, sm["kv_rank"], rng.choice([0.05, 0.125, 0.3]),
                        (sm["rot"]["base"], sm["rot"]["dims"]) if "rot" in sm else None, kv_from=src)
        else:
            rot_dim = rng.choice([0, 2, 8, 16, 32, 64])
            rank = rng.choice([2, 8, 16, 24, 64, 128, 192])
            rot = (rng.choice([100.0, 1e4, 1e6]), rng.choice(list(range(2, rot_dim + 1, 2)) + [rot_dim] * 3)) if rot_dim else None
            mixer = lat(heads, dim, rot_dim, vdim, rank, rng.choice([0.05, 0.125, (dim + rot_dim) ** -0.5, 0.3]), rot)
            owners.append(i)
        kind = rng.random()
        mlp = None
        if kind < 0.3:
            mlp = dense(rng.choice([8, 20, 64, 100]))
        elif kind < 0.9:
            experts = rng.choice([2, 4, 6, 8, 12, 16, 32])
            count = rng.choice(_divisors(experts))
            keep = rng.randint(1, count)
            top = rng.randint(1, min(keep * (experts // count), 6))
            mlp = moe(experts, top, rng.choice([8, 20, 32, 64, 72]), rng.choice([0.5, 1.0, 2.5]),
                      count if rng.random() < 0.8 else None, keep, rng.choice([None, 16, 40, 96]))
            if "groups" not in mlp["router"]:
                mlp["router"]["top"] = min(top, experts)
        layers.append(layer(mixer, mlp))
    vocab = rng.choice([97, 256, 333, 1000])
    emb = {"scale": rng.choice([1.0, 0.5, math.sqrt(width)])}
    if rng.random() < 0.8:
        emb["bigram"] = {"buckets": rng.choice([1, 2, 31, 257, 1024]), "mul_prev": rng.choice([0, 1, 31, 1009]),
                         "mul_cur": rng.choice([0, 1, 17, 65537])}
    return {"architecture": "Munerax", "vocab": vocab, "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5])},
            "embedding": emb, "layers": layers}
