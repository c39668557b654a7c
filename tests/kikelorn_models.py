"""Shared by the Kikelorn tests: small configurations with sizes of their own, weights made here
(larger than the package's random fill, so that softmaxes are sharp and gates matter), and model
folders written from them."""
import json
import math
import os
import struct
import tempfile

import torch

F32, BF16 = torch.float32, torch.bfloat16


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def att(heads, kv_heads, dim, vdim, conv, scale, chunk, r=None, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
         "mask": {"size": chunk}, "v_mix": v_mix}
    if r:
        m["rot"] = r
    return {"type": "attention", "mixer": m}


def lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, r=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if r:
        m["rot"] = r
    return {"type": "latent_attention", "mixer": m}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def config(vocab, width, eps, scale, mult, taps, layers):
    return {"architecture": "Kikelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "residual_mult": mult, "canon": {"taps": taps}, "layers": layers}


# odd sizes everywhere: the recurrent layer first, a latent layer whose rotated part turns only in its
# first values and one without frequency scaling, attention layers of different head counts and head
# sizes (as many key heads as query heads in two, a third as many in another), values wider and narrower
# than the keys, chunks of 24 and 50 positions (neither divides a page of 64), convolutions of 2, 3
# and 5 taps, three mixing layers of which the first is not the model's first attention layer, a
# layer without feed-forward, two taps in front of the sublayers
KK_ODD = config(137, 40, 2e-5, 3.3, 0.6, 2, [
    with_mlp(gru(56), 24),
    with_mlp(att(3, 3, 10, 6, 3, 0.31, 24, rot(100.0, 6)), 36),
    with_mlp(lat(3, 10, 6, 12, 14, 10, 0.23, rot(1e4, 4, (3.0, 64, 16.0, 2.0))), None),
    with_mlp(att(4, 2, 8, 12, 2, 0.35, 50, rot(1e4, 8), v_mix=True), 20),
    with_mlp(lat(2, 6, 8, 5, 24, 18, 0.3, rot(5e3, 8)), 44),
    with_mlp(att(6, 2, 12, 12, 5, 0.28, 24, rot(500.0, 4, (2.0, 32, 8.0, 1.0)), v_mix=True), 16),
    with_mlp(att(2, 2, 16, 12, 3, 0.25, 50, None, v_mix=True), None),
])
# sizes nearer to a served model's: multiples of 16 throughout, keys and values of one size in one
# attention layer (the tensor-core prompt kernel's case), four taps in front of the sublayers, one
# tap on q, k and v in one layer
KK_WIDE = config(300, 128, 1e-6, 11.0, 0.8, 4, [
    with_mlp(att(4, 2, 64, 64, 4, 0.125, 96, rot(1e4, 32), v_mix=True), 192),
    with_mlp(lat(4, 32, 32, 32, 64, 48, 0.125, rot(1e5, 32, (4.0, 128, 32.0, 1.0))), 128),
    with_mlp(gru(192), 256),
    with_mlp(att(8, 2, 32, 64, 1, 0.18, 200, rot(1e6, 16), v_mix=True), 64),
    with_mlp(lat(8, 64, 16, 64, 128, 96, 0.11, rot(1e4, 16)), 192),
])
CONFIGS = {"odd": KK_ODD, "wide": KK_WIDE}


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a Kikelorn model, from its config alone."""
    w, taps = cfg["width"], cfg["canon"]["taps"]
    out = {"embed": ((cfg["vocab"], w), "table"), "final.norm": ((w,), "norm")}
    for i, lay in enumerate(cfg["layers"]):
        p, m, q = f"l{i}.", lay["mixer"], f"l{i}.mix."
        subs = ("1", "2") if lay.get("mlp") else ("1",)
        for s in subs:
            out.update({p + "norm" + s: ((w,), "norm"), p + "canon" + s: ((w, taps), "conv"),
                        p + "rg" + s: ((w, w), "gate"), p + "rg" + s + ".b": ((w,), "bias")})
        if lay["type"] == "attention":
            a, g, d, dv, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            out.update({q + "q": ((a * d, w), "matrix"), q + "k": ((g * d, w), "matrix"), q + "v": ((g * dv, w), "matrix"),
                        q + "q.norm": ((a * d,), "norm"), q + "k.norm": ((g * d,), "norm"),
                        q + "q.conv": ((a * d, t), "conv1"), q + "k.conv": ((g * d, t), "conv1"), q + "v.conv": ((g * dv, t), "conv1"),
                        q + "g": ((a, w), "gate"), q + "o": ((w, a * dv), "matrix")})
            if m.get("v_mix"):
                out[q + "vmix"] = ((), "mix")
        elif lay["type"] == "latent_attention":
            a, d, rd, dv, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({q + "dq": ((qr, w), "matrix"), q + "dq.norm": ((qr,), "norm"), q + "uq": ((a * (d + rd), qr), "matrix"),
                        q + "dkv": ((r + rd, w), "matrix"), q + "dkv.norm": ((r,), "norm"), q + "uk": ((a * d, r), "matrix"),
                        q + "uv": ((a * dv, r), "matrix"), q + "g": ((a * dv, w), "gate"), q + "o": ((w, a * dv), "matrix")})
        else:
            n = m["width"]
            out.update({q + "z": ((n, w), "gate"), q + "z.b": ((n,), "bias"), q + "x": ((n, w), "matrix"), q + "x.b": ((n,), "bias"),
                        q + "g": ((n, w), "matrix"), q + "o": ((w, n), "matrix")})
        if lay.get("mlp"):
            ff = lay["mlp"]["ff"]
            out.update({p + "mlp.up": ((ff, w), "matrix"), p + "mlp.up.b": ((ff,), "bias"),
                        p + "mlp.down": ((w, ff), "matrix"), p + "mlp.down.b": ((w,), "bias")})
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
        elif kind == "bias":
            t = 0.5 * t
        elif kind == "mix":
            t = 0.3 + 0.2 * torch.rand(shape, generator=g)
        elif kind == "conv":        # in front of a sublayer: a correction of the input
            t = t * (0.5 / math.sqrt(shape[1]))
        elif kind == "conv1":       # on q, k, v: the last tap weighs the token itself
            t = t * 0.4
            t[..., -1] += 1.0
        elif kind == "gate":
            t = t * (2.0 / math.sqrt(shape[1]))
        else:
            t = t * ((1.0 if steady else 1.6) / math.sqrt(shape[1]))
        out[name] = t.to(dt)
    return out


def write_folder(cfg, weights):
    folder = tempfile.mkdtemp(prefix="bfi_kikelorn_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        flat = t.contiguous().reshape(-1)       # a tensor may have no dimensions at all
        raw = flat.view(torch.int16 if t.dtype == BF16 else torch.int32).numpy().tobytes()
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


def random_config(seed):
    """A configuration drawn from a seed: two to six layers of the three kinds in any order, sizes
    from lists that hold odd ones and values that make other sizes equal or 1, rotation over a whole
    head, a part of it or none, with and without frequency scaling, chunks from 1 position to more
    than the prompts, 1 to 6 taps, mixing layers or none, layers with and without feed-forward."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 48, 64, 96, 160])
    mix_shape = (rng.choice([1, 2, 4]), rng.choice([4, 8, 20, 32]))       # kv_heads and vdim of the layers that mix values
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(["attention", "latent_attention", "mingru"])
        if kind == "attention":
            mixes = rng.random() < 0.6
            g, dv = mix_shape if mixes else (rng.choice([1, 2, 3]), rng.choice([2, 8, 16, 40]))
            a = g * rng.choice([1, 2, 4])
            d = rng.choice([2, 8, 16, 32, 64])
            r = None
            if rng.random() < 0.85:
                dims = rng.choice(list(range(2, d + 1, 2)) + [d] * 3)
                sc = (rng.choice([2.0, 4.0, 8.0]), rng.choice([16, 64, 256]), rng.choice([8.0, 32.0]), rng.choice([1.0, 2.0])) \
                    if rng.random() < 0.3 else None
                r = rot(rng.choice([100.0, 1e4, 1e6]), dims, sc)
            lay = att(a, g, d, dv, rng.randint(1, 6), rng.choice([0.1, d ** -0.5, 0.4]), rng.choice([1, 2, 7, 64, 100, 128, 1000]), r, mixes)
        elif kind == "latent_attention":
            rd = rng.choice([0, 2, 8, 16, 32])
            r = None
            if rd and rng.random() < 0.9:
                sc = (rng.choice([2.0, 8.0]), rng.choice([32, 1024]), rng.choice([16.0, 24.0]), 1.0) if rng.random() < 0.6 else None
                r = rot(rng.choice([1e3, 3e5]), rd, sc)
            d = rng.choice([4, 8, 16, 32])
            lay = lat(rng.choice([1, 2, 3, 4, 8]), d, rd, rng.choice([4, 8, 16, 32, 40]), rng.choice([2, 8, 16, 24, 64, 128]),
                      rng.choice([1, 6, 16, 48]), rng.choice([0.1, (d + rd) ** -0.5, 0.3]), r)
        else:
            lay = gru(rng.choice([1, 8, 33, 64, 100]))
        layers.append(with_mlp(lay, rng.choice([None, 8, 20, 64, 100])))
    return config(rng.choice([97, 256, 333]), width, rng.choice([1e-6, 1e-5]), rng.choice([1.0, 0.5, math.sqrt(width)]),
                  rng.choice([1.0, 0.7, 0.25]), rng.randint(1, 5), layers)
