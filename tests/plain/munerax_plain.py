"""A plain, slow implementation of the Munerax design: whole sequences, no cache, float64, one
function per mechanism, written from the design's equations and sharing nothing with the
package.  The tests compare the package's kernels, parts and engine with it.

Notation: ``x`` is the residual stream ``[T, width]``; ``h`` a normed copy of it; linear weights
are ``[out, in]`` and act as ``W x``; ``w[name]`` is a tensor of the checkpoint.

The input is ``embed[token] * scale + bigram[bucket(previous token, token)]``.  A layer is
``x += mixer(norm1(x))``, then ``x += ff(norm2(x))``; the mixer is latent attention (keys and values
of all heads are made from one small vector per token, which a later layer may borrow), the
feed-forward a dense gated one or a routed one.  The logits are ``embed @ norm(x)``.
"""
import json
import math
import os
import struct

import torch

F = torch.float64


# ------------------------------------------------------------------------------- files
def read_tensors(path):
    """name -> tensor of a safetensors file (8-byte length, JSON header, raw data)."""
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(F) if t.is_floating_point() else t
    return out


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------------------- small functions
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def rms(x, eps):
    """x divided by its root mean square over the last dimension; eps sits inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, weight, eps):
    return rms(x, eps) * weight


# ------------------------------------------------------------------------------- input
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """The row of the bigram table for every token: a hash of (previous token, token), and the
    table's last row (number ``buckets``) for a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(w, cfg, tokens):
    e = cfg.get("embedding") or {}
    x = w["embed"][list(tokens)] * float(e.get("scale", 1.0))
    b = e.get("bigram")
    if b:
        x = x + w["bigram"][bigram_rows(list(tokens), b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x


# ------------------------------------------------------------------------------- rotary
def rotate_half(x, positions, base, dims):
    """x [T, heads, d].  Of each head's first ``dims`` values, value i (i < dims/2) and value
    i + dims/2 form a pair that turns by the angle position * base^(-2i/dims); the rest pass."""
    if not dims:
        return x.clone()
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = torch.tensor(float(base), dtype=F) ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------- latent attention
def latent_of(w, p, m, h, eps):
    """What a layer with a down projection of its own keeps per token: the normed latent ``c``
    ``[T, kv_rank]`` and the rotated key part ``[T, rot_dim]`` that all heads share."""
    T = h.shape[0]
    r, rd = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = norm(d[:, :r], w[p + "dkv.norm"], eps)
    kr = d[:, r:r + rd].reshape(T, 1, rd)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    kr = rotate_half(kr, range(T), rot["base"], rot.get("dims", rd)).reshape(T, rd)
    return c, kr


def sink_softmax(scores, sink):
    """Causal softmax over each row of ``scores`` [T, T] whose denominator also holds exp(sink)."""
    T = scores.shape[0]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    s = scores.masked_fill(~mask, -math.inf)
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, torch.as_tensor(sink, dtype=F))
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))


def latent_attention(w, p, m, h, eps, latent):
    """h [T, width] -> [T, width].  ``latent`` is (c, rotated key part) of this layer or of the
    layer it borrows from."""
    T = h.shape[0]
    H, d, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = latent
    q = (h @ w[p + "q"].T).reshape(T, H, d + rd)
    qn = q[..., :d]
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    qr = rotate_half(q[..., d:], range(T), rot["base"], rot.get("dims", rd))
    kn = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        scores = (qn[:, a] @ kn[:, a].T + qr[:, a] @ kr.T) * float(m["scale"])
        out[:, a] = sink_softmax(scores, w[p + "sink"][a]) @ v[:, a]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------------- feed-forward
def dense_ff(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(w, p, h):
    return relu_squared(h @ w[p + "up"].T) @ w[p + "down"].T


def route(z, top, count, keep, scale, margins=None):
    """Router logits z [T, E] -> (chosen experts [T, top], their weights [T, top]).  Scores are
    sigmoid(z); a group's score is the sum of its two largest; experts outside the ``keep`` best
    groups cannot be chosen; the weights are the chosen scores times ``scale``.  ``margins`` (a list)
    receives, per token, by how much the last group kept and the last expert chosen won."""
    T, E = z.shape
    s = torch.sigmoid(z)
    allowed = torch.ones(T, E, dtype=torch.bool)
    gap = torch.full((T,), math.inf, dtype=F)
    if count > 1 and keep < count:
        per = E // count
        g = s.reshape(T, count, per)
        gs = g.topk(min(2, per), dim=-1).values.sum(dim=-1)    # [T, count]
        order = gs.sort(dim=-1, descending=True)
        gap = order.values[:, keep - 1] - order.values[:, keep]
        ok = torch.zeros(T, count, dtype=torch.bool)
        ok.scatter_(1, order.indices[:, :keep], True)
        allowed = ok[:, :, None].expand(T, count, per).reshape(T, E)
    order = s.masked_fill(~allowed, -math.inf).sort(dim=-1, descending=True)
    if top < E:
        gap = torch.minimum(gap, order.values[:, top - 1] - order.values[:, top])
    if margins is not None:
        margins.extend(float(v) for v in gap)
    pick = order.indices[:, :top]
    return pick, s.gather(1, pick) * scale


def routed_ff(w, p, f, h, margins=None):
    r = f["router"]
    groups = r.get("groups") or {}
    count = groups.get("count", 1)
    z = h @ w[p + "router"].T
    pick, weight = route(z, r["top"], count, groups.get("keep", count), float(r.get("scale", 1.0)), margins)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for k in range(r["top"]):
            e = int(pick[t, k])
            out[t] += weight[t, k] * expert(w, f"{p}e{e}.", h[t:t + 1])[0]
    if f.get("shared"):
        out = out + expert(w, p + "shared.", h)
    return out


# ------------------------------------------------------------------------------- the model
def forward_layers(w, cfg, tokens, margins=None):
    """The residual stream after every layer, [layers, T, width].  ``margins`` (a list) receives by
    how much every routing decision was won."""
    eps = float(cfg["norm"]["eps"])
    x = embed(w, cfg, tokens)
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = norm(x, w[p + "norm1"], eps)
        src = m.get("kv_from")
        if src is None:
            kept[i] = latent_of(w, p + "mix.", m, h, eps)
            src = i
        x = x + latent_attention(w, p + "mix.", m, h, eps, kept[src])
        f = layer.get("mlp")
        if f is not None:
            h = norm(x, w[p + "norm2"], eps)
            x = x + (dense_ff(w, p + "mlp.", h) if f.get("kind", "dense") == "dense" else routed_ff(w, p + "mlp.", f, h, margins))
        after.append(x.clone())
    return torch.stack(after)


def forward_each(w, cfg, tokens, margins=None):
    """Logits [T, vocab] at every position of ``tokens``."""
    x = forward_layers(w, cfg, tokens, margins)[-1]
    return norm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ w["embed"].T
