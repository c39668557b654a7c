"""A plain, slow implementation of the Kikelorn design: whole sequences, no cache, float64, one
function per mechanism, written from the design's equations and sharing nothing with the
package.  The tests compare the package's kernels, parts and engine with it.

Notation: ``x`` is the residual stream ``[T, width]``; linear weights are ``[out, in]`` and act as
``W x``; ``w[name]`` is a tensor of the checkpoint; ``m`` is the residual multiplier.

The input is ``embed[token] * scale``.  A layer runs two sublayers, the mixer and (where the layer
has one) the feed-forward, each in the same arrangement around the residual stream:

    h   = x + conv(x)                      a causal convolution over time per channel ("canon")
    y   = sublayer(h) * sigmoid(W_rg x + b_rg)
    x  += m * norm(y)

The mixer is chunked attention with short convolutions on q, k, v, latent attention with a query
latent, or a minGRU; the feed-forward is ``W_down gelu_tanh(W_up h + b_up) + b_down``.  The logits
are ``embed @ norm(x)``.
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


def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    """x divided by its root mean square over the last dimension; eps sits inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, weight, eps):
    return rms(x, eps) * weight


def causal_conv(u, taps_w):
    """``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` per channel, zeros before the first row.
    ``u`` is ``[T, C]``, ``taps_w`` ``[C, taps]``; the last tap multiplies the row itself."""
    T, C = u.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y


# ------------------------------------------------------------------------------- rotation
def rotary_angles(positions, dims, base, scaling=None):
    """cos and sin ``[T, dims/2]`` of ``p * f_i``, ``f_i = base^(-2i/dims)``, with the frequencies
    slowed down and the magnitudes raised where ``scaling`` (factor, original, fast, slow) says so."""
    i = torch.arange(dims // 2, dtype=F)
    f = float(base) ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def dim_of(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    a = torch.tensor(list(positions), dtype=F)[:, None] * f[None, :]
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate(v, cos, sin, dims, layout):
    """Turn the first ``dims`` values of every head of ``v`` ``[T, heads, d]``.  ``layout`` "half":
    value i pairs with value i + dims/2; "interleaved": value 2i with value 2i + 1."""
    out = v.clone()
    half = dims // 2
    if layout == "half":
        a, b = v[..., :half], v[..., half:dims]
    else:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    ra, rb = a * c - b * s, b * c + a * s
    if layout == "half":
        out[..., :half], out[..., half:dims] = ra, rb
    else:
        out[..., 0:dims:2], out[..., 1:dims:2] = ra, rb
    return out


# ------------------------------------------------------------------------------- softmax attention
def masked_attention(q, k, v, scale, visible):
    """``q`` ``[T, H, d]``, ``k`` ``[T, H, d]``, ``v`` ``[T, H, dv]``; ``visible(i, j)`` says whether
    token i sees token j.  Returns ``[T, H, dv]``."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=F)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j)]
        for a in range(H):
            s = torch.stack([(q[i, a] * k[j, a]).sum() for j in js]) * scale
            p = torch.softmax(s, dim=0)
            out[i, a] = (p[:, None] * v[js, a]).sum(dim=0)
    return out


def fast_masked_attention(q, k, v, scale, mask):
    """The same with a boolean mask ``[T, T]`` and matrix products (for long sequences)."""
    s = torch.einsum("iad,jad->aij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("aij,jad->iad", p, v)


def chunk_mask(T, size):
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def causal_mask(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


# ------------------------------------------------------------------------------- mixers
def chunked_attention(w, p, mc, h, eps, v_first, is_first):
    """Grouped-query attention within chunks of ``mask.size`` positions.  Returns the mixer's output
    and the values it used (what a later layer mixes in when this is the first mixing layer)."""
    T = h.shape[0]
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q, k = norm(q, w[p + "q.norm"], eps), norm(k, w[p + "k.norm"], eps)
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    rot = mc.get("rot")
    if rot:
        cos, sin = rotary_angles(range(T), rot["dims"], rot["base"], rot.get("scaling"))
        q, k = rotate(q, cos, sin, rot["dims"], "half"), rotate(k, cos, sin, rot["dims"], "half")
    if mc.get("v_mix") and not is_first:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    o = fast_masked_attention(q, kk, vv, mc["scale"], chunk_mask(T, mc["mask"]["size"]))
    gate = torch.sigmoid(h @ w[p + "g"].T)                 # one number per head
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T, v


def latent_attention(w, p, mc, h, eps):
    """Queries through a normed latent; keys and values of all heads from one normed latent and one
    rotated key part that the heads share; causal softmax; a gate per output value."""
    T = h.shape[0]
    H, d, rd, dv, r = mc["heads"], mc["dim"], mc["rot_dim"], mc["vdim"], mc["kv_rank"]
    cq = norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, d + rd)
    q_n, q_r = q[..., :d], q[..., d:]
    kv = h @ w[p + "dkv"].T
    c = norm(kv[:, :r], w[p + "dkv.norm"], eps)
    k_r = kv[:, r:].view(T, 1, rd)
    k_n = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    rot = mc.get("rot")
    if rot:
        cos, sin = rotary_angles(range(T), rot["dims"], rot["base"], rot.get("scaling"))
        q_r, k_r = rotate(q_r, cos, sin, rot["dims"], "interleaved"), rotate(k_r, cos, sin, rot["dims"], "interleaved")
    qq = torch.cat([q_n, q_r], dim=-1)
    kk = torch.cat([k_n, k_r.expand(T, H, rd)], dim=-1)
    o = fast_masked_attention(qq, kk, v, mc["scale"], causal_mask(T)).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mingru_candidate(u):
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru(w, p, h):
    """``S_t = (1 - z_t) S_(t-1) + z_t cand_t`` per channel from a zero state; the output is
    ``W_o (S_t * silu(W_g h_t))``."""
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    cand = mingru_candidate(h @ w[p + "x"].T + w[p + "x.b"])
    S = torch.zeros(z.shape[1], dtype=F)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S)
    return (torch.stack(rows) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(w, p, h):
    return gelu_tanh(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


# ------------------------------------------------------------------------------- the model
def sublayer_step(w, cfg, x, layer, which, fn):
    """One sublayer in the arrangement of the module's header; ``which`` is "1" (mixer) or "2"."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    h = x + causal_conv(x, w[f"{layer}canon{which}"])
    y = fn(h) * torch.sigmoid(x @ w[f"{layer}rg{which}"].T + w[f"{layer}rg{which}.b"])
    return x + m * norm(y, w[f"{layer}norm{which}"], eps)


def forward(cfg, w, tokens, keep_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and, when asked, the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][list(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    v_first = None
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, mc = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            state = {}

            def mixer(h, mc=mc, p=p, state=state):
                first = v_first is None
                o, v = chunked_attention(w, p + "mix.", mc, h, eps, v_first, first)
                state["v"] = v if (mc.get("v_mix") and first) else None
                return o
            x = sublayer_step(w, cfg, x, p, "1", mixer)
            if state.get("v") is not None:
                v_first = state["v"]
        elif layer["type"] == "latent_attention":
            x = sublayer_step(w, cfg, x, p, "1", lambda h, mc=mc, p=p: latent_attention(w, p + "mix.", mc, h, eps))
        elif layer["type"] == "mingru":
            x = sublayer_step(w, cfg, x, p, "1", lambda h, p=p: mingru(w, p + "mix.", h))
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            x = sublayer_step(w, cfg, x, p, "2", lambda h, p=p: dense_ff(w, p + "mlp.", h))
        after.append(x)
    logits = norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if keep_layers else logits
