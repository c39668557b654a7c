"""Munerax through the package against the plain implementation (tests/plain/munerax_plain.py):
every mechanism's kernels alone, then whole models with sizes of their own, stepped whole, token by
token, in portions, in unequal batches, over reused slots and pages, and generated from greedily.

Some tests shape their inputs so that one key, the sink, the gate or one expert decides the result."""
import json
import math
import os

import pytest
import torch

from helpers import rel_err
from munerax_models import BF16, F32, make_weights, model, prompts, random_config, write_folder
from plain import munerax_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def tol(dt):
    return 3e-5 if dt in (F32, "float32") else 6e-2


def close(got, ref, dtype, rows=None):
    """Whether a model's output is the plain implementation's.  float32: every value, to 3e-5 of the
    largest.  bfloat16: only the ``rows`` whose routers decided clearly are held to it (see
    ``steady_prompt``); rounding is amplified where a token happens to be badly conditioned, so 95 %
    of those rows (all but one, of few) must lie within the tolerance and every row must be finite
    and within 1; the float32 run is the sharp test."""
    if dtype in (F32, "float32"):
        return rel_err(got, ref) < tol(dtype)
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    if got.shape != ref.shape or not torch.isfinite(got).all():
        return False
    err = (got - ref).abs().reshape(got.shape[0], -1).max(dim=1).values / max(1e-6, float(ref.abs().max()))
    if float(err.max()) >= 1.0:
        return False
    if rows is not None:
        err = err[rows]
    return int((err > tol(dtype)).sum()) <= max(1, err.numel() // 20)


def ops():
    from builderforce_inference_b200.kernels import ops as o
    return o


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def q64(t, dt):
    """The values a tensor of storage type ``dt`` holds, as float64."""
    return t.to(dt).to(torch.float64)


def engine(name, dtype, **kw):
    from builderforce_inference_b200.engine.engine import Engine
    folder, cfg, w = model(name, dtype)
    return Engine.load(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw), cfg, w


def S(slot, tokens, want=None):
    from builderforce_inference_b200.engine.engine import SequenceStep
    return SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)


def steady_prompt(cfg, w, length, dtype, seed0=5, least=0.015):
    """(ids, the plain model's logits, the rows a run in ``dtype`` is held to) of a random prompt.
    In bfloat16 a router that decides by a hair may be turned by rounding, and the token then takes
    other experts than the plain model's: only tokens all of whose routing decisions are won by
    ``least`` are compared (later tokens read a turned token as one key among many)."""
    ids = prompts(cfg["vocab"], [length], seed0)[0]
    won = []
    ref = P.forward_each(w, cfg, ids, won)
    rows = torch.ones(length, dtype=torch.bool)
    if dtype != "float32" and won:
        rows = torch.tensor(won).reshape(-1, length).min(dim=0).values > least
        assert length < 20 or int(rows.sum()) >= length // 3
    return ids, ref, rows


# ------------------------------------------------------------------------------------------------
# the hashed bigram embedding and its per-sequence state
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 7, 13), (1, 3, 5), (1021, 2 ** 31 - 1, 65537), (8, 0, 1), (8, 1, 0)])
def test_bigram_rows_across_steps_and_in_reused_slots(dt, buckets, mul_prev, mul_cur):
    o = ops()
    width, vocab = 24, 5000
    g = torch.Generator().manual_seed(buckets)
    table = torch.randn(buckets + 1, width, generator=g).to(dt)
    a, b, c = (torch.randint(0, vocab, (n,), generator=g).tolist() for n in (9, 4, 6))
    want = {k: q64(table, dt)[P.bigram_rows(s, buckets, mul_prev, mul_cur)] for k, s in (("a", a), ("b", b), ("c", c))}
    last = torch.full((4, 1), 4999, dtype=torch.int32, device=DEV)      # stale values: a first token must not read them

    def step(parts):
        """parts: (slot, start, ids); a padding row stands between the sequences."""
        ids, pos, slot, cu, sl = [], [], [], [0], []
        for s, start, toks in parts:
            ids += list(toks)
            pos += list(range(start, start + len(toks)))
            slot += [s] * len(toks)
            cu.append(len(ids))
            sl.append(s)
        ids.append(0), pos.append(0), slot.append(-1)
        x = torch.full((len(ids), width), 2.0, dtype=F32, device=DEV)
        o.bigram_add(table.to(DEV), i32(ids), i32(pos), i32(slot), last, x, mul_prev, mul_cur, vocab)
        o.keep_last_tokens(i32(ids), i32(cu), i32(sl), last, len(sl))
        assert float((x[-1] - 2.0).abs().max()) == 0.0                  # the padding row is left alone
        return x[:-1].double().cpu() - 2.0

    got = step([(2, 0, a[:5]), (0, 0, b[:1])])                           # two prompts begin
    assert rel_err(got, torch.cat([want["a"][:5], want["b"][:1]])) < 1e-6
    got = step([(0, 1, b[1:2]), (2, 5, a[5:6])])                         # one token each: the previous one is the state's
    assert rel_err(got, torch.stack([want["b"][1], want["a"][5]])) < 1e-6
    got = step([(2, 6, a[6:]), (0, 2, b[2:])])                           # portions
    assert rel_err(got, torch.cat([want["a"][6:], want["b"][2:]])) < 1e-6
    got = step([(2, 0, c)])                                              # the slot is used again by another sequence
    assert rel_err(got, want["c"]) < 1e-6
    assert int(last[2, 0]) == c[-1] and int(last[0, 0]) == b[-1] and int(last[1, 0]) == 4999


# ------------------------------------------------------------------------------------------------
# latent attention: the kernels in a row, over a hand-made paged cache
# ------------------------------------------------------------------------------------------------
class Rows:
    """A hand-made paged cache of one row per token whose pages are handed out in a scrambled order
    and start as NaN."""

    def __init__(self, n_slots, max_len, row, rank, dt, seed=0):
        from builderforce_inference_b200.cache import KVView
        blocks = (max_len + 63) // 64
        n_pages = n_slots * blocks + 3
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.table = torch.tensor(perm[:n_slots * blocks], dtype=torch.int32).reshape(n_slots, blocks)
        self.k = torch.full((n_pages, 1, 64, row), float("nan"), dtype=dt, device=DEV)
        self.view = KVView(self.k, self.k, self.table.to(DEV), 1, row, None, v_dim=rank, values_in_keys=True)

    def read(self, slot, n):
        return torch.stack([self.k[int(self.table[slot, p // 64]), 0, p % 64, :] for p in range(n)]).double().cpu()


class Latent:
    """One latent attention layer given by its sizes: random matrices, and projection rows laid out
    as the kernels read them ([queries | gate logits | pad | down projection])."""

    def __init__(self, heads, d, rd, dv, rank, rot, dt, seed=0, scale=0.2, base=100.0, eps=1e-5, pad=3, splits=None):
        self.a, self.d, self.rd, self.dv, self.r, self.rot, self.dt = heads, d, rd, dv, rank, rot, dt
        self.splits = splits          # not None: the tensor-core attention, cut into this many key ranges (0: its own choice)
        self.scale, self.base, self.eps = scale, base, eps
        g = torch.Generator().manual_seed(seed)
        self.g = g
        self.uk = (torch.randn(heads * d, rank, generator=g) / math.sqrt(rank)).to(dt)
        self.uv = (torch.randn(heads * dv, rank, generator=g) / math.sqrt(rank)).to(dt)
        self.nw = (1 + 0.2 * torch.randn(rank, generator=g)).to(dt)
        self.sink = torch.randn(heads, generator=g)
        self.gate_off = heads * (d + rd)
        self.kv_off = self.gate_off + heads + pad
        self.cols = self.kv_off + rank + rd
        self.table = None
        if rot:
            half = rot // 2
            f = torch.tensor(base, dtype=torch.float64) ** (-2.0 * torch.arange(half, dtype=torch.float64) / rot)
            ang = torch.arange(1024, dtype=torch.float64)[:, None] * f[None, :]
            self.table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous().to(DEV)

    def rows(self, n, amp=1.0):
        return (amp * torch.randn(n, self.cols, generator=self.g)).to(self.dt)

    def plain(self, proj, latent_from=None):
        """The plain layer on projection rows: the matrices that make them are slices of an identity."""
        a, d, rd, dv, r = self.a, self.d, self.rd, self.dv, self.r
        eye = torch.eye(self.cols, dtype=P.F)
        w = {"q": eye[:self.gate_off], "g": eye[self.gate_off:self.gate_off + a], "dkv": eye[self.kv_off:],
             "dkv.norm": q64(self.nw, self.dt), "uk": q64(self.uk, self.dt), "uv": q64(self.uv, self.dt),
             "sink": self.sink.double(), "o": torch.eye(a * dv, dtype=P.F)}
        m = {"heads": a, "dim": d, "rot_dim": rd, "vdim": dv, "kv_rank": r, "scale": self.scale}
        if self.rot:
            m["rot"] = {"base": self.base, "dims": self.rot}
        h = q64(proj, self.dt)
        latent = latent_from if latent_from is not None else P.latent_of(w, "", m, h, self.eps)
        return P.latent_attention(w, "", m, h, self.eps, latent), latent

    def run(self, proj, cache, seqs, write=True, sink=True, gate=True):
        """seqs: (slot, start, tokens) in the order of ``proj``'s rows; a padding row is added."""
        o = ops()
        a, d, rd, dv, r, dt = self.a, self.d, self.rd, self.dv, self.r, self.dt
        pos, slot, cu = [], [], [0]
        for s, start, t in seqs:
            pos += list(range(start, start + t))
            slot += [s] * t
            cu.append(cu[-1] + t)
        n = cu[-1] + 1
        pos.append(0), slot.append(-1)
        p = torch.cat([proj.to(dt), torch.full((1, self.cols), float("nan"), dtype=dt)]).to(DEV)
        qa = torch.full((n, a * (r + rd)), float("nan"), dtype=dt, device=DEV)
        o.latent_prepare(p, qa, a, d, rd, r, self.kv_off, self.nw.to(DEV), self.eps, self.table, self.rot, i32(pos), i32(slot),
                         cache.view, write)
        o.latent_absorb(p, self.uk.to(DEV), qa, i32(slot), a, d, rd, r)
        lat = torch.full((n, a * r), float("nan"), dtype=dt, device=DEV)
        sinks = self.sink.float().to(DEV) if sink else None
        if self.splits is not None:
            from types import SimpleNamespace
            from builderforce_inference_b200.engine.context import Workspace
            from builderforce_inference_b200.kernels import fast_ops
            ctx = SimpleNamespace(n_seqs=len(seqs), max_seq_tokens=max(t for _, _, t in seqs), cu_seqlens=i32(cu),
                                  seq_slot=i32([s for s, _, _ in seqs]), seq_start=i32([st for _, st, _ in seqs]),
                                  workspace=Workspace(DEV), pages_bucket=0)
            # the kernel multiplies by the gates itself; the expansion then gets none
            assert fast_ops.attention_latent_bf16(ctx, qa, lat, cache.view, a, self.scale, sinks, splits=self.splits or None,
                                                  gate=p[:, self.gate_off:self.gate_off + a] if gate else None)
            gate = False
        else:
            o.attention_paged(qa, qa.stride(0), lat, cache.view, i32(cu), i32([s for s, _, _ in seqs]),
                              i32([st for _, st, _ in seqs]), len(seqs), max(t for _, _, t in seqs), a, self.scale, sinks)
        out = torch.full((n, a * dv), 9.0, dtype=dt, device=DEV)
        o.latent_expand(lat, self.uv.to(DEV), p[:, self.gate_off:self.gate_off + a] if gate else None, out, i32(slot), a, dv, r)
        assert float((out[-1].float() - 9.0).abs().max()) == 0.0       # the padding row is left alone
        return out[:-1].double().cpu()


SIZES = [(3, 10, 6, 12, 14, 6), (2, 8, 6, 5, 14, 4), (4, 16, 8, 16, 24, 8), (1, 12, 8, 30, 24, 0), (5, 48, 32, 40, 64, 32),
         (8, 64, 32, 64, 128, 32), (2, 4, 0, 4, 2, 0), (6, 128, 64, 128, 448, 64)]


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("heads,d,rd,dv,rank,rot", SIZES)
def test_latent_kernels_in_a_mixed_batch(dt, heads, d, rd, dv, rank, rot):
    """A whole prompt, a prompt's second portion over a page border and a single token in one step,
    then a layer without a down projection of its own reading the same rows."""
    L = Latent(heads, d, rd, dv, rank, rot, dt, seed=heads * 100 + d)
    t = 1e-5 if dt == F32 else 2.5e-2
    n0, n1, n2 = 70, 131, 66
    p0, p1, p2 = L.rows(n0), L.rows(n1), L.rows(n2)
    r0, lat0 = L.plain(p0)
    r1, lat1 = L.plain(p1)
    r2, lat2 = L.plain(p2)
    cache = Rows(3, 192, rank + rd, rank, dt, seed=d)
    L.run(p1[:60], cache, [(1, 0, 60)])
    L.run(p2[:n2 - 1], cache, [(0, 0, n2 - 1)])
    got = L.run(torch.cat([p0, p1[60:], p2[n2 - 1:]]), cache, [(2, 0, n0), (1, 60, n1 - 60), (0, n2 - 1, 1)])
    assert rel_err(got, torch.cat([r0, r1[60:], r2[n2 - 1:]])) < t
    # the cached rows: the normed latent and the turned shared key part
    rows = cache.read(1, n1)
    assert rel_err(rows, torch.cat([lat1[0], lat1[1]], dim=1)) < (1e-5 if dt == F32 else 1e-2)
    # another layer (its own heads and sizes) borrows them
    B = Latent(heads + 1, d + 2, rd, max(1, dv - 3), rank, rot, dt, seed=7, scale=0.15)
    pb = B.rows(n1)
    rb, _ = B.plain(pb, (q64(rows[:, :rank], dt), q64(rows[:, rank:], dt)))
    before = cache.k.clone()
    got = B.run(pb[100:], cache, [(1, 100, n1 - 100)], write=False)
    assert rel_err(got, rb[100:]) < t
    assert torch.equal(torch.nan_to_num(before), torch.nan_to_num(cache.k))          # a borrower writes nothing
    # without sink and gate: a sink of no weight and gates that are wide open
    p0[:, L.gate_off:L.gate_off + heads] = 40.0
    L.sink = torch.full((heads,), -1e30)
    got = L.run(p0, Rows(1, 128, rank + rd, rank, dt), [(0, 0, n0)], sink=False, gate=False)
    assert rel_err(got, L.plain(p0)[0]) < t and rel_err(got, r0) > 10 * t


TC_SIZES = [(5, 48, 32, 40, 64, 32), (8, 64, 32, 64, 128, 32), (6, 128, 64, 128, 448, 64), (16, 32, 16, 24, 512, 16),
            (2, 16, 16, 16, 16, 16), (40, 8, 16, 8, 48, 8), (1, 24, 32, 12, 256, 32), (2, 8, 192, 8, 512, 64)]


@pytest.mark.parametrize("splits", [0, 1, 3, 7])
@pytest.mark.parametrize("heads,d,rd,dv,rank,rot", TC_SIZES)
def test_tensor_core_latent_attention_in_a_mixed_batch(heads, d, rd, dv, rank, rot, splits):
    """The bfloat16 kernel over stacked (token, head) rows, whole and cut into key ranges (more ranges
    than a short sequence has tiles too): a prompt, a portion that starts inside a page behind a cached
    prefix, single tokens at a tile's and a page's first and last place, over pages that start as NaN."""
    L = Latent(heads, d, rd, dv, rank, rot, BF16, seed=heads * 100 + d, splits=splits)
    n0, n1, n2, n3, n4 = 70, 200, 65, 33, 32
    ps = [L.rows(n) for n in (n0, n1, n2, n3, n4)]
    refs = [L.plain(p)[0] for p in ps]
    cache = Rows(5, 256, rank + rd, rank, BF16, seed=d)
    L.run(ps[1][:37], cache, [(1, 0, 37)])
    for i, n in ((2, n2), (3, n3), (4, n4)):
        L.run(ps[i][:n - 1], cache, [(i, 0, n - 1)])
    got = L.run(torch.cat([ps[0], ps[1][37:]]), cache, [(0, 0, n0), (1, 37, n1 - 37)])
    assert rel_err(got, torch.cat([refs[0], refs[1][37:]])) < 2.5e-2
    got = L.run(torch.cat([ps[i][-1:] for i in (2, 3, 4)]), cache, [(2, n2 - 1, 1), (3, n3 - 1, 1), (4, n4 - 1, 1)])
    assert rel_err(got, torch.cat([refs[i][-1:] for i in (2, 3, 4)])) < 2.5e-2
    # the general kernel on the same rows: the two differ by rounding only
    G = Latent(heads, d, rd, dv, rank, rot, BF16, seed=heads * 100 + d)
    both = [(0, 0, n0)]
    assert rel_err(L.run(ps[0], cache, both, write=False), G.run(ps[0], cache, both, write=False)) < 1.5e-2


def test_tensor_core_latent_attention_declines_what_it_does_not_take():
    """Sizes that are not multiples of 16 run the general kernel; nothing is launched for them."""
    for heads, d, rd, dv, rank, rot in [(3, 10, 6, 12, 14, 6), (4, 16, 8, 16, 24, 8)]:
        L = Latent(heads, d, rd, dv, rank, rot, BF16, splits=0)
        with pytest.raises(AssertionError):
            L.run(L.rows(5), Rows(1, 64, rank + rd, rank, BF16), [(0, 0, 5)])


@pytest.mark.parametrize("dt,splits", [(F32, None), (BF16, None), (BF16, 0), (BF16, 4)])
@pytest.mark.parametrize("through", ["latent", "shared part"])
def test_one_loud_key_far_back_at_page_borders_and_the_first_tokens(dt, splits, through):
    """One key among hundreds stands out for every query (through the latent, or through the shared
    key part's values that do not turn): the tokens from it on hear it, in a prompt, in a portion
    that starts behind it, and token by token; the tokens before it do not."""
    for loud in (3, 31, 32, 63, 64, 65, 127, 128):
        L = Latent(3, 8, 8 if splits is None else 16, 6, 16, 4, dt, seed=loud, splits=splits)
        n = 330
        proj = L.rows(n, amp=0.05)
        a, d, rd, r, ko = L.a, L.d, L.rd, L.r, L.kv_off
        if through == "latent":
            # the loud token's latent is one unit vector (normed: sqrt(rank) * its weight), the others
            # have nothing along it and little weight elsewhere; every query's unrotated part lies
            # along what W_uk makes of that vector
            L.nw = torch.full((r,), 0.02).to(dt)
            L.nw[2] = 1.0
            proj[:, ko + 2] = 0.0
            proj[loud, ko:ko + r] = 0.0
            proj[loud, ko + 2] = 5.0
            for h in range(a):
                proj[:, h * (d + rd):h * (d + rd) + d] = 3.0 * L.uk.float()[h * d:(h + 1) * d, 2].sign()
        else:
            proj[loud, ko + r + 6] = 5.0
            for h in range(a):
                proj[:, h * (d + rd) + d + 6] = 5.0
        L.scale, L.sink = 1.0, torch.tensor([0.0, -1.0, 2.0])
        proj[:, L.gate_off:L.gate_off + a] = 4.0
        ref, lat = L.plain(proj)
        # the value the loud key brings, per head: W_uv c_loud (gated)
        heard = (q64(L.uv, dt).reshape(a, L.dv, r) @ lat[0][loud]).reshape(-1) * torch.sigmoid(torch.tensor(4.0, dtype=P.F))
        t = 1e-5 if dt == F32 else 3e-2
        cache = Rows(3, n + 60, r + rd, r, dt, seed=loud)
        whole = L.run(proj, cache, [(0, 0, n)])
        assert rel_err(whole, ref) < t
        for p in list(range(max(0, loud - 2), loud + 3)) + [n - 1]:
            is_heard = float((whole[p] - heard).abs().max()) < 0.15 * float(heard.abs().max())
            assert is_heard == (p >= loud), (loud, p)
        L.run(proj[:loud + 1], cache, [(1, 0, loud + 1)])
        rest = L.run(proj[loud + 1:], cache, [(1, loud + 1, n - loud - 1)])
        assert rel_err(rest, ref[loud + 1:]) < t
        L.run(proj[:n - 1], cache, [(2, 0, n - 1)])
        one = L.run(proj[n - 1:], cache, [(2, n - 1, 1)])
        assert rel_err(one, ref[n - 1:]) < t and float((one[0] - heard).abs().max()) < 0.15 * float(heard.abs().max())


@pytest.mark.parametrize("dt", [F32, BF16])
def test_a_sink_and_a_gate_per_head(dt):
    L = Latent(4, 8, 4, 5, 8, 4, dt, seed=2)
    n = 70
    proj = L.rows(n, amp=0.3)
    L.sink = torch.tensor([-30.0, 30.0, 0.0, 0.5])
    g0 = L.gate_off
    proj[:, g0:g0 + 4] = torch.tensor([30.0, 30.0, 30.0, -30.0])
    ref, lat = L.plain(proj)
    got = L.run(proj, Rows(1, n, L.r + L.rd, L.r, dt), [(0, 0, n)])
    assert rel_err(got, ref) < (1e-5 if dt == F32 else 2e-2)
    got = got.reshape(n, 4, 5)
    # a huge sink takes all the weight of its head, a closed gate all the output of its head, and of no other
    assert float(got[:, 1].abs().max()) < 1e-6 and float(got[:, 3].abs().max()) < 1e-6
    assert float(got[:, 0].abs().max()) > 0.05 and float(got[:, 2].abs().max()) > 0.05
    # the first token has one key: its weight is exp(s) / (exp(s) + exp(sink)), the sink unscaled
    v0 = q64(L.uv, dt).reshape(4, 5, L.r) @ lat[0][0]
    h = q64(proj, dt)
    qn, qr = h[0, 2 * 12:2 * 12 + 8], h[0, 2 * 12 + 8:2 * 12 + 12]
    kn = q64(L.uk, dt).reshape(4, 8, L.r)[2] @ lat[0][0]
    s = float((qn @ kn + qr @ lat[1][0]) * L.scale)
    want = v0[2] * math.exp(s) / (math.exp(s) + 1.0)
    assert float((got[0, 2] - want).abs().max()) < (1e-5 if dt == F32 else 2e-2) * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------------
# the latent attention part, through the registry and the package's own cache
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_latent_part_prompt_portions_single_tokens_and_freed_pages(dtype):
    """The mixer as the model builds it, over the package's cache: a prompt whole, the same prompt
    in portions and then token by token in a slot and pages that another sequence has used."""
    from builderforce_inference_b200.cache import SequenceCache
    from builderforce_inference_b200.engine.context import Workspace, build_context
    from builderforce_inference_b200.engine.decoder import Runtime
    from builderforce_inference_b200.parts import MIXERS, PartSpec
    width, a, d, rd, dv, r = 56, 3, 12, 8, 10, 20
    rot = PartSpec("rotary", {"theta": 500.0, "rot_dim": 8, "pairing": "half"})
    part = MIXERS.build(PartSpec("latent_attention", {"width": width, "n_heads": a, "dim": d, "rot_dim": rd, "v_dim": dv,
                                                      "kv_rank": r, "position": rot, "eps": 1e-5, "scale": 0.3,
                                                      "sink": "learned", "gate": True}))
    g = torch.Generator().manual_seed(11)
    w = {}
    for name, ps in part.all_param_specs().items():
        t = torch.randn(ps.shape, generator=g)
        w[name] = (1 + 0.1 * t if ps.role == "norm" else t if name == "sink" else t / math.sqrt(ps.shape[-1])).to(dtype)
    rt, ws = Runtime(DEV, dtype), Workspace(DEV)
    part.prepare(rt, 512)
    part.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
    cache = SequenceCache([part.cache_need()], [None], 64 * 6, 512, dtype, DEV)
    n = 150
    h = torch.randn(n, width, generator=g).to(dtype)
    pw = {k.replace("_proj", "").replace("dkv_norm", "dkv.norm"): q64(v, dtype) for k, v in w.items()}
    m = {"heads": a, "dim": d, "rot_dim": rd, "vdim": dv, "kv_rank": r, "scale": 0.3, "rot": {"base": 500.0, "dims": 8}}
    ref = P.latent_attention(pw, "", m, q64(h, dtype), 1e-5, P.latent_of(pw, "", m, q64(h, dtype), 1e-5))

    def run(slot, start, count):
        cache.begin_step([slot], [count])
        ctx = build_context([(slot, start, [1] * count)], dtype, ws, DEV)
        out = torch.zeros(count, width, dtype=F32, device=DEV)
        part.forward(ctx, h[start:start + count].to(DEV), out, cache.run_cache(0))
        cache.end_step([slot], [count])
        return out.double().cpu()

    t = 1e-5 if dtype == F32 else 2.5e-2
    first = cache.acquire()
    cache.poison()
    assert rel_err(run(first, 0, n), ref) < t
    cache.release(first)
    cache.poison(1e4)                              # what the first sequence left must not matter
    slot = cache.acquire()
    outs, at = [], 0
    for c in (2, 62, 1, 2, 63):                    # portions that end at, before and behind a page's edge
        outs.append(run(slot, at, c))
        at += c
    while at < n:
        outs.append(run(slot, at, 1))
        at += 1
    assert rel_err(torch.cat(outs), ref) < t
    cache.release(slot)
    cache.check()


# ------------------------------------------------------------------------------------------------
# the feed-forwards
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_dense_feed_forward_with_the_tanh_gelu(dtype):
    from builderforce_inference_b200.engine.context import Workspace, build_context
    from builderforce_inference_b200.engine.decoder import Runtime
    from builderforce_inference_b200.parts import FEED_FORWARDS, PartSpec
    width, ff = 88, 136
    part = FEED_FORWARDS.build(PartSpec("gated_mlp", {"width": width, "inner": ff, "activation": "gelu_tanh"}))
    g = torch.Generator().manual_seed(3)
    w = {k: (torch.randn(ps.shape, generator=g) * (2.0 / math.sqrt(ps.shape[1]))).to(dtype) for k, ps in part.all_param_specs().items()}
    part.load_all({k: v.to(DEV) for k, v in w.items()}, Runtime(DEV, dtype))
    ws = Workspace(DEV)
    pw = {"gate": q64(w["gate_proj"], dtype), "up": q64(w["up_proj"], dtype), "down": q64(w["down_proj"], dtype)}
    for rows in (1, 5, 40, 200):                   # few rows and many rows take different kernels
        h = (2.0 * torch.randn(rows, width, generator=g)).to(dtype)      # gate inputs on both sides of the bend
        res = torch.randn(rows, width, generator=g)
        out = res.clone().to(DEV)
        part.forward(build_context([(0, 0, [1] * rows)], dtype, ws, DEV), h.to(DEV), out)
        ref = res.double() + P.dense_ff(pw, "", q64(h, dtype))
        assert rel_err(out, ref) < (1e-5 if dtype == F32 else 1.5e-2), rows
    z = torch.linspace(-6, 6, 25, dtype=P.F)
    assert float(P.gelu_tanh(z)[0]) < 0 and abs(float(P.gelu_tanh(z)[-1]) - 6.0) < 1e-6


@pytest.mark.parametrize("E,top,groups,keep", [(12, 2, 3, 1), (6, 3, 3, 2), (5, 1, 1, 1), (64, 6, 8, 3), (40, 8, 1, 1),
                                               (8, 2, 8, 3), (8, 8, 4, 4), (16, 4, 4, 4), (9, 3, 3, 3), (2, 1, 2, 1)])
def test_sigmoid_router_with_groups_counted_by_their_two_best(E, top, groups, keep):
    o = ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    n = 300
    z = 2.0 * torch.randn(n, E, generator=g)
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(n, top, dtype=F32, device=DEV)
    o.moe_route(z.to(DEV), E, None, idx, wt, top, groups, keep, 1.7, None, o.SCORE_SIGMOID, 2)
    rep = []
    ridx, rw = P.route(z.double(), top, groups, keep, 1.7, rep)
    got = idx.cpu().long()
    sure = torch.tensor(rep) > 1e-6
    assert int(sure.sum()) > n * 0.9
    assert torch.equal(got[sure], ridx[sure])             # best first, as the plain top-k lists them
    assert rel_err(wt.cpu()[sure], rw[sure]) < 1e-5
    # where the best single expert's group loses by its sum, it is not chosen
    if groups > 1 and keep < groups and E // groups > 1:
        best = z.argmax(dim=1)
        assert int((got != best[:, None]).all(dim=1).sum()) > 0
    # the same decision with the logits made in the kernel, from float32 and from bfloat16 inputs
    width = 72
    w_r = torch.randn(E, width, generator=g) * (3.0 / math.sqrt(width))
    h = torch.randn(n, width, generator=g)
    slots = [0] * n
    slots[5] = -1
    for dt in (F32, BF16):
        idx.fill_(-7)
        o.moe_router(h.to(dt).to(DEV), w_r.to(DEV), E, None, i32(slots), idx, wt, top, groups, keep, 0.6, None, o.SCORE_SIGMOID, 2)
        rep = []
        ridx, rw = P.route(q64(h, dt) @ w_r.double().T, top, groups, keep, 0.6, rep)
        sure = torch.tensor(rep) > 1e-5
        sure[5] = False
        got = idx.cpu().long()
        assert torch.equal(got[sure], ridx[sure]) and rel_err(wt.cpu()[sure], rw[sure]) < 1e-5
        assert int(got[5, 0]) == -7                       # a padding row is left alone


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("width,ff,E,top,shared", [(40, 24, 6, 3, 12), (128, 64, 8, 2, 96), (72, 20, 4, 1, None), (64, 8, 16, 16, 40)])
def test_squared_relu_experts_both_ways_and_the_shared_expert(dt, width, ff, E, top, shared):
    """The routed part as the model builds it: few tokens read the chosen experts' weights, many
    tokens run every expert and weigh; a shared expert is added as it is."""
    from builderforce_inference_b200.engine.context import Workspace, build_context
    from builderforce_inference_b200.engine.decoder import Runtime
    from builderforce_inference_b200.parts import FEED_FORWARDS, PartSpec
    dtype = dt
    part = FEED_FORWARDS.build(PartSpec("mixture_of_experts", {
        "width": width, "n_experts": E, "top": top, "inner": ff, "n_groups": 1, "keep_groups": 1, "shared_inner": shared,
        "correction": False, "weight_scale": 1.3, "score": "sigmoid", "group_top": 2, "expert": "relu_squared", "shared_gate": False}))
    g = torch.Generator().manual_seed(width + ff)
    w = {}
    for name, ps in part.all_param_specs().items():
        k = 6.0 if name == "router" else 1.5
        w[name] = (torch.randn(ps.shape, generator=g) * (k / math.sqrt(ps.shape[1]))).to(dtype)
    part.load_all({k: v.to(DEV) for k, v in w.items()}, Runtime(DEV, dtype))
    ws = Workspace(DEV)
    pw = {"router": q64(w["router"], dtype)}
    for e in range(E):
        pw[f"e{e}.up"], pw[f"e{e}.down"] = q64(w[f"experts.{e}.up_proj"], dtype), q64(w[f"experts.{e}.down_proj"], dtype)
    f = {"router": {"experts": E, "top": top, "scale": 1.3}}
    if shared:
        pw["shared.up"], pw["shared.down"] = q64(w["shared.up_proj"], dtype), q64(w["shared.down_proj"], dtype)
        f["shared"] = {"ff": shared}
    for rows in (1, 3, 70, 300):
        h = torch.randn(rows, width, generator=g).to(dtype)
        res = torch.randn(rows, width, generator=g)
        rep = []
        ref = res.double() + P.routed_ff(pw, "", f, q64(h, dtype), rep)
        sure = torch.tensor(rep) > 1e-4            # both sides read the same stored values: only the sums' order differs
        out = res.clone().to(DEV)
        part.forward(build_context([(0, 0, [1] * rows)], dtype, ws, DEV), h.to(DEV), out)
        assert int(sure.sum()) >= rows * 0.9
        assert rel_err(out.cpu()[sure], ref[sure]) < (1e-5 if dt == F32 else 2.5e-2), rows
        stored = torch.zeros(rows, width, dtype=F32, device=DEV) + 7.0
        part.forward_store(build_context([(0, 0, [1] * rows)], dtype, ws, DEV), h.to(DEV), stored)
        assert rel_err(stored.cpu()[sure], (ref - res.double())[sure]) < (1e-5 if dt == F32 else 2.5e-2), rows
    # an expert alone: one expert, top 1; negative inputs of the activation give nothing
    assert float(P.relu_squared(torch.tensor([-2.0, 3.0], dtype=P.F))[0]) == 0.0


# ------------------------------------------------------------------------------------------------
# whole models
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_whole_prompts_and_every_layer(name, dtype):
    from builderforce_inference_b200.engine.context import build_context
    eng, cfg, w = engine(name, dtype)
    ids, ref, rows = steady_prompt(cfg, w, 200, dtype)
    layers = P.forward_layers(w, cfg, ids)
    slot = eng.acquire()
    assert close(eng.step([S(slot, ids)]), ref, dtype, rows)
    eng.release(slot)
    # the residual stream after every layer
    slot = eng.acquire()
    eng.cache.begin_step([slot], [len(ids)])
    ctx = build_context([(slot, 0, ids)], eng.dtype, eng.workspace, eng.device, eng.status)
    x = eng.decoder.embed(ctx, eng.cache)
    for i in range(len(cfg["layers"])):
        eng.decoder.run_layers(ctx, x, eng.cache, i, i + 1)
        assert close(x, layers[i], dtype, rows), i
    eng.cache.end_step([slot], [len(ids)])
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_prompt_then_token_by_token_over_several_pages(name, dtype, graphs):
    eng, cfg, w = engine(name, dtype, use_graphs=graphs)
    ids, ref, rows = steady_prompt(cfg, w, 210, dtype, seed0=40)
    slot = eng.acquire()
    head = 3
    outs = [eng.step([S(slot, ids[:head])]).clone()]
    for t in ids[head:]:
        outs.append(eng.step([S(slot, [t])]).clone())
    assert close(torch.cat(outs), ref, dtype, rows)
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_portions_of_a_prompt_down_to_two_tokens(name, dtype):
    eng, cfg, w = engine(name, dtype)
    ids, ref, rows = steady_prompt(cfg, w, 201, dtype, seed0=70)
    for cuts in ([2, 2, 3, 64, 65, 63, 2], [128, 73], [1, 7, 1, 130, 62], [1, 200], [193, 2, 6]):
        slot = eng.acquire()
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([S(slot, ids[at:at + c])]).clone())
            at += c
        assert at == len(ids)
        assert close(torch.cat(outs), ref, dtype, rows), cuts
        eng.release(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_unequal_batches_reused_slots_and_poisoned_pages(name, dtype):
    eng, cfg, w = engine(name, dtype, max_tokens=1024)
    eng.cache.poison()
    lengths = [70, 5, 131, 1]
    made = [steady_prompt(cfg, w, n + 6, dtype, seed0=100 + 20 * i) for i, n in enumerate(lengths)]
    seqs, refs, rows = [m[0] for m in made], [m[1] for m in made], [m[2] for m in made]
    for round_ in range(2):                               # the second round runs in slots and pages that were used
        slots = [eng.acquire() for _ in seqs]
        got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lengths)])
        want = torch.cat([r[:n] for r, n in zip(refs, lengths)])
        assert close(got, want, dtype, torch.cat([r[:n] for r, n in zip(rows, lengths)])), round_
        live = list(range(len(seqs)))
        for step in range(6):                             # decoded together; the shortest leave first
            got = eng.step([S(slots[i], [seqs[i][lengths[i] + step]]) for i in live])
            want = torch.stack([refs[i][lengths[i] + step] for i in live])
            assert close(got, want, dtype, torch.stack([rows[i][lengths[i] + step] for i in live])), (round_, step)
            if step in (1, 3):
                eng.release(slots[live.pop(1)])
        for i in live:
            eng.release(slots[i])
        eng.cache.check()
        eng.cache.poison()
        seqs, refs, rows, lengths = seqs[::-1], refs[::-1], rows[::-1], lengths[::-1]     # other sequences in the slots the first round used


def test_batch_against_each_alone_in_float32():
    eng, cfg, w = engine("odd", "float32")
    seqs = prompts(cfg["vocab"], [33, 140, 2, 71], seed=9)
    slots = [eng.acquire() for _ in seqs]
    together = eng.step([S(sl, s) for sl, s in zip(slots, seqs)]).clone()
    nxt = eng.step([S(sl, [7]) for sl in slots]).clone()
    for sl in slots:
        eng.release(sl)
    at = 0
    for i, s in enumerate(seqs):
        sl = eng.acquire()
        alone = eng.step([S(sl, s)]).clone()
        # the products' tiles differ with the number of rows, so sums differ in their last bits
        assert rel_err(together[at:at + len(s)], alone) < 1e-5
        assert rel_err(nxt[i:i + 1], eng.step([S(sl, [7])])) < 1e-5
        eng.release(sl)
        at += len(s)


def test_the_previous_token_and_a_far_token_reach_the_logits():
    """Through the whole model: changing a sequence's first token changes the last position's logits
    300 tokens on (every earlier key is read), and changing only the token before a decoded one
    changes that token's bigram row although the cache of the earlier tokens is the same."""
    eng, cfg, w = engine("odd", "float32")
    ids = prompts(cfg["vocab"], [300], seed=77)[0]
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    sl = eng.acquire()
    a = eng.step([S(sl, ids, [299])]).clone()
    eng.release(sl)
    sl = eng.acquire()
    eng.step([S(sl, other[:298], [])])
    b = torch.cat([eng.step([S(sl, [t])]) for t in other[298:]])[-1:].clone()
    eng.release(sl)
    ref_a, ref_b = P.forward_each(w, cfg, ids)[299:], P.forward_each(w, cfg, other)[299:]
    assert rel_err(a, ref_a) < 3e-5 and rel_err(b, ref_b) < 3e-5
    assert rel_err(ref_a, ref_b) > 1e-3                    # the test's premise: the far token matters


@pytest.mark.parametrize("seed", range(101, 117))
def test_random_configurations_in_float32(seed):
    """Configurations drawn from a seed (layer order, every size, borrowed caches, groups, with and
    without feed-forward, shared expert, rotation and bigram table): an unequal batch of prompts, five
    tokens decoded together, and the longest prompt again in portions, against the plain
    implementation.  A prompt whose routers decide by less than 1e-4 somewhere is not compared."""
    from builderforce_inference_b200.engine.engine import Engine
    cfg = random_config(seed)
    w = make_weights(cfg, seed, F32)
    eng = Engine.load(write_folder(cfg, w), dtype="float32", max_tokens=2048)
    w64 = {k: v.to(torch.float64) for k, v in w.items()}
    lens = [(1, 5, 70, 130, 260)[seed % 5], (2, 33, 200)[seed % 3], (1, 64, 129)[seed % 2]]
    seqs = prompts(cfg["vocab"], [n + 5 for n in lens], seed)
    refs, steady = [], []
    for s in seqs:
        rep = []
        refs.append(P.forward_each(w64, cfg, s, rep))
        steady.append(not rep or min(rep) > 1e-4)
    slots = [eng.acquire() for _ in seqs]
    got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        if steady[i]:
            assert rel_err(got[at:at + n], refs[i][:n]) < 4e-4, (i, cfg)
        at += n
    for step in range(5):
        got = eng.step([S(sl, [s[n + step]]) for sl, s, n in zip(slots, seqs, lens)])
        for i, n in enumerate(lens):
            if steady[i]:
                assert rel_err(got[i:i + 1], refs[i][n + step:n + step + 1]) < 4e-4, (i, step, cfg)
    for sl in slots:
        eng.release(sl)
    i = max(range(3), key=lambda k: lens[k])
    sl, outs, at = eng.acquire(), [], 0
    for c in [max(1, lens[i] // 3), 2, 1, 97, 10 ** 6]:
        c = min(c, lens[i] - at)
        if c > 0:
            outs.append(eng.step([S(sl, seqs[i][at:at + c])]).clone())
            at += c
    if steady[i]:
        assert rel_err(torch.cat(outs), refs[i][:lens[i]]) < 4e-4, cfg
    eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("seed", [201, 202, 203, 204])
def test_random_configurations_in_bfloat16(seed):
    from builderforce_inference_b200.engine.engine import Engine
    cfg = random_config(seed)
    w = make_weights(cfg, seed, BF16, steady=True)
    eng = Engine.load(write_folder(cfg, w), dtype="bfloat16", max_tokens=2048)
    w64 = {k: v.to(torch.float64) for k, v in w.items()}
    ids, ref, rows = steady_prompt(cfg, w64, 150, "bfloat16", seed0=seed)
    sl = eng.acquire()
    outs = [eng.step([S(sl, ids[:100])]).clone(), eng.step([S(sl, ids[100:140])]).clone()]
    outs += [eng.step([S(sl, [t])]).clone() for t in ids[140:]]
    assert close(torch.cat(outs), ref, "bfloat16", rows), cfg
    eng.release(sl)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(dtype):
    from builderforce_inference_b200.engine.api import Model
    from builderforce_inference_b200.sampling.params import SampleParams
    folder, cfg, w = model("odd", dtype)
    m = Model.load(folder, dtype=dtype, max_tokens=1024)
    ps = prompts(cfg["vocab"], [12, 3, 40, 1], seed=21)
    n_new = 24
    outs = m.generate_batch(ps, SampleParams(temperature=0.0, max_tokens=n_new), ignore_eos=True)
    for p, got in zip(ps, outs):
        got = list(got)
        assert len(got) == n_new
        # every generated id is the plain model's best id given the ids before it, or (bfloat16) a near tie
        full = p + got
        ref = P.forward_each(w, cfg, full)
        for i, tok in enumerate(got):
            row = ref[len(p) + i - 1]
            if int(torch.argmax(row)) != tok:
                assert dtype == "bfloat16" and float(row.max() - row[tok]) < 0.05 * float(row.max() - row.min())


def test_trace_replay_and_command_line_take_the_model():
    import subprocess
    import sys
    import tempfile

    import numpy as np

    from helpers import ROOT
    folder, cfg, w = model("odd", "float32")
    a, b = prompts(cfg["vocab"], [40, 9], seed=31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:40], "want": [8]}], "end": ["a"]}]
    out_dir = tempfile.mkdtemp(prefix="bfi_trace_")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
                        "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    assert [line for line in r.stdout.splitlines() if line.startswith("done ")] == ["done 0", "done 1", "done 2"]
    ra, rb = P.forward_each(w, cfg, a), P.forward_each(w, cfg, b)
    got0 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(3, -1).copy())
    assert rel_err(got0, torch.stack([ra[0], ra[29], rb[7]])) < 3e-5
    got1 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "1.f32"), dtype="<f4").reshape(1, -1).copy())
    assert rel_err(got1, ra[30:31]) < 3e-5
    got2 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(1, -1).copy())
    assert rel_err(got2, ra[39:40]) < 3e-5
    # the command line generates from it
    r = subprocess.run([sys.executable, "-m", "builderforce_inference_b200", "run", folder, " ".join(map(str, a[:12])), "--dtype", "float32",
                        "--max-tokens", "6", "--ignore-eos", "--max-tokens-cached", "256"], capture_output=True, text=True, cwd=ROOT,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    new = [int(t) for t in r.stdout.replace(",", " ").split()][-6:]
    full = a[:12] + new
    ref = P.forward_each(w, cfg, full)
    assert [int(torch.argmax(ref[11 + i])) for i in range(6)] == new
