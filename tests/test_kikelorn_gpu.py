"""Kikelorn through the package against the plain implementation (tests/plain/kikelorn_plain.py):
every mechanism's kernels alone, then whole models with sizes of their own, stepped whole, token by
token, in portions, in unequal batches, over reused slots and pages, and generated from greedily.

Some tests shape their inputs so that one far token, a chunk's edge or a gate decides the result."""
import json
import os

import pytest
import torch

from helpers import rel_err
from kikelorn_models import BF16, F32, att, config, gru, lat, make_weights, model, prompts, random_config, rot, with_mlp, write_folder
from plain import kikelorn_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F = torch.float64


def tol(dt):
    return 3e-5 if dt in (F32, "float32") else 6e-2


def close(got, ref, dtype):
    """Whether a model's output is the plain implementation's.  float32: every value, to 3e-5 of the
    largest.  bfloat16: rounding is amplified where a token happens to be badly conditioned, so 95 %
    of the rows (all but one, of few) must lie within the tolerance and every row must be finite and
    within 1; the float32 run is the sharp test."""
    if dtype in (F32, "float32"):
        return rel_err(got, ref) < tol(dtype)
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    if got.shape != ref.shape or not torch.isfinite(got).all():
        return False
    err = (got - ref).abs().reshape(got.shape[0], -1).max(dim=1).values / max(1e-6, float(ref.abs().max()))
    return float(err.max()) < 1.0 and int((err > tol(dtype)).sum()) <= max(1, err.numel() // 20)


def ops():
    from builderforce_inference_b200.kernels import ops as o
    return o


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def q64(t, dt):
    """The values a tensor of storage type ``dt`` holds, as float64."""
    return t.to(dt).to(F)


def engine(name, dtype, **kw):
    from builderforce_inference_b200.engine.engine import Engine
    folder, cfg, w = model(name, dtype)
    return Engine.load(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw), cfg, w


def engine_of(cfg, seed, dtype="float32", **kw):
    from builderforce_inference_b200.engine.engine import Engine
    w = make_weights(cfg, seed, F32 if dtype == "float32" else BF16, steady=dtype != "float32")
    eng = Engine.load(write_folder(cfg, w), dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw)
    return eng, {k: v.to(F) for k, v in w.items()}


def S(slot, tokens, want=None):
    from builderforce_inference_b200.engine.engine import SequenceStep
    return SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)


def packed(steps):
    """Index arrays of a step ``[(slot, tokens brought), ...]``: token_slot, cu_seqlens, seq_slot."""
    slot_of, cu, slots = [], [0], []
    for slot, n in steps:
        slot_of += [slot] * n
        cu.append(cu[-1] + n)
        slots.append(slot)
    return i32(slot_of), i32(cu), i32(slots)


# ------------------------------------------------------------------------------------------------
# the convolution over time, its options and its per-sequence state
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("din,dout", [(F32, F32), (BF16, BF16), (F32, BF16)])
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("C,off,mix_off", [(37, 3, 20), (40, 8, 24)])
def test_convolution_with_its_options_in_portions_and_single_tokens(din, dout, taps, C, off, mix_off):
    """Three sequences in slots 4, 0 and 2 advance together through steps of unequal portions, down
    to single tokens; the output (the input plus its convolution), the copy of the input and the
    mixing of the last channels are the plain ones over the whole sequences.  Channels and offsets
    in whole groups of 8 take the kernels that move 16 bytes at a time (2 to 4 taps: the one that
    slides a window along a thread's tokens)."""
    o = ops()
    g = torch.Generator().manual_seed(taps)
    lens = {4: 31, 0: 9, 2: 17}
    u = {s: torch.randn(n, C + off, generator=g).to(din) for s, n in lens.items()}
    w = torch.randn(C, taps, generator=g).to(dout)
    src = {s: torch.randn(n, C - mix_off, generator=g).to(dout) for s, n in lens.items()}
    lam = torch.tensor([0.35], dtype=torch.float32, device=DEV)
    state = torch.zeros(6, taps - 1, C, dtype=torch.float32, device=DEV)
    ref = {}
    for s in lens:
        uu = q64(u[s], din)[:, off:]
        y = uu + P.causal_conv(uu, q64(w, dout))
        y[:, mix_off:] = (1.0 - 0.35) * y[:, mix_off:] + 0.35 * q64(src[s], dout)
        ref[s] = y
    plan = [[(4, 7), (0, 1), (2, 2)], [(4, 1), (0, 1), (2, 1)], [(4, 1), (0, 1), (2, 1)], [(4, 2), (0, 6), (2, 13)], [(4, 20)]]
    at = {s: 0 for s in lens}
    for step in plan:
        rows = torch.cat([u[s][at[s]:at[s] + n] for s, n in step]).to(DEV)
        mixes = torch.cat([src[s][at[s]:at[s] + n] for s, n in step]).to(DEV)
        slot_of, cu, slots = packed(step)
        y = torch.empty(rows.shape[0], C, dtype=dout, device=DEV)
        cp = torch.empty_like(y)
        dst = torch.empty(rows.shape[0], C - mix_off, dtype=dout, device=DEV)
        single = all(n == 1 for _, n in step)
        o.causal_conv(rows, off, C, w.to(DEV), None, state, y, slot_of, cu, slots, len(step), single_tokens=single,
                      act=o.CONV_ACT_NONE, add_input=True, copy=cp, mix_off=mix_off, mix_src=mixes, mix_dst=dst, mix_lambda=lam)
        want = torch.cat([ref[s][at[s]:at[s] + n] for s, n in step])
        assert rel_err(y, want) < (1e-5 if dout == F32 else 1e-2), (taps, step)
        assert torch.equal(dst, y[:, mix_off:])
        assert torch.equal(cp.cpu(), rows[:, off:].to(dout).cpu())
        for s, n in step:
            at[s] += n


@pytest.mark.parametrize("din", [F32, BF16])
@pytest.mark.parametrize("taps", [2, 3, 4, 6])
def test_convolution_over_many_channels_and_sequences_that_end_inside_a_thread(din, taps):
    """512 channels, five sequences of 1 to 301 tokens whose borders fall anywhere within the four
    tokens a thread owns, a second step that goes on from the kept inputs, then single tokens."""
    o = ops()
    C = 512
    g = torch.Generator().manual_seed(taps)
    lens = [301, 1, 6, 2, 131]
    extra = 9
    u = [torch.randn(n + extra, C, generator=g).to(din) for n in lens]
    w = (0.5 * torch.randn(C, taps, generator=g)).to(BF16)
    refs = [q64(x, din) + P.causal_conv(q64(x, din), q64(w, BF16)) for x in u]
    state = torch.zeros(5, taps - 1, C, dtype=torch.float32, device=DEV)
    at = [0] * 5
    for step in ([(i, n) for i, n in enumerate(lens)], [(0, 3), (2, 1), (4, 5)], [(i, 1) for i in range(5)], [(i, 1) for i in (4, 1, 0)]):
        rows = torch.cat([u[i][at[i]:at[i] + n] for i, n in step]).to(DEV)
        slot_of, cu, slots = packed(step)
        y, cp = torch.empty(rows.shape[0], C, dtype=BF16, device=DEV), torch.empty(rows.shape[0], C, dtype=BF16, device=DEV)
        o.causal_conv(rows, 0, C, w.to(DEV), None, state, y, slot_of, cu, slots, len(step), single_tokens=all(n == 1 for _, n in step),
                      act=o.CONV_ACT_NONE, add_input=True, copy=cp)
        want = torch.cat([refs[i][at[i]:at[i] + n] for i, n in step])
        assert rel_err(y, want) < 1e-2, (taps, step)
        assert torch.equal(cp.cpu(), rows.to(BF16).cpu())
        for i, n in step:
            at[i] += n


def test_convolution_keeps_silu_and_bias_for_the_state_space_part():
    o = ops()
    C, taps = 20, 4
    g = torch.Generator().manual_seed(1)
    u, w, b = torch.randn(11, C, generator=g), torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    state = torch.zeros(2, taps - 1, C, dtype=torch.float32, device=DEV)
    y = torch.empty(11, C, dtype=torch.float32, device=DEV)
    slot_of, cu, slots = packed([(1, 11)])
    o.causal_conv(u.to(DEV), 0, C, w.to(DEV), b.to(DEV), state, y, slot_of, cu, slots, 1)
    assert rel_err(y, P.silu(P.causal_conv(u.to(F), w.to(F)) + b.to(F))) < 1e-5
    assert torch.allclose(state[1].cpu(), u[-3:])


# ------------------------------------------------------------------------------------------------
# the recurrence with one state value per channel
# ------------------------------------------------------------------------------------------------
def plain_scan(proj, C, bz, bu, S0):
    z = torch.sigmoid(proj[:, :C] + bz)
    cand = P.mingru_candidate(proj[:, C:2 * C] + bu)
    S, out = S0.clone(), []
    for t in range(proj.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out.append(S * P.silu(proj[t, 2 * C:3 * C]))
    return torch.stack(out), S


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("C", [1, 33, 100, 192])
def test_gated_scan_in_long_and_short_pieces_with_slow_and_fast_channels(dt, C):
    """Sequences of 1, 5, 300 and 1000 tokens in one step (the long ones are cut into segments that
    run side by side), then further pieces and single tokens from the state that step left.  Half of
    the channels forget slowly (a gate bias of -7), so the first tokens still weigh on the last."""
    o = ops()
    g = torch.Generator().manual_seed(C)
    lens = [1, 5, 300, 1000]
    slots = [3, 0, 5, 2]
    extra = 40
    proj = [torch.randn(n + extra, 3 * C + 2, generator=g).to(dt) for n in lens]
    bz = torch.where(torch.arange(C) % 2 == 0, torch.tensor(-7.0), torch.tensor(0.3)) + 0.1 * torch.randn(C, generator=g)
    bu = 0.5 * torch.randn(C, generator=g)
    refs = [plain_scan(q64(p, dt)[:, 2:], C, bz.to(F), bu.to(F), torch.zeros(C, dtype=F))[0] for p in proj]
    # the premise: without the first 100 tokens the last output of the long sequence is another
    late = plain_scan(q64(proj[3], dt)[100:, 2:], C, bz.to(F), bu.to(F), torch.zeros(C, dtype=F))[0]
    assert C == 1 or rel_err(late[-1 - extra:], refs[3][-1 - extra:]) > 1e-3
    state = torch.full((6, C), 7.0, dtype=torch.float32, device=DEV)
    state[slots] = 0.0                                   # what taking a slot does
    at = [0] * 4
    for step in ([(i, n) for i, n in enumerate(lens)], [(2, 17), (3, 2)], [(0, 1), (1, 1), (2, 1), (3, 1)], [(3, 20), (1, 3)]):
        rows = torch.cat([proj[i][at[i]:at[i] + n] for i, n in step]).to(DEV)
        _, cu, sl = packed([(slots[i], n) for i, n in step])
        y = torch.empty(rows.shape[0], C, dtype=dt, device=DEV)
        o.gated_scan(rows, 2, 2 + C, 2 + 2 * C, C, bz.to(DEV), bu.to(DEV), y, state, cu, sl, len(step), max(n for _, n in step))
        want = torch.cat([refs[i][at[i]:at[i] + n] for i, n in step])
        assert rel_err(y, want) < (2e-5 if dt == F32 else 1.5e-2), step
        for i, n in step:
            at[i] += n
    assert torch.all(state[[1, 4]] == 7.0)               # other slots' state is not touched


def test_gated_scan_without_output_gate_and_with_the_identity_candidate():
    o = ops()
    C = 10
    g = torch.Generator().manual_seed(0)
    proj = torch.randn(50, 2 * C, generator=g)
    state = torch.zeros(1, C, dtype=torch.float32, device=DEV)
    y = torch.empty(50, C, dtype=torch.float32, device=DEV)
    _, cu, sl = packed([(0, 50)])
    o.gated_scan(proj.to(DEV), 0, C, None, C, None, None, y, state, cu, sl, 1, 50, cand=o.SCAN_CAND_IDENTITY)
    z, u = torch.sigmoid(proj[:, :C].to(F)), proj[:, C:].to(F)
    Sv, rows = torch.zeros(C, dtype=F), []
    for t in range(50):
        Sv = (1 - z[t]) * Sv + z[t] * u[t]
        rows.append(Sv)
    assert rel_err(y, torch.stack(rows)) < 1e-5 and rel_err(state[0], Sv) < 1e-5


# ------------------------------------------------------------------------------------------------
# what stands around a sublayer's output
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("gdt", [F32, BF16])
@pytest.mark.parametrize("width", [40, 128, 2050])
def test_gated_normed_scaled_add(gdt, width):
    o = ops()
    g = torch.Generator().manual_seed(width)
    x, y = torch.randn(9, width, generator=g), 3.0 * torch.randn(9, width, generator=g)
    logits, bias, w = (2.0 * torch.randn(9, width + 4, generator=g)).to(gdt), torch.randn(width, generator=g).to(gdt), torch.randn(width, generator=g).to(gdt)
    xd = x.to(DEV)
    o.norm_add(xd, y.to(DEV), w.to(DEV), 1e-5, mult=0.7, gate=logits.to(DEV)[:, 4:], gate_bias=bias.to(DEV))
    yy = y.to(F) * torch.sigmoid(q64(logits, gdt)[:, 4:] + q64(bias, gdt))
    assert rel_err(xd, x.to(F) + 0.7 * P.norm(yy, q64(w, gdt), 1e-5)) < 1e-5
    # without gate and factor it is the plain normed add
    xd = x.to(DEV)
    o.norm_add(xd, y.to(DEV), w.to(DEV), 1e-5)
    assert rel_err(xd, x.to(F) + P.norm(y.to(F), q64(w, gdt), 1e-5)) < 1e-5


@pytest.mark.parametrize("rows", [5, 700])
@pytest.mark.parametrize("width", [1024, 2048, 4096, 8192])
def test_gated_normed_scaled_add_of_wide_rows_few_and_many(rows, width):
    """The widths at which a thread keeps 1, 2, 4 and 8 groups of four values, in the form for few rows
    (everything asked for at once) and the form for many."""
    o = ops()
    g = torch.Generator().manual_seed(width + rows)
    x, y = torch.randn(rows, width, generator=g), 3.0 * torch.randn(rows, width, generator=g)
    logits, bias, w = (2.0 * torch.randn(rows, width, generator=g)).to(BF16), torch.randn(width, generator=g).to(BF16), (1.0 + 0.3 * torch.randn(width, generator=g)).to(BF16)
    xd = x.to(DEV)
    o.norm_add(xd, y.to(DEV), w.to(DEV), 1e-6, mult=0.4, gate=logits.to(DEV), gate_bias=bias.to(DEV))
    yy = y.to(F) * torch.sigmoid(q64(logits, BF16) + q64(bias, BF16))
    assert rel_err(xd, x.to(F) + 0.4 * P.norm(yy, q64(w, BF16), 1e-6)) < 1e-5


@pytest.mark.parametrize("odt", [F32, BF16])
@pytest.mark.parametrize("taps", [2, 3, 4])
@pytest.mark.parametrize("width", [40, 2048])
def test_gated_normed_add_that_also_makes_the_next_convolution(odt, taps, width):
    """Single-token steps: the kernel behind a sublayer also makes the input of the next one from the
    row it has just written and the slots' kept inputs, and moves those on; three steps in a row over
    slots 5, 0 and 3 (and a padding row) against the plain convolution over the rows so far."""
    o = ops()
    g = torch.Generator().manual_seed(taps * width)
    slots = [5, 0, 3]
    cw = (0.4 * torch.randn(width, taps, generator=g)).to(odt)
    nw, gb = (1.0 + 0.2 * torch.randn(width, generator=g)).to(odt), torch.randn(width, generator=g).to(odt)
    state = torch.zeros(6, taps - 1, width, dtype=torch.float32, device=DEV)
    seen = {s: [] for s in slots}                      # the rows of x each slot has brought so far
    slot_of = i32(slots + [-1])
    for step in range(3):
        x, y = torch.randn(4, width, generator=g), 2.0 * torch.randn(4, width, generator=g)
        gl = torch.randn(4, width, generator=g).to(odt)
        xd = x.to(DEV)
        h = torch.full((4, width), 7.0, dtype=odt, device=DEV)
        plain = torch.full((4, width), 7.0, dtype=odt, device=DEV)
        o.norm_add(xd, y.to(DEV), nw.to(DEV), 1e-5, mult=0.6, gate=gl.to(DEV), gate_bias=gb.to(DEV),
                   conv=(cw.to(DEV), state, slot_of, h, plain))
        want_x = x.to(F) + 0.6 * P.norm(y.to(F) * torch.sigmoid(q64(gl, odt) + q64(gb, odt)), q64(nw, odt), 1e-5)
        assert rel_err(xd, want_x) < 1e-5
        for r, s_ in enumerate(slots):
            seen[s_].append(xd[r].to(F).cpu())
            rows = torch.stack(seen[s_])
            want_h = (rows + P.causal_conv(rows, q64(cw, odt)))[-1]
            assert rel_err(h[r], want_h) < (1e-5 if odt == F32 else 1e-2), (step, r)
            assert torch.equal(plain[r].cpu(), xd[r].to(odt).cpu())
            kept = rows[-(taps - 1):]
            assert torch.allclose(state[s_][taps - 1 - kept.shape[0]:].cpu().to(F), kept)
        assert torch.all(h[3] == 7.0) and torch.all(state[[1, 2, 4]] == 0.0)      # the padding row and other slots are left alone


def test_bias_with_gelu_and_gates_in_whole_groups_of_eight():
    o = ops()
    g = torch.Generator().manual_seed(8)
    for rows, cols, fill_cols in ((3, 512, 128), (300, 3072, 1024), (64, 64, 256)):
        u, b, b2 = (2.0 * torch.randn(rows, cols, generator=g)).to(BF16), torch.randn(cols, generator=g).to(BF16), torch.randn(fill_cols, generator=g).to(BF16)
        ud = u.to(DEV)
        fill = torch.full((rows, fill_cols + 8), 9.0, dtype=torch.float32, device=DEV)
        o.bias_act(ud, b.to(DEV), ud, fill=fill[:, :fill_cols], fill_bias=b2.to(DEV))        # in place, as the feed-forward runs it
        assert rel_err(ud, P.gelu_tanh(q64(u, BF16) + q64(b, BF16))) < 1e-2
        assert torch.equal(fill[:, :fill_cols].cpu(), b2.float().expand(rows, fill_cols)) and torch.all(fill[:, fill_cols:] == 9.0)
        for group in (1, 64):
            x, gl = torch.randn(rows, cols, generator=g).to(BF16), torch.randn(rows, cols // group, generator=g).to(BF16)
            xd = x.to(DEV)
            o.sigmoid_gate(xd, gl.to(DEV), group)
            assert rel_err(xd, q64(x, BF16) * torch.sigmoid(q64(gl, BF16)).repeat_interleave(group, dim=1)) < 1e-2


@pytest.mark.parametrize("dt", [F32, BF16])
def test_bias_with_tanh_gelu_and_the_gates_per_value_and_per_head(dt):
    o = ops()
    g = torch.Generator().manual_seed(4)
    u, b, b2 = (2.0 * torch.randn(7, 300, generator=g)).to(dt), torch.randn(300, generator=g).to(dt), torch.randn(520, generator=g).to(dt)
    y = torch.empty(7, 300, dtype=dt, device=DEV)
    fill = torch.full((7, 524), 9.0, dtype=torch.float32, device=DEV)
    o.bias_act(u.to(DEV), b.to(DEV), y, fill=fill[:, :520], fill_bias=b2.to(DEV))
    assert rel_err(y, P.gelu_tanh(q64(u, dt) + q64(b, dt))) < (1e-5 if dt == F32 else 1e-2)
    assert torch.equal(fill[:, :520].cpu(), b2.float().expand(7, 520)) and torch.all(fill[:, 520:] == 9.0)
    for group in (1, 12):
        x, gl = torch.randn(5, 36, generator=g).to(dt), torch.randn(5, 36 // group + 3, generator=g).to(dt)
        xd = x.to(DEV)
        o.sigmoid_gate(xd, gl.to(DEV)[:, 3:], group)
        want = q64(x, dt) * torch.sigmoid(q64(gl, dt)[:, 3:]).repeat_interleave(group, dim=1)
        assert rel_err(xd, want) < (1e-5 if dt == F32 else 1e-2)


# ------------------------------------------------------------------------------------------------
# whole models
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_whole_prompts_and_every_layer(name, dtype):
    from builderforce_inference_b200.engine.context import build_context
    eng, cfg, w = engine(name, dtype)
    ids = prompts(cfg["vocab"], [230], 5)[0]
    ref, layers = P.forward(cfg, w, ids, keep_layers=True)
    slot = eng.acquire()
    assert close(eng.step([S(slot, ids)]), ref, dtype)
    eng.release(slot)
    slot = eng.acquire()
    eng.cache.begin_step([slot], [len(ids)])
    ctx = build_context([(slot, 0, ids)], eng.dtype, eng.workspace, eng.device, eng.status)
    x = eng.decoder.embed(ctx, eng.cache)
    for i in range(len(cfg["layers"])):
        eng.decoder.run_layers(ctx, x, eng.cache, i, i + 1)
        assert close(x, layers[i], dtype), i
    eng.cache.end_step([slot], [len(ids)])
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_prompt_then_token_by_token_over_several_pages(name, dtype, graphs):
    eng, cfg, w = engine(name, dtype, use_graphs=graphs)
    ids = prompts(cfg["vocab"], [215], 40)[0]
    ref = P.forward(cfg, w, ids)
    slot = eng.acquire()
    head = 3
    outs = [eng.step([S(slot, ids[:head])]).clone()]
    for t in ids[head:]:
        outs.append(eng.step([S(slot, [t])]).clone())
    assert close(torch.cat(outs), ref, dtype)
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_portions_of_a_prompt_down_to_two_tokens(name, dtype):
    eng, cfg, w = engine(name, dtype)
    ids = prompts(cfg["vocab"], [201], 70)[0]
    ref = P.forward(cfg, w, ids)
    for cuts in ([2, 2, 3, 64, 65, 63, 2], [128, 73], [1, 7, 1, 130, 62], [1, 200], [193, 2, 6], [23, 1, 1, 25, 50, 101]):
        slot = eng.acquire()
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([S(slot, ids[at:at + c])]).clone())
            at += c
        assert at == len(ids)
        assert close(torch.cat(outs), ref, dtype), cuts
        eng.release(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_unequal_batches_reused_slots_and_poisoned_pages(name, dtype):
    eng, cfg, w = engine(name, dtype, max_tokens=1024)
    eng.cache.poison()
    lengths = [70, 5, 131, 1]
    seqs = prompts(cfg["vocab"], [n + 6 for n in lengths], 100)
    refs = [P.forward(cfg, w, s) for s in seqs]
    for round_ in range(2):                               # the second round runs in slots and pages that were used
        slots = [eng.acquire() for _ in seqs]
        got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lengths)])
        assert close(got, torch.cat([r[:n] for r, n in zip(refs, lengths)]), dtype), round_
        live = list(range(len(seqs)))
        for step in range(6):                             # decoded together; the shortest leave first
            got = eng.step([S(slots[i], [seqs[i][lengths[i] + step]]) for i in live])
            assert close(got, torch.stack([refs[i][lengths[i] + step] for i in live]), dtype), (round_, step)
            if step in (1, 3):
                eng.release(slots[live.pop(1)])
        for i in live:
            eng.release(slots[i])
        eng.cache.check()
        eng.cache.poison()
        seqs, refs, lengths = seqs[::-1], refs[::-1], lengths[::-1]     # other sequences in the slots the first round used


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_middling_sizes_whole_in_portions_and_decoded(dtype):
    """Width 512, heads of 64 and 128, a latent of 128 + 32, a minGRU of 768: the sizes at which the
    bfloat16 run takes the tensor-core products and every kernel its 16-byte form."""
    cfg = config(1000, 512, 1e-6, 22.6, 0.8, 3, [
        with_mlp(att(8, 2, 64, 64, 4, 0.125, 150, rot(1e4, 64), v_mix=True), 1536),
        with_mlp(lat(8, 64, 32, 64, 128, 192, 0.1, rot(1e5, 32, (8.0, 128, 16.0, 1.0))), 1024),
        with_mlp(gru(768), 1536),
        with_mlp(att(4, 2, 128, 64, 2, 0.09, 64, rot(5e5, 32), v_mix=True), None),
        with_mlp(lat(4, 32, 64, 128, 256, 96, 0.1, rot(1e4, 64)), 2048)])
    eng, w = engine_of(cfg, 7, dtype, max_tokens=4096)
    seqs = prompts(1000, [390, 17], 3)
    refs = [P.forward(cfg, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    outs = [[], []]
    got = eng.step([S(slots[0], seqs[0][:300]), S(slots[1], seqs[1][:9])])
    outs[0].append(got[:300].clone()), outs[1].append(got[300:].clone())
    got = eng.step([S(slots[0], seqs[0][300:380]), S(slots[1], seqs[1][9:13])])
    outs[0].append(got[:80].clone()), outs[1].append(got[80:].clone())
    for k in range(4):
        got = eng.step([S(slots[0], [seqs[0][380 + k]]), S(slots[1], [seqs[1][13 + k]])])
        outs[0].append(got[:1].clone()), outs[1].append(got[1:].clone())
    for k in range(4, 10):
        outs[0].append(eng.step([S(slots[0], [seqs[0][380 + k]])]).clone())
    assert close(torch.cat(outs[0]), refs[0], dtype) and close(torch.cat(outs[1]), refs[1], dtype)
    for sl in slots:
        eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_cut_into_micro_batches_of_64_tokens(dtype):
    """The engine cuts a step of many tokens into micro-batches; with 64 tokens each the cuts fall
    inside the sequences, between them and at a chunk's edge, and every state has to carry over."""
    eng, cfg, w = engine("odd", dtype, prefill_chunk_tokens=64)
    seqs = prompts(cfg["vocab"], [200, 70, 3, 64], 13)
    refs = [P.forward(cfg, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    got = eng.step([S(sl, s) for sl, s in zip(slots, seqs)])
    assert close(got, torch.cat(refs), dtype)
    for sl in slots:
        eng.release(sl)
    eng.cache.check()


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


# ------------------------------------------------------------------------------------------------
# chunk edges, far tokens and the first tokens
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunk", [40, 64, 100])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_token_just_inside_and_just_outside_the_chunk(chunk, decoded):
    """One attention layer (two taps in front of the sublayers, two on q, k and v, no feed-forward),
    so position i reads tokens i - 2 .. i directly and, through the keys, tokens from two before its
    chunk's first position on.  Changing the third token before the chunk changes nothing at the
    chunk's last position; changing the chunk's first token does.  In a prompt, and with the last
    chunk decoded token by token (its first token then arrives alone, pages and chunk edges apart)."""
    cfg = config(97, 32, 3e-6, 2.0, 0.65, 2, [with_mlp(att(4, 2, 8, 12, 2, 0.5, chunk, rot(1e4, 8), v_mix=True), None)])
    eng, w = engine_of(cfg, 11)
    n_chunks = 3
    i = n_chunks * chunk - 1                   # the last position of the third chunk
    first = (n_chunks - 1) * chunk
    ids = prompts(97, [i + 1], chunk)[0]

    def run(tokens):
        sl = eng.acquire()
        if decoded:
            eng.step([S(sl, tokens[:first - 1], [])])
            out = torch.cat([eng.step([S(sl, [t])]) for t in tokens[first - 1:]])[-1:].clone()
        else:
            out = eng.step([S(sl, tokens, [i])]).clone()
        eng.release(sl)
        return out

    base, ref = run(ids), P.forward(cfg, w, ids)[i:i + 1]
    assert rel_err(base, ref) < 3e-5
    outside = list(ids)
    outside[first - 3] = (ids[first - 3] + 1) % 97
    assert rel_err(run(outside), base) < 1e-6
    assert rel_err(P.forward(cfg, w, outside)[i:i + 1], ref) < 1e-9
    inside = list(ids)
    inside[first] = (ids[first] + 1) % 97
    ref_in = P.forward(cfg, w, inside)[i:i + 1]
    assert rel_err(ref_in, ref) > 1e-4                     # the premise: the chunk's first token matters at its last
    assert rel_err(run(inside), ref_in) < 3e-5
    # the first position of a chunk sees itself only (and what the convolutions reach)
    assert rel_err(eng_first(eng, ids, first), P.forward(cfg, w, ids)[first:first + 1]) < 3e-5


def eng_first(eng, ids, pos):
    sl = eng.acquire()
    out = eng.step([S(sl, ids[:pos + 1], [pos])]).clone()
    eng.release(sl)
    return out


@pytest.mark.parametrize("kind", ["latent", "gru"])
def test_the_first_token_reaches_a_position_hundreds_of_tokens_on(kind):
    """One layer of latent attention (every earlier key is read; the positions pass 4 times the
    length the frequency scaling starts from), or a minGRU whose gates are biased towards keeping:
    changing the sequence's first token changes the logits 330 tokens on, through a prompt and
    through tokens decoded one by one."""
    if kind == "latent":
        cfg = config(97, 32, 3e-6, 2.0, 0.55, 3, [with_mlp(lat(3, 8, 8, 8, 16, 12, 0.6, rot(1e4, 8, (4.0, 64, 32.0, 1.0))), 24)])
    else:
        cfg = config(97, 32, 3e-6, 2.0, 0.55, 3, [with_mlp(gru(48), 24)])
    w32 = make_weights(cfg, 5, F32)
    if kind == "gru":
        w32["l0.mix.z"] = w32["l0.mix.z"] * 0.05             # gates near 0.001 whatever the token
        w32["l0.mix.z.b"] = w32["l0.mix.z.b"] * 0.1 - 7.0
    from builderforce_inference_b200.engine.engine import Engine
    eng = Engine.load(write_folder(cfg, w32), dtype="float32", max_tokens=1024)
    w = {k: v.to(F) for k, v in w32.items()}
    n = 331
    ids = prompts(97, [n], seed=77)[0]
    other = [(ids[0] + 1) % 97] + ids[1:]
    sl = eng.acquire()
    a = eng.step([S(sl, ids, [n - 1])]).clone()
    eng.release(sl)
    sl = eng.acquire()
    eng.step([S(sl, other[:n - 40], [])])
    b = torch.cat([eng.step([S(sl, [t])]) for t in other[n - 40:]])[-1:].clone()
    eng.release(sl)
    ref_a, ref_b = P.forward(cfg, w, ids)[n - 1:], P.forward(cfg, w, other)[n - 1:]
    assert rel_err(a, ref_a) < 3e-5 and rel_err(b, ref_b) < 3e-5
    assert rel_err(ref_a, ref_b) > 3e-4                    # the test's premise: the far token matters


# ------------------------------------------------------------------------------------------------
# configurations drawn at random
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("seed", range(101, 117))
def test_random_configurations_in_float32(seed):
    """Configurations drawn from a seed (layer order, every size, taps, chunks, rotation, mixing
    layers, with and without feed-forward): an unequal batch of prompts, five tokens decoded
    together, and the longest prompt again in portions, against the plain implementation."""
    cfg = random_config(seed)
    eng, w = engine_of(cfg, seed)
    lens = [(1, 5, 70, 130, 260)[seed % 5], (2, 33, 200)[seed % 3], (1, 64, 129)[seed % 2]]
    seqs = prompts(cfg["vocab"], [n + 5 for n in lens], seed)
    refs = [P.forward(cfg, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        assert rel_err(got[at:at + n], refs[i][:n]) < 1e-4, (i, cfg)
        at += n
    for step in range(5):
        got = eng.step([S(sl, [s[n + step]]) for sl, s, n in zip(slots, seqs, lens)])
        for i, n in enumerate(lens):
            assert rel_err(got[i:i + 1], refs[i][n + step:n + step + 1]) < 1e-4, (i, step, cfg)
    for sl in slots:
        eng.release(sl)
    i = max(range(3), key=lambda k: lens[k])
    sl, outs, at = eng.acquire(), [], 0
    for c in [max(1, lens[i] // 3), 2, 1, 97, 10 ** 6]:
        c = min(c, lens[i] - at)
        if c > 0:
            outs.append(eng.step([S(sl, seqs[i][at:at + c])]).clone())
            at += c
    assert rel_err(torch.cat(outs), refs[i][:lens[i]]) < 1e-4, cfg
    eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("seed", [201, 202, 203, 204])
def test_random_configurations_in_bfloat16(seed):
    cfg = random_config(seed)
    eng, w = engine_of(cfg, seed, "bfloat16")
    ids = prompts(cfg["vocab"], [150], seed)[0]
    ref = P.forward(cfg, w, ids)
    sl = eng.acquire()
    outs = [eng.step([S(sl, ids[:100])]).clone(), eng.step([S(sl, ids[100:140])]).clone()]
    outs += [eng.step([S(sl, [t])]).clone() for t in ids[140:]]
    assert close(torch.cat(outs), ref, "bfloat16"), cfg
    eng.release(sl)


# ------------------------------------------------------------------------------------------------
# the public entry points
# ------------------------------------------------------------------------------------------------
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
        ref = P.forward(cfg, w, p + got)
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
    ra, rb = P.forward(cfg, w, a), P.forward(cfg, w, b)
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
    ref = P.forward(cfg, w, a[:12] + new)
    assert [int(torch.argmax(ref[11 + i])) for i in range(6)] == new
