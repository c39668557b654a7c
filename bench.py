"""Benchmark: decode and prefill throughput of the Qwen3-4B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the default batch (8), timed on
the device over K single-token steps after W warm-up steps; ``e2e`` is the same through
``Model.generate_batch`` with host token ids in and out (``e2e_b1``: at batch 1); ``prefill`` is a
2,048-token prompt, with a breakdown of one instrumented step by kernel class; ``points`` holds
decode at batch 1 and 64; ``decode_points`` holds, for batch 1, 8 and 64, a point right after the
prompts (lengths uniform in [128, 2048]) and a point with every sequence at 4,080 to 4,096 tokens,
the end of the benchmark's context, each with its step time, mean context, bytes and fraction of
the memory bandwidth; ``roofline`` relates the main decode step to the memory bandwidth.  The model
has the layer sizes of the benchmark configuration with random weights and synthetic token ids;
``--layers`` runs fewer layers of the same sizes (``config`` names both).

``--model 8b`` and ``--model 32b`` run the workloads named for those shapes instead (an unequal
batch of 16 prompts of 64 to 4,096 tokens with 256 decode steps and an 8,192-token prompt; decode
at batch 1 and 32 behind 2,048-token prompts and a 2,048-token prompt) and print one line each.

``--design datasun`` leaves the benchmark aside and runs the Datasun design (parallel blocks,
three lightning-attention layers to one windowed softmax-attention layer) beside Qwen3 at equal
layer sizes, a few sizes, random weights: a 2,048-token prompt with its breakdown by kernel class,
and decode at batch 8 and 64 behind 1,024-token prompts.  One line.  ``--design bepilorn`` does
the same for the Bepilorn design (three state-space layers to one pair of chunked sink attention
and gated linear attention, a routed feed-forward) beside Datasun and Qwen3, with the milliseconds
of every kernel of a prompt step and of a single-token step.  ``--design munerax`` and
``--design kikelorn`` do it for those designs (Kikelorn: chunked attention, latent attention with a
query latent, a minGRU and chunked attention again, in out-norm blocks) beside the designs closest
to them and Qwen3.

The work is one GPU's: for ``--gpus`` above 1 it says so and exits with 2.  The reference arm
(``--impl reference``) is unavailable: the reference is a Rust workspace, there is no Rust
toolchain or network here to build it, and its CUDA path runs none of its kernels for bfloat16
weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (Qwen3-4B shape)
CONFIG_4B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=2560,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728,
                 vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 max_position_embeddings=40960)
# the other shapes of the same architecture, for runs beside the benchmark (``--model``)
SHAPES = {
    "4b": CONFIG_4B,
    "8b": dict(CONFIG_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(CONFIG_4B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600,
                tie_word_embeddings=False),
}
FULL_LAYERS = 36
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS)
    src = "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            for k in out:
                if isinstance(data.get(k), (int, float)) and data[k] > 0:
                    out[k] = float(data[k])
            src = "measured"
        except (OSError, ValueError):
            pass
    out["source"] = src
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0, set()
        for p in self.samples:
            try:
                sm.append(int(float(p[0])))
                mx = max(mx, int(float(p[1])))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def decode_run(model, batch, steps, warmup, seed, lens=None):
    """One varlen prefill (untimed), then warm-up and timed single-token steps; device-timed.
    ``lens``: the prompts' lengths (default: uniform in [128, 2048])."""
    import torch
    from builderforce_inference_b200.engine.engine import SequenceStep
    eng = model.engine
    g = torch.Generator().manual_seed(seed)
    vocab = eng.spec.vocab_size
    if lens is None:
        lens = torch.randint(128, 2049, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    slots = [eng.acquire() for _ in range(batch)]
    eng.step([SequenceStep(s, p, ()) for s, p in zip(slots, prompts)], check=False)
    toks = [int(t) for t in torch.randint(0, vocab, (batch,), generator=g).tolist()]

    def one():
        return eng.step([SequenceStep(s, (t,), (0,)) for s, t in zip(slots, toks)], check=False)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    bytes_before = eng.decode_step_bytes()
    launches0 = eng.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = eng.kernel_launches() - launches0
    step_bytes = (bytes_before + eng.decode_step_bytes()) / 2.0
    eng.check_status()
    ctx_mean = sum(eng.length(s) for s in slots) / batch
    for s in slots:
        eng.release(s)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launches,
            "step_bytes": step_bytes, "ctx_mean": ctx_mean}


def point(run, pk):
    """A decode point as it goes into the line: rate, step time, mean context at the end of the
    timed steps, the bytes a step has to read and their rate as a fraction of the copy bandwidth."""
    gbs = run["step_bytes"] / (run["ms_per_step"] / 1e3) / 1e9
    return {"tok_s": round(run["tok_s"], 1), "ms_per_step": round(run["ms_per_step"], 4),
            "ctx_mean": round(run["ctx_mean"], 1), "step_bytes": int(run["step_bytes"]),
            "gb_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}


def e2e_run(model, batch, steps, warmup, seed):
    """The same through ``Model.generate_batch``: host ids in, host ids out, every step."""
    import torch
    from builderforce_inference_b200 import SampleParams
    g = torch.Generator().manual_seed(seed)
    vocab = model.n_vocab()
    lens = torch.randint(128, 2049, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
    stamps = []
    model.stepper.on_tokens = lambda n: stamps.append((time.perf_counter(), n))
    try:
        model.generate_batch(prompts, SampleParams(max_tokens=warmup + steps + 1), ignore_eos=True)
    finally:
        model.stepper.on_tokens = None
    # stamps[0] follows the prefill; stamps[i] follows decode step i
    t0, t1 = stamps[warmup][0], stamps[warmup + steps][0]
    tokens = sum(n for _, n in stamps[warmup + 1:warmup + steps + 1])
    return {"tok_s": tokens / (t1 - t0), "h2d": model.stepper.h2d_bytes, "d2h": model.stepper.d2h_bytes}


def prefill_flops(c, layers, lens):
    """Floating-point operations of one prompt step over sequences of ``lens`` tokens, logits at
    each sequence's last token."""
    h, d, nq, nkv, inter = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"], \
        c["intermediate_size"]
    tokens = sum(lens)
    per_layer = 2 * tokens * (h * (nq + 2 * nkv) * d + nq * d * h + 3 * h * inter)
    attn = sum(4 * nq * d * n * (n + 1) / 2 for n in lens)
    return layers * (per_layer + attn) + 2 * h * c["vocab_size"] * len(lens)


KERNEL_CLASSES = (("products", ("gemm", "skinny")), ("attention", ("attention",)),
                  ("recurrence", ("lightning", "decay_scan", "causal_conv")), ("experts", ("moe_",)))


def prefill_breakdown(eng, step, by_kernel=False):
    """One instrumented prompt step: a CUDA event before and after every kernel, so the kernels run
    strictly one after the other (an event between two launches ends their overlap).  Returns the
    milliseconds by kernel class, the time between kernels (the GPU waiting for the host), and the
    whole of the instrumented step, which is therefore longer than a plain one."""
    import torch
    from builderforce_inference_b200.kernels import library as L
    marks, open_ = [], []

    def watch(name, what):
        if what == "begin":
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            open_.append(e)
        else:
            e0 = open_.pop()
            if what == "end":
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                marks.append((name, e0, e1))

    torch.cuda.synchronize()
    L.set_call_observer(watch)
    try:
        step()
    finally:
        L.set_call_observer(None)
    torch.cuda.synchronize()
    out = {"products_ms": 0.0, "attention_ms": 0.0, "other_ms": 0.0}
    for name, e0, e1 in marks:
        cls = next((c for c, keys in KERNEL_CLASSES if any(k in name for k in keys)), "other")
        out[cls + "_ms"] = out.get(cls + "_ms", 0.0) + e0.elapsed_time(e1)
    whole = marks[0][1].elapsed_time(marks[-1][2]) if marks else 0.0
    out["gaps_ms"] = max(0.0, whole - sum(out.values()))
    out = {k: round(v, 3) for k, v in out.items()}
    out["instrumented_ms"] = round(whole, 3)
    out["kernels"] = len(marks)
    if by_kernel:
        names = {}
        for name, e0, e1 in marks:
            names[name] = names.get(name, 0.0) + e0.elapsed_time(e1)
        out["by_kernel_ms"] = {k.replace("bfi_", ""): round(v, 3) for k, v in sorted(names.items(), key=lambda kv: -kv[1])}
    return out


def prefill_run(model, tokens, reps, layers, c=None, lens=None, breakdown=False, by_kernel=False):
    import torch
    from builderforce_inference_b200.engine.engine import SequenceStep
    eng = model.engine
    g = torch.Generator().manual_seed(99)
    lens = lens or [tokens]
    prompts = [torch.randint(0, eng.spec.vocab_size, (n,), generator=g).tolist() for n in lens]
    times = []

    def run_once():
        slots = [eng.acquire() for _ in prompts]
        try:
            eng.step([SequenceStep(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)], check=False)
        finally:
            torch.cuda.synchronize()
            for s in slots:
                eng.release(s)

    for i in range(reps + 2):
        slots = [eng.acquire() for _ in prompts]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        eng.step([SequenceStep(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)], check=False)
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(e0.elapsed_time(e1))
        for s in slots:
            eng.release(s)
    ms = statistics.median(times)
    out = {"ms": ms, "tok_s": sum(lens) / (ms / 1e3), "flops": prefill_flops(c or CONFIG_4B, layers, lens)}
    if breakdown:
        out["breakdown"] = prefill_breakdown(eng, run_once, by_kernel)
    return out


def side_run(a, model, shape_cfg, pk) -> dict:
    """The workloads named for the 8B and 32B shapes, beside the benchmark: one line of numbers."""
    layers = a.layers
    out = {}
    if a.shape_name == "8b":
        lens = [64 + round(i * (4096 - 64) / 15) for i in range(16)]            # 64 .. 4,096, then 256 more each
        pf = prefill_run(model, 0, 3, layers, shape_cfg, lens=lens)
        out["unequal16_prefill"] = {"tokens": sum(lens), "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                                    "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        decode_run(model, 16, 2, 3, seed=3, lens=lens)
        out["unequal16_decode256"] = point(decode_run(model, 16, 256, 3, seed=4, lens=lens), pk)
        pf = prefill_run(model, 8192, 3, layers, shape_cfg)
        out["prefill_8192"] = {"tokens": 8192, "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                               "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    else:
        for b in (1, 32):
            decode_run(model, b, 2, 3, seed=3, lens=[2048] * b)
            out[f"decode_b{b}_prompt2048"] = point(decode_run(model, b, 32, 3, seed=4, lens=[2048] * b), pk)
        pf = prefill_run(model, 2048, 3, layers, shape_cfg)
        out["prefill_2048"] = {"tokens": 2048, "ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1),
                               "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    return out


# layer sizes for the runs of one design beside another (``--design``): width, heads, kv heads, head size, inner size
DESIGN_SIZES = {"w2048": (2048, 16, 4, 128, 6144), "w2560": (2560, 32, 8, 128, 9728), "w4096": (4096, 32, 8, 128, 12288)}
DESIGN_VOCAB = 32768
DESIGN_WINDOW = 1024


def datasun_config(width, heads, kv, d, ff, layers):
    """A Datasun model of these layer sizes: every fourth layer windowed softmax attention, the
    others lightning attention with head decays between 1 - 2^-5 and 1 - 2^-8."""
    light = {"heads": heads, "dim": d, "vdim": d, "decay": [1.0 - 2.0 ** -(5.0 + 3.0 * i / max(heads - 1, 1)) for i in range(heads)]}
    att = {"heads": heads, "kv_heads": kv, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": DESIGN_WINDOW},
           "rot": {"base": 1e6, "dims": d // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    return {"architecture": "Datasun", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [{"type": "attention" if i % 4 == 3 else "lightning", "mixer": att if i % 4 == 3 else light, "mlp": mlp}
                       for i in range(layers)]}


BEPILORN_EXPERTS = 16          # experts of the routed feed-forward in the design runs; 4 are used, in 4 groups of which 2 are kept


def bepilorn_config(width, heads, kv, d, ff, layers):
    """A Bepilorn model of these layer sizes: every fourth layer the pair of chunked sink attention
    and gated linear attention, the others state-space layers whose heads have the attention's
    sizes; a routed feed-forward whose four used experts and shared expert together have the dense
    feed-forward's inner size."""
    ssm = {"heads": heads, "vdim": d, "state": d, "groups": kv, "conv": 4, "norm_groups": kv}
    pair = {"left": {"heads": heads, "kv_heads": kv, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": DESIGN_WINDOW},
                     "rot": {"base": 1e6, "dims": d // 2}},
            "right": {"heads": heads, "dim": d, "vdim": d, "tau": 8.0, "rank": 64}, "left_scale": 0.5, "right_scale": 1.0}
    expert_ff = ff // 6 // 128 * 128            # a sixth of the dense inner size, in whole tiles
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": ff - 4 * expert_ff},
           "router": {"experts": BEPILORN_EXPERTS, "top": 4, "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Bepilorn", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
            "layers": [{"type": "parallel" if i % 4 == 3 else "mamba2", "mixer": pair if i % 4 == 3 else ssm, "mlp": mlp}
                       for i in range(layers)]}


MUNERAX_LATENT = 512           # values of the cached latent in the design runs; 64 more are the shared rotated key part


def munerax_config(width, heads, kv, d, ff, layers):
    """A Munerax model of these layer sizes: latent attention whose heads have half of the
    attention's head size unrotated and half rotated, values of the attention's head size, and a
    cache row of 512 + d/2 values; every fourth layer reads the cache of the layer before it; the
    first layer's feed-forward is dense, the others' routed as Bepilorn's in these runs."""
    half = d // 2
    expert_ff = ff // 6 // 128 * 128
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": ff - 4 * expert_ff},
           "router": {"experts": BEPILORN_EXPERTS, "top": 4, "scale": 1.0, "groups": {"count": 4, "keep": 2}}}
    out = []
    for i in range(layers):
        mixer = {"heads": heads, "dim": half, "rot_dim": half, "vdim": d, "kv_rank": MUNERAX_LATENT, "scale": d ** -0.5,
                 "rot": {"base": 1e6, "dims": half}}
        if i % 4 == 3:
            mixer["kv_from"] = i - 1
        out.append({"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe})
    return {"architecture": "Munerax", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}}, "layers": out}


KIKELORN_TAPS = 4              # taps of the convolutions in the design runs, in front of the sublayers and on q, k, v


def kikelorn_config(width, heads, kv, d, ff, layers):
    """A Kikelorn model of these layer sizes: of every four layers the first and the last are
    chunked attention (values of the keys' size, four taps on q, k and v, values mixed with the first
    layer's), the second is latent attention as Munerax's in these runs (a cache row of 512 + d/2
    values) with a query latent of 3/8 of the width, the third a minGRU of 3/2 of the width; a dense
    feed-forward with biases in every layer."""
    half = d // 2
    att = {"heads": heads, "kv_heads": kv, "dim": d, "vdim": d, "conv": KIKELORN_TAPS, "scale": d ** -0.5,
           "mask": {"size": DESIGN_WINDOW}, "rot": {"base": 1e6, "dims": half}, "v_mix": True}
    lat = {"heads": heads, "dim": half, "rot_dim": half, "vdim": d, "kv_rank": MUNERAX_LATENT, "q_rank": 3 * width // 8,
           "scale": d ** -0.5, "rot": {"base": 1e6, "dims": half, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    gru = {"width": 3 * width // 2}
    kinds = [("attention", att), ("latent_attention", lat), ("mingru", gru), ("attention", att)]
    return {"architecture": "Kikelorn", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "canon": {"taps": KIKELORN_TAPS},
            "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": {"kind": "dense", "ff": ff}} for i in range(layers)]}


def decode_breakdown(model, batch, ctx_len):
    """One instrumented single-token step (no graph, an event around every kernel) behind prompts of
    ``ctx_len`` tokens: milliseconds by kernel."""
    import torch
    from builderforce_inference_b200.engine.engine import SequenceStep
    eng = model.engine
    g = torch.Generator().manual_seed(7)
    slots = [eng.acquire() for _ in range(batch)]
    eng.step([SequenceStep(s, torch.randint(0, eng.spec.vocab_size, (ctx_len,), generator=g).tolist(), ()) for s in slots], check=False)
    graphs, eng.use_graphs = eng.use_graphs, False
    try:
        def one():
            eng.step([SequenceStep(s, (1,), (0,)) for s in slots], check=False)
        one()
        return prefill_breakdown(eng, one, by_kernel=True)
    finally:
        eng.use_graphs = graphs
        for s in slots:
            eng.release(s)


def design_run(a) -> int:
    import torch
    from builderforce_inference_b200 import Model
    pk = peaks()
    layers = a.layers or 8
    clocks = ClockSampler()
    clocks.start()
    out = {}
    for name in (a.sizes.split(",") if a.sizes else sorted(DESIGN_SIZES)):
        width, heads, kv, d, ff = DESIGN_SIZES[name]
        qwen3 = dict(CONFIG_4B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads,
                     num_key_value_heads=kv, head_dim=d, intermediate_size=ff, vocab_size=DESIGN_VOCAB)
        if a.design == "kikelorn":      # beside the design with the same latent attention, the one with chunked attention and a recurrence, and the dense one
            configs = {"kikelorn": kikelorn_config(width, heads, kv, d, ff, layers),
                       "munerax": munerax_config(width, heads, kv, d, ff, layers),
                       "bepilorn": bepilorn_config(width, heads, kv, d, ff, layers), "qwen3": qwen3}
            if a.only:
                configs = {k: v for k, v in configs.items() if k in a.only.split(",")}
        elif a.design == "munerax":     # beside the routed design and beside the dense softmax-attention one
            configs = {"munerax": munerax_config(width, heads, kv, d, ff, layers),
                       "bepilorn": bepilorn_config(width, heads, kv, d, ff, layers), "qwen3": qwen3}
        elif a.design == "bepilorn":    # beside the closest design the package has, and beside the dense one
            configs = {"bepilorn": bepilorn_config(width, heads, kv, d, ff, layers),
                       "datasun": datasun_config(width, heads, kv, d, ff, layers), "qwen3": qwen3}
        else:
            configs = {"datasun": datasun_config(width, heads, kv, d, ff, layers), "qwen3": qwen3}
        for design, cfg in configs.items():
            model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=64 * 2048, max_seq_len=CONTEXT, max_batch=64)
            by_kernel = a.design in ("bepilorn", "munerax", "kikelorn")
            pf = prefill_run(model, PREFILL_TOKENS, 5, layers, breakdown=True, by_kernel=by_kernel)
            row = {"prefill_2048": {"ms": round(pf["ms"], 3), "tok_s": round(pf["tok_s"], 1), "breakdown": pf["breakdown"]}}
            for b in (8, 64):
                decode_run(model, b, 2, 3, seed=3, lens=[1024] * b)
                r = decode_run(model, b, 32, 3, seed=4, lens=[1024] * b)
                row[f"decode_b{b}"] = {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 4),
                                       "weight_bytes": int(model.engine.decoder.n_weight_bytes), "launches_per_step": r["launches"] // 32}
                if by_kernel:
                    row[f"decode_b{b}"]["breakdown"] = decode_breakdown(model, b, 1024)
            out.setdefault(name, {})[design] = row
            del model
            torch.cuda.empty_cache()
    pattern = {"datasun": "lightning x3, attention (window %d) x1" % DESIGN_WINDOW,
               "bepilorn": "state space x3, chunked attention (chunk %d) + gated linear attention x1; %d experts, 4 used, and a shared one"
                           % (DESIGN_WINDOW, BEPILORN_EXPERTS),
               "munerax": "latent attention (cache row %d + head/2) x4, the fourth reading the third's cache; dense feed-forward in "
                          "layer 0, then %d experts, 4 used, and a shared one" % (MUNERAX_LATENT, BEPILORN_EXPERTS),
               "kikelorn": "chunked attention (chunk %d, %d taps on q, k, v), latent attention (cache row %d + head/2, query latent), "
                           "minGRU, chunked attention; out-norm blocks with %d taps in front of every sublayer and a gate behind it; "
                           "dense feed-forward with biases" % (DESIGN_WINDOW, KIKELORN_TAPS, MUNERAX_LATENT, KIKELORN_TAPS)}[a.design]
    beside = {"bepilorn": "datasun and qwen3", "munerax": "bepilorn and qwen3",
              "kikelorn": "munerax, bepilorn and qwen3"}.get(a.design, "qwen3")
    print(json.dumps({"workloads": a.design + " beside " + beside
                      + " at equal layer sizes, builder-run beside the benchmark", "dtype": "bf16",
                      "layers": layers, "pattern": pattern, "vocab": DESIGN_VOCAB,
                      "peaks": pk["source"], "sizes": out, "clocks": clocks.stop()}))
    return 0


KERNEL_SHAPES = {"qkv": (6144, 2560, 0), "o": (2560, 4096, 1), "gateup": (19456, 2560, 2), "down": (2560, 9728, 1),
                 "head": (151936, 2560, 0)}


def kernel_run(a) -> int:
    """Times ONE kernel on one workload (for profiling under ncu and for the files in profiles/):
    ``--kernel skinny_gemm|gemm_tcgen05 --shape qkv|o|gateup|down|head --rows M`` or
    ``--kernel attention_decode|attention_prefill|attention_prefill_tcgen05 --rows B_or_T --ctx C``
    (``--seqs N``: N prompts of --rows tokens each),
    ``--kernel qk_norm_rope --rows T``, ``--kernel decay_scan --rows T [--seqs N]`` / ``--kernel decay_step --rows B`` (the
    recurrence with a step size per head over prompts / over single tokens), ``--kernel attention_latent --seqs N --rows T --ctx C
    --heads H`` (the latent attention; --rows 1: single tokens behind C cached ones), ``--kernel weight_stream --shape S [--stages R] [--ksplit Z]`` (the
    matrix read once through the few-row products' TMA rings and nothing else: the floor under
    them), ``--kernel causal_conv|gated_scan|norm_add_gated|bias_gelu --seqs N --rows T --width W`` (what stands in front
    of and behind an out-norm block's sublayers, the minGRU's recurrence, the dense feed-forward's bias and GELU).
    Weights rotate over enough copies to exceed L2.  Prints one JSON line."""
    import torch
    from builderforce_inference_b200.kernels import fast_ops
    dev = torch.device("cuda:0")
    reps = a.steps
    if a.kernel == "weight_stream":
        # the floor under the few-row products: the matrix read once through their TMA rings, nothing else
        n, k, _ = KERNEL_SHAPES[a.shape]
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]

        stages = a.stages
        # K split as the few-row product plans it: enough blocks for two per SM, at least 8 k blocks each
        tiles, kblocks, n_sm = (n + 127) // 128, (k + 63) // 64, fast_ops.sm_count(dev)
        ksplit = a.ksplit or (max(1, min(8, 2 * n_sm // tiles, kblocks // 8)) if tiles * 2 <= 2 * n_sm else 1)

        def one(i):
            if not fast_ops.weight_stream(ws[i % copies], stages=stages, ksplit=ksplit):
                raise SystemExit("weight_stream does not take this matrix")
        bytes_moved, flops = n * k * 2, 0.0
        what = {"shape": a.shape, "N": n, "K": k, "stages": stages, "ksplit": ksplit}
    elif a.kernel in ("skinny_gemm", "gemm_tcgen05"):
        n, k, epi = KERNEL_SHAPES[a.shape]
        m = a.rows
        copies = max(2, int(400e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(m, n // 2 if epi == 2 else n, device=dev, dtype=torch.float32 if epi == 1 else torch.bfloat16)
        fn = fast_ops.skinny_gemm if a.kernel == "skinny_gemm" else fast_ops.gemm_tcgen05

        def one(i):
            if not fn(x, ws[i % copies], out, epi):
                raise SystemExit(f"{a.kernel} does not take M={m} N={n} K={k}")
        bytes_moved, flops = n * k * 2, 2.0 * m * n * k
        what = {"shape": a.shape, "M": m, "N": n, "K": k, "epilogue": epi}
    elif a.kernel in ("lightning_chunks", "lightning_scan"):
        # the decayed linear attention: --seqs prompts of --rows tokens (chunks), or --rows sequences of one token (scan)
        from builderforce_inference_b200.kernels import ops
        c = CONFIG_4B
        h, d = c["num_attention_heads"], c["head_dim"]
        chunks = a.kernel == "lightning_chunks"
        n_seq, t_new = (a.seqs, a.rows) if chunks else (a.rows, 1)
        cols = 4 * h * d
        copies = 1 if chunks else max(2, int(400e6 // (n_seq * h * d * d * 4)) + 1)
        proj = torch.randn(n_seq * t_new, cols, device=dev, dtype=torch.bfloat16)
        o = torch.empty(n_seq * t_new, h * d, device=dev, dtype=torch.float32)
        states = [torch.zeros(n_seq, h, d, d, device=dev, dtype=torch.float32) for _ in range(copies)]
        decay = torch.linspace(0.96, 0.996, h, device=dev, dtype=torch.float32)
        cu = torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seq, dtype=torch.int32, device=dev)

        def one(i):
            if chunks:
                if not fast_ops.lightning_chunks_bf16(proj, 0, h * d, 2 * h * d, o, states[0], decay, cu, slots, n_seq, h, d, d):
                    raise SystemExit("lightning_chunks does not take this shape")
            else:
                ops.lightning_scan(proj, 0, h * d, 2 * h * d, o, states[i % copies], decay, cu, slots, n_seq, h, d, d,
                                   ops.LIGHT_ACT_SILU, True, True)
        bytes_moved = n_seq * h * d * d * 4 * 2 + n_seq * t_new * (3 * h * d * 2 + h * d * 4)
        # per token and head: scores and their use within a chunk (causal half of 64 x 64), q S and the state update
        flops = n_seq * t_new * h * (2.0 * d * d * 2 + (2.0 * 32 * (d + d) if chunks else 0.0))
        what = {"seqs": n_seq, "new_tokens": t_new, "heads": h, "dim": d, "vdim": d}
    elif a.kernel in ("causal_conv", "gated_scan", "norm_add_gated", "bias_gelu"):
        # the kernels around an out-norm block's sublayers and of the minGRU: --seqs prompts of --rows tokens, --width channels
        from builderforce_inference_b200.kernels import ops
        n_seq, t_new, w = a.seqs, a.rows, a.width
        n = n_seq * t_new
        copies = max(2, int(600e6 // (n * w * 12)) + 1)
        cu = torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seq, dtype=torch.int32, device=dev)
        slot_of = slots.repeat_interleave(t_new)
        bf, single = torch.bfloat16, t_new == 1
        if a.kernel == "causal_conv":       # x + conv(x) off the float32 stream, with the plain copy: what stands in front of a sublayer
            taps = KIKELORN_TAPS
            xs = [torch.randn(n, w, device=dev) for _ in range(copies)]
            cw = torch.randn(w, taps, device=dev, dtype=bf) * 0.3
            state = torch.zeros(n_seq, taps - 1, w, device=dev)
            h, plain = torch.empty(n, w, device=dev, dtype=bf), torch.empty(n, w, device=dev, dtype=bf)

            def one(i):
                ops.causal_conv(xs[i % copies], 0, w, cw, None, state, h, slot_of, cu, slots, n_seq, single_tokens=single,
                                act=ops.CONV_ACT_NONE, add_input=True, copy=plain)
            bytes_moved = n * w * (4 + 2 + 2)
        elif a.kernel == "gated_scan":      # the minGRU's recurrence over [z | u | g] with its output gate
            projs = [torch.randn(n, 3 * w, device=dev, dtype=bf) for _ in range(copies)]
            bz, bu = torch.randn(w, device=dev), torch.randn(w, device=dev)
            state = torch.zeros(n_seq, w, device=dev)
            y = torch.empty(n, w, device=dev, dtype=bf)

            def one(i):
                ops.gated_scan(projs[i % copies], 0, w, 2 * w, w, bz, bu, y, state, cu, slots, n_seq, t_new)
            bytes_moved = n * w * 2 * 4
        elif a.kernel == "norm_add_gated":  # x += mult * norm(y * sigmoid(g + b)): what stands behind a sublayer
            ys = [torch.randn(n, w, device=dev) for _ in range(copies)]
            x = torch.zeros(n, w, device=dev)
            gl = torch.randn(n, w, device=dev, dtype=bf)
            gb, nw = torch.randn(w, device=dev, dtype=bf), torch.ones(w, device=dev, dtype=bf)

            def one(i):
                ops.norm_add(x, ys[i % copies], nw, 1e-6, mult=0.7, gate=gl, gate_bias=gb)
            bytes_moved = n * w * (4 + 2 + 4 + 4)
        else:                               # gelu_tanh(u + b) in place, and the next product's bias into its float32 target rows
            ff = 3 * w
            us_ = [torch.randn(n, ff, device=dev, dtype=bf) for _ in range(copies)]
            b1, b2 = torch.randn(ff, device=dev, dtype=bf), torch.randn(w, device=dev, dtype=bf)
            fill = torch.empty(n, w, device=dev)

            def one(i):
                ops.bias_act(us_[i % copies], b1, us_[i % copies], fill=fill, fill_bias=b2)
            bytes_moved = n * (ff * 4 + w * 4)
        flops = 0.0
        what = {"seqs": n_seq, "new_tokens": t_new, "width": w}
    elif a.kernel in ("decay_scan", "decay_step"):
        # the recurrence with a step size per head (state-space form): --seqs prompts of --rows tokens (chunked from 192
        # tokens on), or --rows sequences of one token
        from builderforce_inference_b200.kernels import ops
        c = CONFIG_4B
        h, g, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        prompt = a.kernel == "decay_scan"
        n_seq, t_new = (a.seqs, a.rows) if prompt else (a.rows, 1)
        n = n_seq * t_new
        copies = 1 if prompt else max(2, int(400e6 // (n_seq * h * d * d * 4)) + 1)
        bc = torch.randn(n, 2 * g * d, device=dev, dtype=torch.bfloat16)
        x = torch.randn(n, h * d, device=dev, dtype=torch.bfloat16)
        raw = torch.randn(n, h, device=dev, dtype=torch.bfloat16)
        o = torch.empty(n, h * d, device=dev, dtype=torch.float32)
        states = [torch.zeros(n_seq, h, d, d, device=dev, dtype=torch.float32) for _ in range(copies)]
        bias, rate, skip = (torch.rand(h, device=dev) + 0.5 for _ in range(3))
        cu = torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev)
        slots = torch.arange(n_seq, dtype=torch.int32, device=dev)
        chunked = {}
        if prompt and t_new >= 192:
            n_chunks = n // 64 + n_seq
            chunked = {"chunk_len": 64, "max_chunks": (t_new + 63) // 64,
                       "chunk_state": torch.empty(n_chunks, h * d * d, device=dev), "chunk_decay": torch.empty(n_chunks, h * d, device=dev)}

        def one(i):
            ops.decay_scan(bc, g * d, 0, x, 0, raw, 0, o, states[i % copies], cu, slots, n_seq, h, d, d, h // g, ops.DECAY_STEP, bias,
                           rate=rate, skip=skip, few_tokens=not prompt, single_tokens=not prompt, **chunked)
        bytes_moved = n_seq * h * d * d * 4 * 2 + n * ((2 * g * d + h * d + h) * 2 + h * d * 4)
        # per token and state element: the update (multiply, multiply-add) and the output's multiply-add; chunked, the
        # earlier tokens' part of the output once more
        flops = n * h * d * d * (7.0 if chunked else 5.0)
        what = {"seqs": n_seq, "new_tokens": t_new, "heads": h, "groups": g, "dim": d, "vdim": d, "chunked": bool(chunked)}
    elif a.kernel == "qk_prepare":
        # bias, row norm, adjacent-pair rotation over half a head, keys as values, cache write of one prompt of --rows tokens
        from builderforce_inference_b200.cache import KVView
        from builderforce_inference_b200.kernels import ops
        from builderforce_inference_b200.parts.rotary import rotary_table
        c = CONFIG_4B
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        t = a.rows
        blocks = (t + 63) // 64
        table = torch.arange(blocks, dtype=torch.int32, device=dev).reshape(1, blocks)
        copies = 4
        kvs = [KVView(torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16),
                      torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16), table, nkv, d, None)
               for _ in range(copies)]
        qks = [torch.randn(t, (nq + nkv) * d, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
        bq, bk = (torch.zeros(n * d, device=dev, dtype=torch.bfloat16) for n in (nq, nkv))
        wq, wk = (torch.ones(n * d, device=dev, dtype=torch.bfloat16) for n in (nq, nkv))
        res = torch.zeros(t, c["hidden_size"], device=dev)
        bo = torch.zeros(c["hidden_size"], device=dev, dtype=torch.bfloat16)
        rope = rotary_table(c["rope_theta"], d // 2, t, dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        slot = torch.zeros(t, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        def one(i):
            ops.qk_prepare(qks[i % copies], nq, nkv, d, pos, slot, kvs[i % copies], ops.FLAG_WRITE_CACHE | ops.FLAG_VALUES_ARE_KEYS,
                           q_bias=bq, k_bias=bk, q_norm_w=wq, k_norm_w=wk, norm_mode=ops.NORM_ROW, eps=1e-6, rope_table=rope,
                           rot_dim=d // 2, pairing=ops.PAIR_ADJACENT, residual=res, out_bias=bo, status=status)
        bytes_moved = t * ((2 * nq + 3 * nkv) * d * 2 + 2 * c["hidden_size"] * 4)
        flops = 0.0
        what = {"tokens": t, "q_heads": nq, "kv_heads": nkv, "head_dim": d}
    elif a.kernel == "qk_norm_rope":
        # q/k norm + rotation + cache write of one prompt of --rows tokens
        from builderforce_inference_b200.cache import KVView
        from builderforce_inference_b200.kernels import ops
        from builderforce_inference_b200.parts.rotary import rotary_table
        c = CONFIG_4B
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        t = a.rows
        blocks = (t + 63) // 64
        table = torch.arange(blocks, dtype=torch.int32, device=dev).reshape(1, blocks)
        copies = 4
        kvs = [KVView(torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16),
                      torch.zeros(blocks, nkv, 64, d, device=dev, dtype=torch.bfloat16), table, nkv, d, None)
               for _ in range(copies)]
        qkvs = [torch.randn(t, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
        norm_w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        rope = rotary_table(c["rope_theta"], d, t, dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        slot = torch.zeros(t, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)

        def one(i):
            ops.qk_norm_rope_cache(qkvs[i % copies], nq, nkv, d, norm_w, norm_w, c["rms_norm_eps"], rope, d, pos, slot,
                                   kvs[i % copies], ops.FLAG_WRITE_CACHE, status)
        bytes_moved = t * (2 * nq + 3 * nkv) * d * 2          # q read and written, k and v read and written to the cache
        flops = 0.0
        what = {"tokens": t, "q_heads": nq, "kv_heads": nkv, "head_dim": d}
    elif a.kernel == "attention_latent":
        # the latent attention over a cache of one row per token (512 + 64 values, the first 512 the value): --seqs
        # sequences that bring --rows tokens each behind --ctx cached ones in all (--rows 1: single tokens)
        from builderforce_inference_b200.cache import KVView
        from builderforce_inference_b200.engine.context import Workspace
        from types import SimpleNamespace
        heads, rank, d = a.heads, MUNERAX_LATENT, MUNERAX_LATENT + 64
        n_seq, t_new = a.seqs, a.rows
        ctx_len = max(a.ctx, t_new)
        blocks = (ctx_len + 63) // 64
        n_pages = n_seq * blocks
        table = torch.randperm(n_pages).to(torch.int32).reshape(n_seq, blocks).to(dev)
        copies = max(2, int(400e6 // (n_pages * 64 * d * 2)) + 1) if t_new == 1 else 1
        kvs = []
        for _ in range(copies):
            k = (torch.randn(n_pages, 1, 64, d, device=dev) * 0.5).to(torch.bfloat16)
            kvs.append(KVView(k, k, table, 1, d, None, v_dim=rank, values_in_keys=True))
        q = (torch.randn(n_seq * t_new, heads * d, device=dev) * 0.1).to(torch.bfloat16)
        out = torch.empty(n_seq * t_new, heads * rank, device=dev, dtype=torch.bfloat16)
        ctx = SimpleNamespace(n_seqs=n_seq, max_seq_tokens=t_new, workspace=Workspace(dev), pages_bucket=0,
                              cu_seqlens=torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev),
                              seq_slot=torch.arange(n_seq, dtype=torch.int32, device=dev),
                              seq_start=torch.full((n_seq,), ctx_len - t_new, dtype=torch.int32, device=dev))
        sinks = torch.zeros(heads, device=dev)

        def one(i):
            if not fast_ops.attention_latent_bf16(ctx, q, out, kvs[i % copies], heads, d ** -0.5, sinks):
                raise SystemExit("attention_latent does not take this shape")
        pairs = n_seq * heads * sum(ctx_len - t_new + i + 1 for i in range(t_new))
        bytes_moved = n_seq * ctx_len * d * 2 + n_seq * t_new * heads * (d + rank) * 2
        flops = 2.0 * pairs * (d + rank)                # scores over the whole row, the weighted sum over the latent
        what = {"seqs": n_seq, "new_tokens": t_new, "context": ctx_len, "heads": heads, "row": d, "latent": rank}
    else:
        from builderforce_inference_b200.cache import KVView
        c = CONFIG_4B
        nq, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        decode = a.kernel == "attention_decode"
        n_seq = a.rows if decode else a.seqs
        t_new = 1 if decode else a.rows
        ctx_len = a.ctx if decode else t_new
        blocks = (ctx_len + 63) // 64
        n_pages = n_seq * blocks
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).reshape(n_seq, blocks)
        cache_bytes = n_pages * nkv * 64 * d * 2 * 2
        copies = max(2, int(400e6 // cache_bytes) + 1) if decode else 1
        kvs = [KVView(torch.randn(n_pages, nkv, 64, d, device=dev, dtype=torch.bfloat16),
                      torch.randn(n_pages, nkv, 64, d, device=dev, dtype=torch.bfloat16), table, nkv, d, None)
               for _ in range(copies)]
        q = torch.randn(n_seq * t_new, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
        out = torch.empty(n_seq * t_new, nq * d, device=dev, dtype=torch.bfloat16)

        class Ctx:
            pass
        ctx = Ctx()
        from builderforce_inference_b200.engine.context import Workspace
        ctx.workspace = Workspace(dev)
        ctx.n_seqs, ctx.n_tokens, ctx.max_seq_tokens = n_seq, n_seq * t_new, t_new
        ctx.seq_slot = torch.arange(n_seq, dtype=torch.int32, device=dev)
        ctx.seq_start = torch.full((n_seq,), ctx_len - t_new, dtype=torch.int32, device=dev)
        ctx.cu_seqlens = torch.arange(0, (n_seq + 1) * t_new, t_new, dtype=torch.int32, device=dev)
        ctx.total_pages = torch.tensor([n_seq * blocks], dtype=torch.int32, device=dev)
        fn = {"attention_decode": fast_ops.attention_decode_bf16, "attention_prefill": fast_ops.attention_prefill_bf16,
              "attention_prefill_tcgen05": fast_ops.attention_prefill_tcgen05_bf16}[a.kernel]
        def one(i):
            if not fn(ctx, q, out, kvs[i % copies], nq, d ** -0.5):
                raise SystemExit(f"{a.kernel} does not take this shape")
        bytes_moved = n_seq * ctx_len * 2 * nkv * d * 2
        flops = 4.0 * nq * d * n_seq * (ctx_len if decode else t_new * (t_new + 1) / 2)
        what = {"seqs": n_seq, "new_tokens": t_new, "context": ctx_len, "q_heads": nq, "kv_heads": nkv, "head_dim": d}
    for i in range(3):
        one(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.eager:                             # plain launches (for captures under ncu)
        e0.record()
        for i in range(reps):
            one(i)
        e1.record()
    else:
        graph = torch.cuda.CUDAGraph()      # one graph of all launches: no host gaps between short kernels
        with torch.cuda.graph(graph):
            for i in range(reps):
                one(i)
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / reps
    pk = peaks()
    print(json.dumps({"kernel": a.kernel, **what, "us": round(us, 2), "launches": reps,
                      "GB_s": round(bytes_moved / us / 1e3, 1), "TFLOP_s": round(flops / us / 1e6, 1),
                      "frac_hbm": round(bytes_moved / us / 1e3 / pk["hbm_gbs"], 3),
                      "frac_bf16": round(flops / us / 1e6 / pk["bf16_tflops"], 3), "peaks": pk["source"],
                      "note": ("plain launches: short kernels include launch gaps" if a.eager else
                               "launches replayed from one CUDA graph") + ", operands rotating over more than L2"}))
    return 0


TRACE_UNITS = [("core", "elementwise"), ("core", "sampling"), ("core", "gemm_simt"), ("fast", "gemm_tcgen05"),
               ("fast", "attention_decode"), ("fast", "attention_prefill_tcgen05")]


def timeline_run(a) -> int:
    """``--timeline``: one decode step's kernels on the GPU's own clock.  The libraries are built
    with time stamps in the kernels (BFI_B200_TRACE=1, set below before the package loads): the first
    thread of every block records when it starts, when its wait for the kernel before it returns and
    (products and attention) when it ends.  Prints, for the kernels of ``--timeline-layer``, the
    first and last of each stamp in microseconds from the step's start: where the step's time goes
    between the kernels, which no serialised profile shows."""
    import ctypes

    import numpy as np
    import torch
    from builderforce_inference_b200 import Model
    from builderforce_inference_b200.engine.engine import SequenceStep
    from builderforce_inference_b200.kernels.library import library
    layers = a.layers or 12
    cfg = dict(SHAPES[a.shape_name], num_hidden_layers=layers)
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=a.batch * CONTEXT, max_seq_len=CONTEXT, max_batch=a.batch)
    eng = model.engine
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(128, 2049, (a.batch,), generator=g).tolist()
    slots = [eng.acquire() for _ in lens]
    eng.step([SequenceStep(s, torch.randint(0, 1000, (n,), generator=g).tolist(), ()) for s, n in zip(slots, lens)], check=False)

    def one():
        eng.step([SequenceStep(s, (5,), (0,)) for s in slots], check=False)

    if a.timeline_prompt:
        # a prompt step instead: --timeline-prompt tokens, eager launches
        for s in slots:
            eng.release(s)
        prompt = torch.randint(0, 1000, (a.timeline_prompt,), generator=g).tolist()

        def one():                                                     # noqa: F811
            s = eng.acquire()
            eng.step([SequenceStep(s, prompt, (len(prompt) - 1,))], check=False)
            torch.cuda.synchronize()
            eng.release(s)

    for _ in range(6):
        one()
    torch.cuda.synchronize()
    cap = 1 << 18

    def read_all():
        recs = []
        for libname, unit in TRACE_UNITS:
            fn = getattr(library(libname).lib, f"bfi_trace_read_{unit}")
            fn.restype = ctypes.c_long
            buf = np.zeros(2 * cap, dtype=np.uint64)
            n = fn(buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_long(cap))
            for i in range(n):
                key, t = int(buf[2 * i]), int(buf[2 * i + 1])
                recs.append((key >> 32, (key >> 28) & 0xF, t, unit))
        return recs

    read_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    one()
    e1.record()
    torch.cuda.synchronize()
    recs = read_all()
    grids = {}
    for gid, what, t, unit in recs:
        d = grids.setdefault(gid, {"unit": unit, "t": {0: [], 1: [], 2: []}})
        d["t"][what].append(t)
    order = sorted(grids)
    t00 = min(t for _, _, t, _ in recs)
    per_layer = (len(order) - 3) // layers if layers else 9     # beside the layers: embedding, final norm, head
    first = 1 + a.timeline_layer * per_layer
    what = f"one prompt step of {a.timeline_prompt} tokens" if a.timeline_prompt else f"one decode step, batch {a.batch}"
    print(f"{what}, {layers} layers of the {a.shape_name} shape: {e0.elapsed_time(e1):.3f} ms with the stamps; "
          f"{len(order)} kernels, {per_layer} per layer; layer {a.timeline_layer}:")
    print("| # | source file | blocks | first start | last start | first wait over | last wait over | first end | last end |")
    print("|---|---|---|---|---|---|---|---|---|")

    def us(xs, fn):
        return f"{(fn(xs) - t00) / 1e3:.2f}" if xs else "-"

    for i, gid in enumerate(order):
        if not first <= i < first + per_layer + 1:
            continue
        d = grids[gid]
        print(f"| {i} | {d['unit']} | {len(d['t'][0])} | {us(d['t'][0], min)} | {us(d['t'][0], max)} | {us(d['t'][1], min)} | "
              f"{us(d['t'][1], max)} | {us(d['t'][2], min)} | {us(d['t'][2], max)} |")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--timeline", action="store_true", help="print one decode step's kernels on the GPU's clock (see timeline_run)")
    ap.add_argument("--timeline-layer", type=int, default=6)
    ap.add_argument("--timeline-prompt", type=int, default=0, help="with --timeline: a prompt step of this many tokens instead")
    ap.add_argument("--heads", type=int, default=16, help="--kernel attention_latent: query heads")
    ap.add_argument("--seqs", type=int, default=1, help="kernel mode, prompt attention: prompts of --rows tokens each")
    ap.add_argument("--kernel", default=None, choices=["skinny_gemm", "gemm_tcgen05", "weight_stream", "qk_norm_rope", "attention_decode",
                                                       "attention_prefill", "attention_prefill_tcgen05", "lightning_chunks", "lightning_scan",
                                                       "qk_prepare", "decay_scan", "decay_step", "attention_latent", "causal_conv",
                                                       "gated_scan", "norm_add_gated", "bias_gelu"],
                    help="time one kernel instead of the model (see kernel_run)")
    ap.add_argument("--width", type=int, default=2048, help="kernel mode, the channel-wise kernels: channels of a row")
    ap.add_argument("--shape", default="qkv", choices=sorted(KERNEL_SHAPES))
    ap.add_argument("--eager", action="store_true", help="with --kernel: plain launches instead of one CUDA graph")
    ap.add_argument("--stages", type=int, default=6, help="--kernel weight_stream: 16 KB tiles in a block's ring (1..12)")
    ap.add_argument("--ksplit", type=int, default=0, help="--kernel weight_stream: ranges of K (0: as the product plans it)")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", dest="shape_name", default="4b", choices=sorted(SHAPES),
                    help="layer sizes: the benchmark's Qwen3-4B shape, or the 8B / 32B shapes for runs beside it")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers of the same sizes")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--design", default=None, choices=["datasun", "bepilorn", "munerax", "kikelorn"],
                    help="instead of the benchmark: this design beside qwen3 at equal layer sizes (see design_run)")
    ap.add_argument("--sizes", default=None, help="with --design: names of DESIGN_SIZES, comma-separated (default: all)")
    ap.add_argument("--only", default=None, help="with --design kikelorn: the designs to run, comma-separated (default: all four)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace: no Rust toolchain or network here to build it, "
                          "pip cannot install it, and its CUDA backend runs no kernel for bf16 weights"}))
        return 0
    if a.timeline:
        os.environ["BFI_B200_TRACE"] = "1"
        return timeline_run(a)
    if a.kernel is not None:
        return kernel_run(a)
    if a.design is not None:
        return design_run(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for --gpus {a.gpus})")
        return 2
    warmup = max(3, a.warmup)

    import torch
    from builderforce_inference_b200 import Model
    pk = peaks()
    shape_cfg = SHAPES[a.shape_name]
    full_layers = shape_cfg["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg = dict(shape_cfg, num_hidden_layers=a.layers)
    max_batch = a.batch if a.no_points else max(64, a.batch)
    t_load = time.time()
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max(max_batch * CONTEXT, 16384),
                              max_seq_len=max(CONTEXT, 8192) if a.shape_name == "8b" else CONTEXT, max_batch=max_batch)
    print(f"[bench] model ready in {time.time() - t_load:.1f} s", file=sys.stderr, flush=True)

    if a.shape_name != "4b":
        clocks = ClockSampler()
        clocks.start()
        numbers = side_run(a, model, shape_cfg, pk)
        print(json.dumps({"workloads": f"qwen3-{a.shape_name}-shape, builder-run beside the benchmark", "dtype": "bf16",
                          "layers": a.layers, "layers_full": full_layers, "peaks": pk["source"], **numbers,
                          "clocks": clocks.stop()}))
        return 0

    # untimed: compile, capture graphs, size workspaces
    decode_run(model, a.batch, 2, 3, seed=1)
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(model, a.batch, a.steps, warmup, seed=2)
    e2e = e2e_run(model, a.batch, a.steps, warmup, seed=2)
    points, prefill, decode_points, e2e_b1 = {}, None, {}, None
    if not a.no_points:
        deep_steps = 12                                   # 3 warm-up + 12 timed steps end at 4,095 of 4,096
        deep_start = CONTEXT - (3 + deep_steps) - 1    # 4,080
        for b in sorted({1, a.batch, 64}):
            if b == a.batch:
                after = main_run
            else:
                decode_run(model, b, 2, 3, seed=3)         # untimed: graph capture for this batch size
                after = decode_run(model, b, min(a.steps, 32), warmup, seed=4)
            if b in (1, 64):
                points[f"decode_b{b}"] = round(after["tok_s"], 1)
            decode_points[f"b{b}_after_prompt"] = point(after, pk)
            deep = decode_run(model, b, deep_steps, 3, seed=5, lens=[deep_start] * b)
            decode_points[f"b{b}_ctx{CONTEXT}"] = point(deep, pk)
        e1 = e2e_run(model, 1, min(a.steps, 32), warmup, seed=4)          # the prompt of the batch-1 point above
        e2e_b1 = {"value": round(e1["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e1["h2d"],
                  "d2h_bytes_per_step": e1["d2h"]}
        pf = prefill_run(model, PREFILL_TOKENS, 10, a.layers, shape_cfg, breakdown=True)          # median of 10
        prefill = {"value": round(pf["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pf["ms"], 3),
                   "frac": round(pf["flops"] / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                   "breakdown": pf["breakdown"]}
    clk = clocks.stop()

    achieved = main_run["step_bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    c = shape_cfg
    line = {
        "metric": f"Qwen3-{a.shape_name.upper()} bf16 decode tok/s at batch {a.batch} (batch 1/64 in points; prefill tok/s at 2,048 tokens)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights",
        "config": {"model": f"qwen3-{a.shape_name}-shape", "layers": a.layers, "layers_full": full_layers,
                   "hidden": c["hidden_size"], "q_heads": c["num_attention_heads"],
                   "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
                   "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "tied_head": bool(c["tie_word_embeddings"]),
                   "global_batch": a.batch, "seq_len": CONTEXT, "prompt_len": "uniform[128,2048]",
                   "ctx_mean": round(main_run["ctx_mean"], 1), "parallelism": "single-gpu",
                   "l2": "weights read per step exceed L2", "peaks": pk["source"]},
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "clocks": clk,
    }
    if prefill is not None:
        line["prefill"] = prefill
        line["points"] = points
        line["decode_points"] = decode_points
        line["e2e_b1"] = e2e_b1
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
