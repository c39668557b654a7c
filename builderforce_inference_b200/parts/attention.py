"""Grouped-query attention over the paged cache, as a mixer.

Order of operations (crates/bfi-models/src/qwen3.rs:220-242): q, k, v projections without bias;
per-head RMS norm of q and k when ``qk_norm``; position encoding of q and k; k and v appended to
the sequence's cache; causal attention of every new token over the cached keys (all of them, or
the last ``window``); output projection added to the residual stream.

The three projections are one matrix product over the concatenated weights.  Keys and values
are always read from the cache, so a step may bring whole prompts, a continuation of a cached
prefix, or single tokens, and a run may read another run's cache (``run.writes_cache`` false:
this layer then has no k and v projections of its own).

Variants, each a parameter: ``bias`` (q, k, v and output projections carry one); ``qk_norm``
``"head"`` (RMS norm over each head, one weight of ``head_dim``) or ``"row"`` (RMS norm over the
whole q projection and over the whole k projection, weights of that size); ``values`` ``"keys"``
(no v projection: the values are the keys as projected, with their bias, before norm and
rotation); ``sink`` (a score every query sees beside its keys, with no value: the softmax's
denominator carries ``exp(sink)``; a number, or ``"learned"``: one per query head, a tensor of the
checkpoint); ``v_dim`` (value heads of another size than the keys'); ``chunk`` (a token reads only
the keys of its own block of ``chunk`` consecutive positions, blocks counted from position 0);
``out_bias`` (whether the output projection carries a bias when the others do; default: it does);
``exact_weights`` (the softmax's weights stay float32 up to the second product, also in a bfloat16
run: the tensor-core prompt kernel then multiplies with two bfloat16 terms per weight);
the position encoding's pairing and partial width; ``conv_taps`` (a short causal convolution over
time on every channel of q, k and v, directly after the projection and before norm and rotation,
without bias or activation; the last ``taps - 1`` projected rows are kept per sequence, so the mixer
then asks the cache for a fixed-size state beside its pages); ``v_mix`` (``"source"``: the values of
this layer, as they are cached, are also left in a buffer of the step; ``"mix"``: the values become
``(1 - lambda) v + lambda v_source`` with the source layer's values of the same token and a learned
number ``lambda``, before they are cached; both ride on the convolution's kernel); ``gate``
(``"head"``: head a's output is multiplied by ``sigmoid(W_g h)_a``, the logits coming out of the same
product as q, k and v).  The plain
combination (no bias, head norm or none, own values, rotate-half) runs the per-head kernel that
fuses norm, rotation and cache write; the others run the per-token kernel that also adds the
biases, so no variant costs a launch of its own.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, linear
from .base import MIXERS, POSITION_ENCODINGS, KVNeed, Mixer, ParamSpec, PartSpec, StateNeed


@MIXERS.register("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, qk_norm=False, eps: float = 1e-6,
                 window: Optional[int] = None, scale: Optional[float] = None, own_kv: bool = True,
                 bias: bool = False, values: str = "projection", sink=None, v_dim: Optional[int] = None,
                 chunk: Optional[int] = None, out_bias: Optional[bool] = None, exact_weights: bool = False,
                 conv_taps: Optional[int] = None, v_mix: Optional[str] = None, gate: Optional[str] = None):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"GQA: {n_heads} query heads do not divide into {n_kv_heads} kv heads")
        if head_dim % 2 != 0 or head_dim > 512:
            raise ValueError(f"attention kernels take even head sizes up to 512, got {head_dim}")
        if qk_norm is True:
            qk_norm = "head"
        if qk_norm not in (False, None, "head", "row"):
            raise ValueError(f"qk_norm must be false, 'head' or 'row', got {qk_norm!r}")
        if values not in ("projection", "keys"):
            raise ValueError(f"values must be 'projection' or 'keys', got {values!r}")
        if values == "keys" and not own_kv:
            raise ValueError("a layer without keys of its own has no keys to use as values")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive, got {window}")
        if chunk is not None and chunk < 1:
            raise ValueError(f"chunk must be positive, got {chunk}")
        v_dim = head_dim if v_dim is None else int(v_dim)
        if v_dim < 1 or v_dim > 512:
            raise ValueError(f"attention kernels take value sizes from 1 to 512, got {v_dim}")
        if values == "keys" and v_dim != head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if not (sink is None or sink == "learned" or isinstance(sink, (int, float))):
            raise ValueError(f"sink must be a number or 'learned', got {sink!r}")
        if conv_taps is not None and not 1 <= conv_taps <= 16:
            raise ValueError(f"the convolution on q, k and v takes 1 to 16 taps, got {conv_taps}")
        if v_mix not in (None, "source", "mix"):
            raise ValueError(f"v_mix must be 'source' or 'mix', got {v_mix!r}")
        if v_mix is not None and (conv_taps is None or not own_kv or values == "keys"):
            raise ValueError("value mixing rides on the convolution of a layer's own q, k and v")
        if gate not in (None, "head"):
            raise ValueError(f"gate must be 'head', got {gate!r}")
        if conv_taps is not None and not own_kv:
            raise ValueError("a layer that borrows its keys has no convolution on q, k and v")
        self.taps, self.v_mix, self.gate = (None if conv_taps is None else int(conv_taps)), v_mix, gate
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.qk_norm, self.eps, self.window = (qk_norm or None), float(eps), window
        self.bias, self.values_are_keys = bool(bias), values == "keys"
        self.v_dim, self.chunk, self.exact_weights = v_dim, chunk, bool(exact_weights)
        self.out_bias = self.bias if out_bias is None else bool(out_bias)
        if self.out_bias and not self.bias:
            raise ValueError("an output bias without the projections' biases is not a known variant")
        self.learned_sink = sink == "learned"
        self.sink = None if sink is None or self.learned_sink else float(sink)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.own_kv = bool(own_kv)
        self.position = POSITION_ENCODINGS.build(position) if position is not None \
            else POSITION_ENCODINGS.build(PartSpec("none"))
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self.b_q = self.b_k = self.b_v = self.b_o = None

    def children(self):
        return {"position": self.position}

    def param_specs(self) -> Dict[str, ParamSpec]:
        d, h = self.head_dim, self.width
        specs = {"q_proj": ParamSpec((self.n_heads * d, h)), "o_proj": ParamSpec((h, self.n_heads * self.v_dim))}
        if self.own_kv:
            specs["k_proj"] = ParamSpec((self.n_kv_heads * d, h))
            if not self.values_are_keys:
                specs["v_proj"] = ParamSpec((self.n_kv_heads * self.v_dim, h))
        if self.learned_sink:
            specs["sink"] = ParamSpec((self.n_heads,), "matrix")
        if self.taps is not None:
            for name in ("q_proj", "k_proj", "v_proj"):
                if name in specs:
                    specs[name + ".conv"] = ParamSpec((specs[name].shape[0], self.taps))
        if self.v_mix is not None:
            specs["v_mix"] = ParamSpec((), "matrix")       # the source layer's is stored too, and unused
        if self.gate:
            specs["g_proj"] = ParamSpec((self.n_heads, h))
        if self.qk_norm:
            row = self.qk_norm == "row"
            specs["q_norm"] = ParamSpec((self.n_heads * d if row else d,), "norm")
            if self.own_kv:
                specs["k_norm"] = ParamSpec((self.n_kv_heads * d if row else d,), "norm")
        if self.bias:
            for name in ("q_proj", "k_proj", "v_proj") + (("o_proj",) if self.out_bias else ()):
                if name in specs:
                    specs[name + ".bias"] = ParamSpec((specs[name].shape[0],), "matrix")
        return specs

    def _plain(self) -> bool:
        """The combination the per-head kernel (norm, rotate-half, cache write) covers."""
        return not self.bias and not self.values_are_keys and self.qk_norm != "row" \
            and getattr(self.position, "pairing", "half") == "half" and self.v_dim == self.head_dim

    def cache_need(self):
        kv = KVNeed(self.n_kv_heads, self.head_dim, self.window,
                    v_dim=None if self.v_dim == self.head_dim else self.v_dim, chunk=self.chunk)
        if self.taps is None or self.taps == 1:
            return kv
        return (kv, StateNeed((self.taps - 1, self._n_qkv()), "float32"))

    def _n_qkv(self) -> int:
        """Columns of q, k and v together in the projection."""
        n_kv_in = self.n_kv_heads if self.own_kv else 0
        return (self.n_heads + n_kv_in) * self.head_dim + (0 if self.values_are_keys else n_kv_in * self.v_dim)

    def prepare(self, runtime, max_positions: int) -> None:
        self.position.prepare(runtime, max_positions)

    def load(self, tensors, runtime) -> None:
        mats = [tensors["q_proj"]]
        if self.own_kv:
            mats += [tensors["k_proj"]] + ([] if self.values_are_keys else [tensors["v_proj"]])
        if self.taps is not None:
            convs = [tensors[n + ".conv"] for n in ("q_proj", "k_proj", "v_proj") if n + ".conv" in tensors]
            if len({c.dtype for c in convs}) > 1:
                convs = [c.float() for c in convs]
            self.conv_w = torch.cat(convs, dim=0).contiguous()
            self.no_history = torch.empty((1, 0, self.conv_w.shape[0]), dtype=torch.float32, device=runtime.device)
        if self.v_mix == "mix":
            self.mix_lambda = tensors["v_mix"].float().reshape(1).contiguous()
        if self.gate:
            mats.append(tensors["g_proj"])      # the gate's logits come out of the same product, behind q, k and v
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = tensors["o_proj"]
        self.sinks = tensors["sink"].float().contiguous() if self.learned_sink else None
        self.q_norm = tensors.get("q_norm")
        self.k_norm = tensors.get("k_norm")
        if self.q_norm is not None and self.k_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        if self.bias:
            self.b_q, self.b_k, self.b_v = (tensors.get(n + ".bias") for n in ("q_proj", "k_proj", "v_proj"))
            self.b_o = tensors["o_proj.bias"] if self.out_bias else None
            if len({b.dtype for b in (self.b_q, self.b_k, self.b_v) if b is not None}) > 1:
                self.b_q, self.b_k, self.b_v = (None if b is None else b.float() for b in (self.b_q, self.b_k, self.b_v))

    def forward(self, ctx, h, residual, run) -> None:
        self._run(ctx, h, residual, run, EPI_ACCUMULATE)

    def forward_store(self, ctx, h, out, run) -> None:
        if self.b_o is not None:       # the output bias is added to the target's row before the product
            out.zero_()
            self._run(ctx, h, out, run, EPI_ACCUMULATE)
        else:
            self._run(ctx, h, out, run, EPI_STORE)

    def _run(self, ctx, h, residual, run, epilogue) -> None:
        kv = run.kv
        if kv is None:
            raise RuntimeError("attention needs a key/value cache for its run")
        n_kv_in = self.n_kv_heads if self.own_kv else 0
        if run.writes_cache != self.own_kv:
            raise RuntimeError("an attention layer writes the cache exactly when it has k and v projections")
        d = self.head_dim
        n_qkv = self._n_qkv()
        proj = ctx.rows("attn.qkv", self.w_qkv.shape[0])
        linear(h, self.w_qkv, proj, EPI_STORE)
        qkv = proj if proj.shape[1] == n_qkv else proj[:, :n_qkv]
        if self.taps is not None:
            kept = run.state if self.taps > 1 else self.no_history
            if kept is None:
                raise RuntimeError("the convolution on q, k and v needs its per-sequence state")
            conv = ctx.rows("attn.conv", n_qkv)
            n_v = n_kv_in * self.v_dim
            shared = ctx.rows("attn.v_source", n_v) if self.v_mix else None
            ops.causal_conv(proj, 0, n_qkv, self.conv_w, None, kept, conv, ctx.token_slot, ctx.cu_seqlens, ctx.seq_slot,
                            ctx.n_seqs, single_tokens=ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs,
                            act=ops.CONV_ACT_NONE, mix_off=n_qkv - n_v,
                            mix_src=shared if self.v_mix == "mix" else None,
                            mix_dst=shared if self.v_mix == "source" else None,
                            mix_lambda=self.mix_lambda if self.v_mix == "mix" else None)
            qkv = conv

        fused = self.position.fused_rotary()
        write = ops.FLAG_WRITE_CACHE if run.writes_cache else 0
        if not self._plain():
            if fused is None:
                raise RuntimeError("this attention variant needs a position encoding the kernels apply themselves")
            table, rot = fused
            ops.qk_prepare(qkv, self.n_heads, n_kv_in, d, ctx.token_pos, ctx.token_slot, kv,
                           write | (ops.FLAG_VALUES_ARE_KEYS if self.values_are_keys else 0),
                           q_bias=self.b_q, k_bias=self.b_k, v_bias=self.b_v, q_norm_w=self.q_norm, k_norm_w=self.k_norm,
                           norm_mode={None: ops.NORM_NONE, "head": ops.NORM_HEAD, "row": ops.NORM_ROW}[self.qk_norm],
                           eps=self.eps, rope_table=table, rot_dim=rot,
                           pairing=ops.PAIR_ADJACENT if getattr(self.position, "pairing", "half") == "adjacent" else ops.PAIR_HALF,
                           residual=residual, out_bias=self.b_o, status=ctx.status, v_dim=self.v_dim)
        elif fused is not None:
            table, rot = fused
            ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, self.q_norm, self.k_norm, self.eps,
                                   table, rot, ctx.token_pos, ctx.token_slot, kv, write, ctx.status)
        else:
            # a position encoding with code of its own: norms first, then its transform, then the cache
            ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, self.q_norm, self.k_norm, self.eps,
                                   None, 0, ctx.token_pos, ctx.token_slot, kv, ops.FLAG_K_IN_PLACE, ctx.status)
            q_view = qkv[:, :self.n_heads * d].view(-1, self.n_heads, d)
            k_view = qkv[:, self.n_heads * d:(self.n_heads + n_kv_in) * d].view(-1, n_kv_in, d)
            self.position.apply(ctx, q_view, k_view)
            if write:
                ops.qk_norm_rope_cache(qkv, self.n_heads, n_kv_in, d, None, None, self.eps, None, 0,
                                       ctx.token_pos, ctx.token_slot, kv, write, ctx.status)

        out = ctx.rows("attn.out", self.n_heads * self.v_dim)
        self.attend(ctx, qkv, out, kv)
        if self.gate:
            ops.sigmoid_gate(out, proj[:, n_qkv:n_qkv + self.n_heads], self.v_dim)
        linear(out, self.w_o, residual, epilogue)

    def attend(self, ctx, qkv, out, kv) -> None:
        from ..kernels import attention as fast_attention
        sink = self.sinks if self.learned_sink else self.sink
        if fast_attention.attend(ctx, qkv, out, kv, self.n_heads, self.scale, sink, self.exact_weights):
            return
        ops.attention_paged(qkv, qkv.stride(0), out, kv, ctx.cu_seqlens, ctx.seq_slot, ctx.seq_start,
                            ctx.n_seqs, ctx.max_seq_tokens, self.n_heads, self.scale, sink)
