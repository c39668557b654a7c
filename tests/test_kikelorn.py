"""Kikelorn without a GPU: the configuration reader and its refusals by key, the model as data, what
its blocks ask of the cache, the reordering that lets rotation of adjacent pairs run as rotation of
halves, and the plain implementation (tests/plain/kikelorn_plain.py) against closed forms."""
import copy
import math

import pytest
import torch

from kikelorn_models import KK_ODD, KK_WIDE, make_weights, random_config, tensor_shapes
from plain import kikelorn_plain as P

from builderforce_inference_b200.config.base import ConfigError
from builderforce_inference_b200.config.kikelorn import KikelornAttention, KikelornConfig, KikelornLatent, KikelornMinGRU
from builderforce_inference_b200.engine.decoder import expected_tensors
from builderforce_inference_b200.parts.base import BLOCKS, KVNeed, StateNeed
from builderforce_inference_b200.parts.rotary import rotary_table
from builderforce_inference_b200.registry import architecture_for, describe_model

F = torch.float64


# ------------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size_and_constant():
    c = KikelornConfig.from_dict(KK_ODD)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, c.residual_mult, c.canon_taps, len(c.layers)) == (137, 40, 2e-5, 3.3, 0.6, 2, 7)
    g = c.layers[0].mixer
    assert isinstance(g, KikelornMinGRU) and g.width == 56 and c.layers[0].mlp.ff == 24
    a = c.layers[3].mixer
    assert isinstance(a, KikelornAttention)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.scale, a.chunk, a.v_mix) == (4, 2, 8, 12, 2, 0.35, 50, True)
    assert (a.rot.base, a.rot.dims, a.rot.scaling) == (1e4, 8, None) and c.layers[1].mixer.v_mix is False
    m = c.layers[2].mixer
    assert isinstance(m, KikelornLatent) and c.layers[2].mlp is None
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale) == (3, 10, 6, 12, 14, 10, 0.23)
    assert m.rot.dims == 4 and m.rot.scaling_dict() == {"factor": 3.0, "original": 64.0, "fast": 16.0, "slow": 2.0}
    assert c.layers[6].mixer.rot is None
    assert architecture_for(KK_ODD).name == "kikelorn"
    bare = copy.deepcopy(KK_ODD)
    del bare["embedding"], bare["residual_mult"]
    c = KikelornConfig.from_dict(bare)
    assert c.embedding_scale == 1.0 and c.residual_mult == 1.0


def _changed(path, value):
    cfg = copy.deepcopy(KK_ODD)
    node = cfg
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,names", [
    (("vocab",), KeyError, "vocab"),
    (("norm",), KeyError, "norm"),
    (("canon",), KeyError, "canon"),
    (("canon", "taps"), 0, "taps"),
    (("canon", "taps"), 17, "taps"),
    (("layers",), [], "layers"),
    (("layers", 0, "type"), "lstm", "type"),
    (("layers", 0, "mixer", "width"), 0, "width"),
    (("layers", 1, "mixer", "kv_heads"), 2, "kv_heads"),
    (("layers", 1, "mixer", "dim"), 9, "dim"),
    (("layers", 1, "mixer", "mask"), KeyError, "mask"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"),
    (("layers", 1, "mixer", "conv"), KeyError, "conv"),
    (("layers", 1, "mixer", "rot", "dims"), 12, "dims"),
    (("layers", 1, "mixer", "rot", "dims"), 3, "dims"),
    (("layers", 2, "mixer", "q_rank"), KeyError, "q_rank"),
    (("layers", 2, "mixer", "kv_rank"), 600, "kv_rank"),
    (("layers", 2, "mixer", "rot", "scaling", "slow"), KeyError, "slow"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), 0.0, "factor"),
    (("layers", 5, "mixer", "vdim"), 10, "vdim"),              # a mixing layer whose values have another size than the first one's
    (("layers", 1, "mlp", "kind"), "moe", "kind"),
    (("layers", 1, "mlp", "ff"), 0, "ff"),
])
def test_config_refuses_by_key(path, value, names):
    with pytest.raises(ConfigError) as e:
        KikelornConfig.from_dict(_changed(path, value))
    assert names in str(e.value)


# ------------------------------------------------------------------------------------------------ the model as data
@pytest.mark.parametrize("cfg", [KK_ODD, KK_WIDE] + [random_config(s) for s in range(300, 320)])
def test_spec_names_every_tensor_with_its_shape(cfg):
    spec = describe_model(cfg)
    want = expected_tensors(spec)
    have = tensor_shapes(cfg)
    assert set(want) == set(have)
    for name, (shape, _) in have.items():
        assert tuple(want[name].shape) == tuple(shape), name
    assert spec.head_name is None and spec.embedding_scale == cfg["embedding"]["scale"]


def test_the_first_mixing_layer_is_the_source_and_blocks_ask_for_their_state():
    spec = describe_model(KK_ODD)
    blocks = [BLOCKS.build(layer.block) for layer in spec.layers]
    assert [b.mixer().v_mix for b in blocks if hasattr(b.mixer(), "v_mix")] == [None, "source", "mix", "mix"]
    needs = [b.cache_need() for b in blocks]
    w, taps = KK_ODD["width"], KK_ODD["canon"]["taps"]
    own = StateNeed((taps - 1, w), "float32")
    assert needs[0] == (StateNeed((56,), "float32"), own, own)                       # minGRU, then the block's two convolutions
    n_qkv = 3 * 10 + 3 * 10 + 3 * 6
    assert needs[1] == (KVNeed(3, 10, None, v_dim=6, chunk=24), StateNeed((2, n_qkv), "float32"), own, own)
    assert needs[2] == (KVNeed(1, 20, v_dim=14, values_in_keys=True), own)          # no feed-forward: one convolution
    assert needs[6][0] == KVNeed(2, 16, None, v_dim=12, chunk=50) and len(needs[6]) == 3
    # one tap keeps nothing
    one = copy.deepcopy(KK_ODD)
    one["canon"]["taps"] = 1
    one["layers"][1]["mixer"]["conv"] = 1
    b = BLOCKS.build(describe_model(one).layers[1].block)
    assert b.cache_need() == (KVNeed(3, 10, None, v_dim=6, chunk=24),)


def test_reordered_rows_turn_adjacent_pairs_as_halves():
    """Scores over the rotated part are the same when queries and keys are reordered alike: rotating
    adjacent pairs, then reordering (even values first, then odd), equals reordering, then rotating
    halves."""
    from builderforce_inference_b200.parts.latent import LatentAttention
    from builderforce_inference_b200.parts.base import PartSpec
    part = LatentAttention(width=8, n_heads=2, dim=3, rot_dim=6, v_dim=4, kv_rank=6, q_rank=5,
                           position=PartSpec("rotary", {"theta": 100.0, "rot_dim": 4, "pairing": "adjacent"}))
    m = torch.arange(2 * 9 * 5, dtype=torch.float32).reshape(18, 5)
    got = part._reordered(m, 3, 9, 2)
    order = [0, 1, 2, 3, 5, 4, 6, 7, 8]                        # of a head's rows: 3 unrotated, then rows 3..6 as (3, 5, 4, 6), then 2 that do not turn
    assert torch.equal(got, m[[i + 9 * h for h in range(2) for i in order]])
    T, dims = 5, 4
    cos, sin = P.rotary_angles(range(T), dims, 100.0)
    v = torch.randn(T, 1, 6, dtype=F)
    turned = P.rotate(v, cos, sin, dims, "interleaved")
    perm = [0, 2, 1, 3, 4, 5]
    assert torch.allclose(turned[..., perm], P.rotate(v[..., perm], cos, sin, dims, "half"))


@pytest.mark.parametrize("base,dims,scaling", [(3.0e5, 12, (8.0, 256, 16.0, 1.0)), (1e4, 8, None), (100.0, 6, (3.0, 64, 16.0, 2.0)),
                                               (5e3, 2, (2.0, 32, 8.0, 1.0))])
def test_rotation_table_is_the_plain_one(base, dims, scaling):
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    table = rotary_table(base, dims, 700, "cpu", sc)
    cos, sin = P.rotary_angles(range(700), dims, base, sc)
    assert torch.allclose(table[..., 0].double(), cos, atol=1e-6) and torch.allclose(table[..., 1].double(), sin, atol=1e-6)
    if scaling:     # the premise: the scaling changes the low frequencies and the magnitude
        plain_cos, _ = P.rotary_angles(range(700), dims, base)
        assert float((plain_cos - cos).abs().max()) > 1e-2


# ------------------------------------------------------------------------------------------------ the plain implementation
def test_plain_convolution_and_mingru_against_closed_forms():
    u = torch.randn(9, 3, dtype=F)
    w = torch.randn(3, 4, dtype=F)
    y = P.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[5], sum(w[:, j] * u[2 + j] for j in range(4)))
    # a gate that is always 1/2 averages the candidates with weights 2^-(age + 1)
    width, n = 4, 5
    ww = {"z": torch.zeros(n, width, dtype=F), "z.b": torch.zeros(n, dtype=F), "x": torch.randn(n, width, dtype=F),
          "x.b": torch.randn(n, dtype=F), "g": torch.randn(n, width, dtype=F), "o": torch.eye(width, n, dtype=F)}
    h = torch.randn(7, width, dtype=F)
    cand = P.mingru_candidate(h @ ww["x"].T + ww["x.b"])
    S = sum(cand[t] * 0.5 ** (6 - t + 1) for t in range(7))
    assert torch.allclose(P.mingru(ww, "", h)[6], (S * P.silu(h[6] @ ww["g"].T)) @ ww["o"].T)
    assert float(P.mingru_candidate(torch.tensor([0.0], dtype=F))) == 0.5 and abs(float(P.mingru_candidate(torch.tensor([-1e-9], dtype=F))) - 0.5) < 1e-8


def test_plain_chunk_mask_and_value_mixing():
    m = P.chunk_mask(10, 4)
    assert m[3, 0] and not m[4, 3] and m[4, 4] and not m[9, 7] and m[9, 8] and not m[2, 3]
    cfg = copy.deepcopy(KK_ODD)
    w = {k: v.to(F) for k, v in make_weights(cfg, 2, torch.float32).items()}
    ids = list(range(3, 60))
    base = P.forward(cfg, w, ids)
    w2 = dict(w)
    w2["l3.mix.vmix"] = w["l3.mix.vmix"] + 0.5           # the source layer's own factor is not used
    assert torch.equal(P.forward(cfg, w2, ids), base)
    w2["l5.mix.vmix"] = w["l5.mix.vmix"] + 0.5
    assert float((P.forward(cfg, w2, ids) - base).abs().max()) > 1e-6
