"""Munerax without a GPU: the configuration reader and its refusals by key, the model as data, the
cache's bookkeeping for latent rows and for state outside the layers, and the plain implementation
(tests/plain/munerax_plain.py) against closed forms, among them the identity the package's latent
attention rests on."""
import copy
import math

import pytest
import torch

from munerax_models import MX_ODD, MX_WIDE, make_weights, random_config, tensor_shapes
from plain import munerax_plain as P

from builderforce_inference_b200.cache.cache import SequenceCache
from builderforce_inference_b200.cache.plan import kv_bytes_per_token, plan_cache, state_bytes_per_slot
from builderforce_inference_b200.config.base import ConfigError
from builderforce_inference_b200.config.munerax import MuneraxConfig, MuneraxDense, MuneraxMoE
from builderforce_inference_b200.engine.decoder import expected_tensors
from builderforce_inference_b200.parts.base import BLOCKS, INPUT_PARTS, KVNeed, StateNeed
from builderforce_inference_b200.registry import architecture_for, describe_model

F = torch.float64


# ------------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size_and_constant():
    c = MuneraxConfig.from_dict(MX_ODD)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, len(c.layers)) == (131, 40, 2e-5, 3.7, 5)
    assert (c.bigram.buckets, c.bigram.mul_prev, c.bigram.mul_cur) == (53, 7, 13)
    m = c.layers[0].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale, m.rot_base, m.rot_dims, m.kv_from) == \
        (3, 10, 6, 12, 14, 0.21, 100.0, 6, None)
    assert c.layers[1].mixer.kv_from == 0 and c.layers[3].mixer.kv_from == 2 and c.layers[2].mixer.rot_dims == 4
    assert isinstance(c.layers[0].mlp, MuneraxDense) and c.layers[0].mlp.ff == 24 and c.layers[2].mlp is None
    f = c.layers[1].mlp
    assert isinstance(f, MuneraxMoE) and (f.experts, f.top, f.ff, f.groups, f.keep, f.scale, f.shared_ff) == (6, 3, 20, 3, 2, 1.5, 12)
    f = c.layers[3].mlp
    assert (f.groups, f.keep, f.shared_ff, f.scale) == (1, 1, None, 0.8)
    assert architecture_for(MX_ODD).name == "munerax"
    bare = copy.deepcopy(MX_ODD)
    del bare["embedding"]
    c = MuneraxConfig.from_dict(bare)
    assert c.bigram is None and c.embedding_scale == 1.0 and describe_model(bare).input_parts == ()


def _changed(path, value):
    cfg = copy.deepcopy(MX_ODD)
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
    (("layers", 0, "type"), "attention", "type"),
    (("layers", 0, "mixer", "kv_rank"), KeyError, "kv_rank"),
    (("layers", 0, "mixer", "kv_rank"), 15, "kv_rank"),                 # 15 + 6 values in a cache row: odd
    (("layers", 0, "mixer", "rot", "dims"), 8, "dims"),                 # more turned values than the rotated part has
    (("layers", 0, "mixer", "rot", "dims"), 3, "dims"),
    (("layers", 1, "mixer", "kv_from"), 1, "kv_from"),                  # itself
    (("layers", 1, "mixer", "kv_from"), 4, "kv_from"),                  # a later layer
    (("layers", 4, "mixer", "kv_from"), 1, "keeps none"),               # a layer that borrows itself
    (("layers", 1, "mixer", "kv_rank"), 16, "must equal"),              # not its source's
    (("layers", 1, "mixer", "rot", "base"), 50.0, "must equal"),
    (("layers", 1, "mlp", "kind"), "switch", "kind"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),   # 6 experts in 4 groups
    (("layers", 1, "mlp", "router", "groups", "keep"), 1, "groups"),    # 1 group of 2 cannot give 3
    (("layers", 0, "mlp", "ff"), 0, "ff"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("embedding", "bigram", "mul_prev"), -1, "mul_prev"),
])
def test_config_refuses_by_key(path, value, names):
    with pytest.raises(ConfigError) as e:
        MuneraxConfig.from_dict(_changed(path, value))
    assert names in str(e.value)


def test_model_as_data_names_every_tensor_with_its_shape():
    for cfg in (MX_ODD, MX_WIDE) + tuple(random_config(s) for s in range(101, 125)):
        spec = describe_model(cfg)
        want = {n: tuple(s) for n, (s, _) in tensor_shapes(cfg).items()}
        assert {n: tuple(p.shape) for n, p in expected_tensors(spec).items()} == want
        assert spec.head_name is None and spec.embedding_scale == (cfg.get("embedding") or {}).get("scale", 1.0)
        assert [r.layer for r in spec.schedule] == list(range(len(cfg["layers"])))
        assert [r.cache_of for r in spec.schedule] == [l["mixer"].get("kv_from") for l in cfg["layers"]]


def test_cache_needs_rows_of_the_latent_and_the_previous_token():
    spec = describe_model(MX_ODD)
    blocks = [BLOCKS.build(l.block) for l in spec.layers]
    needs = [b.mixer().cache_need() for b in blocks]
    assert needs[0] == KVNeed(1, 20, v_dim=14, values_in_keys=True) and needs[2] == KVNeed(1, 32, v_dim=24, values_in_keys=True)
    assert needs[1] == needs[4] == needs[0] and needs[3] == needs[2]
    cache_of = [r.cache_of for r in spec.schedule]
    # only the two layers with a down projection keep rows, and a row serves as key and value
    assert kv_bytes_per_token(needs, cache_of, 2) == (20 + 32) * 2
    part = INPUT_PARTS.build(spec.input_parts[0][0])
    assert part.cache_need() == StateNeed((1,), "int32")
    assert state_bytes_per_slot(needs + [part.cache_need()], cache_of + [None]) == 4
    plan = plan_cache(needs + [part.cache_need()], cache_of + [None], 1 << 20, 2, n_slots=8)
    assert plan.bytes_per_token == 104 and plan.state_bytes == 32
    assert blocks[2].ffn is None and blocks[2].norm2 is None and "norm2.weight" not in spec.layers[2].names


def test_cache_serves_borrowers_and_state_outside_the_layers():
    spec = describe_model(MX_ODD)
    needs = [BLOCKS.build(l.block).mixer().cache_need() for l in spec.layers]
    cache_of = [r.cache_of for r in spec.schedule]
    cache = SequenceCache(needs, cache_of, 512, 256, torch.float32, torch.device("cpu"), initial_slots=2,
                          model_needs=[StateNeed((1,), "int32")])
    a, b = cache.acquire(), cache.acquire()
    own, borrowed = cache.run_cache(0), cache.run_cache(4)
    assert own.writes_cache and not borrowed.writes_cache and own.kv.k.data_ptr() == borrowed.kv.k.data_ptr()
    assert own.kv.values_in_keys and own.kv.v.data_ptr() == own.kv.k.data_ptr() and own.kv.k.shape[1:] == (1, 64, 20)
    assert not own.kv.plain and own.kv.value_dim == 14
    assert cache.run_cache(3).kv.k.data_ptr() == cache.run_cache(2).kv.k.data_ptr() != own.kv.k.data_ptr()
    state = cache.model_cache(0).state
    assert state.shape == (2, 1) and state.dtype == torch.int32
    state[a, 0], state[b, 0] = 17, 23
    cache.release(a)
    again = cache.acquire()                      # the slot comes back with its state cleared, the other's stays
    assert again == a and int(cache.model_cache(0).state[a, 0]) == 0 and int(cache.model_cache(0).state[b, 0]) == 23
    c = cache.acquire()                          # the slot table grows: the state moves with it
    assert cache.model_cache(0).state.shape[0] >= 3 and int(cache.model_cache(0).state[b, 0]) == 23
    for s in (again, b, c):
        cache.release(s)
    cache.check()


# ------------------------------------------------------------------------------------------------ the plain implementation
def test_plain_bigram_rows():
    assert P.bigram_rows([5, 0, 9, 9], 53, 7, 13) == [53, (5 * 7 + 0) % 53, (0 + 9 * 13) % 53, (9 * 7 + 9 * 13) % 53]
    assert P.bigram_rows([4], 1, 3, 5) == [1] and P.bigram_rows([4, 4, 2], 1, 3, 5) == [1, 0, 0]
    w = {"embed": torch.arange(12, dtype=F).reshape(4, 3), "bigram": 100.0 * torch.arange(9, dtype=F).reshape(3, 3)}
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": 2, "mul_prev": 1, "mul_cur": 1}}}
    x = P.embed(w, cfg, [3, 1, 2])
    assert torch.equal(x[0], w["embed"][3] * 2 + w["bigram"][2]) and torch.equal(x[1], w["embed"][1] * 2 + w["bigram"][0])
    assert torch.equal(x[2], w["embed"][2] * 2 + w["bigram"][1])


def test_plain_activations():
    z = torch.tensor([-3.0, -0.5, 0.0, 0.7, 4.0], dtype=F)
    want = [0.5 * v * (1 + math.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3))) for v in z.tolist()]
    assert torch.allclose(P.gelu_tanh(z), torch.tensor(want, dtype=F), atol=1e-15)
    assert P.relu_squared(z).tolist() == [0.0, 0.0, 0.0, 0.7 ** 2, 16.0]


def test_plain_sink_softmax_counts_the_sink_once_and_unscaled():
    s = torch.tensor([[0.3, 9.0, 9.0], [1.0, -2.0, 9.0], [0.5, 0.25, -1.0]], dtype=F)
    p = P.sink_softmax(s, torch.tensor(0.7, dtype=F))
    assert p[0, 1] == 0 and p[0, 2] == 0 and p[1, 2] == 0
    assert abs(float(p[0, 0]) - math.exp(0.3) / (math.exp(0.3) + math.exp(0.7))) < 1e-15
    den = math.exp(0.5) + math.exp(0.25) + math.exp(-1.0) + math.exp(0.7)
    assert torch.allclose(p[2], torch.tensor([math.exp(0.5), math.exp(0.25), math.exp(-1.0)], dtype=F) / den, atol=1e-15)
    far = P.sink_softmax(s, torch.tensor(50.0, dtype=F))        # a huge sink takes nearly all the weight
    assert float(far.sum()) < 1e-15 * 3 + 1e-10


def test_plain_router_scores_groups_and_weights():
    # 6 experts in 3 groups of 2, keep 2, top 3: group sums of sigmoid scores decide, then the scores
    z = torch.tensor([[2.0, 1.9, 3.0, -5.0, 0.1, 0.0]], dtype=F)
    s = torch.sigmoid(z[0])
    sums = [float(s[0] + s[1]), float(s[2] + s[3]), float(s[4] + s[5])]
    assert sums[0] > sums[2] > sums[1]                     # the group with the single best expert loses
    pick, weight = P.route(z, 3, 3, 2, 1.5)
    assert pick.tolist() == [[0, 1, 4]] and torch.allclose(weight[0], s[[0, 1, 4]] * 1.5)
    pick, weight = P.route(z, 2, 1, 1, 1.0)                # no groups: the best scores
    assert pick.tolist() == [[2, 0]]
    pick, _ = P.route(z, 2, 6, 3, 1.0)                     # groups of one expert: a group's score is its expert's
    assert pick.tolist() == [[2, 0]]
    margins = []
    P.route(z, 3, 3, 2, 1.5, margins)
    assert abs(margins[0] - min(sums[2] - sums[1], float(s[4] - s[5]))) < 1e-15


def _one_layer(seed=0, T=9):
    m = {"heads": 3, "dim": 10, "rot_dim": 6, "vdim": 7, "kv_rank": 12, "scale": 0.3, "rot": {"base": 100.0, "dims": 6}}
    g = torch.Generator().manual_seed(seed)
    w = {"q": torch.randn(3 * 16, 20, generator=g, dtype=F), "dkv": torch.randn(18, 20, generator=g, dtype=F),
         "dkv.norm": 1 + 0.1 * torch.randn(12, generator=g, dtype=F), "uk": torch.randn(30, 12, generator=g, dtype=F),
         "uv": torch.randn(21, 12, generator=g, dtype=F), "sink": torch.randn(3, generator=g, dtype=F),
         "g": torch.randn(3, 20, generator=g, dtype=F), "o": torch.randn(20, 21, generator=g, dtype=F)}
    return m, w, torch.randn(T, 20, generator=g, dtype=F)


def test_plain_latent_attention_equals_attention_in_the_latent_space():
    """The identity the package computes by: scores from the absorbed queries against [c | rotated
    part], weighted sums of the latents, then W_uv; token by token, from nothing but cached rows."""
    m, w, h = _one_layer()
    c, kr = P.latent_of(w, "", m, h, 1e-5)
    ref = P.latent_attention(w, "", m, h, 1e-5, (c, kr))
    T, H, d, rd, dv, r = h.shape[0], 3, 10, 6, 7, 12
    q = (h @ w["q"].T).reshape(T, H, d + rd)
    qr = P.rotate_half(q[..., d:], range(T), 100.0, 6)
    uk, uv = w["uk"].reshape(H, d, r), w["uv"].reshape(H, dv, r)
    rows = torch.cat([c, kr], dim=1)                        # what a cache holds
    out = torch.zeros(T, H * dv, dtype=F)
    for t in range(T):
        for a in range(H):
            qa = torch.cat([uk[a].T @ q[t, a, :d], qr[t, a]])
            s = rows[:t + 1] @ qa * 0.3
            top = max(float(s.max()), float(w["sink"][a]))
            e = torch.exp(s - top)
            p = e / (e.sum() + math.exp(float(w["sink"][a]) - top))
            out[t, a * dv:(a + 1) * dv] = uv[a] @ (p @ rows[:t + 1, :r]) * torch.sigmoid(h[t] @ w["g"][a])
    assert torch.allclose(out @ w["o"].T, ref, atol=1e-10)


def test_plain_latent_rows_are_normed_and_turned_by_position():
    m, w, h = _one_layer(1)
    c, kr = P.latent_of(w, "", m, h, 1e-5)
    d = h @ w["dkv"].T
    assert torch.allclose(c[4], d[4, :12] / torch.sqrt((d[4, :12] ** 2).mean() + 1e-5) * w["dkv.norm"], atol=1e-14)
    assert torch.allclose(kr[0], d[0, 12:], atol=1e-15)                       # position 0 turns nothing
    f1 = 100.0 ** (-2.0 / 6)
    u, v = d[5, 12 + 1], d[5, 12 + 4]                                         # pair (1, 1 + 3) of six
    assert abs(float(kr[5, 1]) - float(u * math.cos(5 * f1) - v * math.sin(5 * f1))) < 1e-12
    assert abs(float(kr[5, 4]) - float(v * math.cos(5 * f1) + u * math.sin(5 * f1))) < 1e-12
    m2 = dict(m, rot={"base": 100.0, "dims": 2})                             # only the first pair turns: (0, 1)
    _, kr2 = P.latent_of(w, "", m2, h, 1e-5)
    assert torch.allclose(kr2[:, 2:], d[:, 14:], atol=1e-15) and not torch.allclose(kr2[3, :2], d[3, 12:14])


def test_plain_model_is_causal_and_borrowers_read_their_source():
    w = {k: v.to(F) for k, v in make_weights(MX_ODD, 4, torch.float32).items()}
    ids = [7, 100, 3, 3, 58, 12, 99, 0, 130, 41]
    full = P.forward_each(w, MX_ODD, ids)
    assert full.shape == (10, 131) and torch.allclose(P.forward_each(w, MX_ODD, ids[:6]), full[:6], atol=1e-9)
    layers = P.forward_layers(w, MX_ODD, ids)
    assert layers.shape == (5, 10, 40)
    # the down projection of a borrowing layer does not exist; its source's decides
    w2 = dict(w)
    w2["l0.mix.dkv"] = w["l0.mix.dkv"] * 1.5
    l2 = P.forward_layers(w2, MX_ODD, ids)
    assert not torch.allclose(l2[1] - l2[0], layers[1] - layers[0])
    # the previous token matters through the bigram table only
    other = P.forward_each(w, MX_ODD, [8] + ids[1:])
    assert not torch.allclose(other[1], full[1])


def test_key_ranges_of_the_latent_attention_fill_whole_waves():
    from builderforce_inference_b200.kernels.fast_ops import LATENT_TILES_PER_RANGE, latent_splits
    n_sm = 148
    for n_seqs in (1, 2, 7, 8, 31, 32, 64, 100, 147, 148, 400):
        for rows in (1, 16, 32, 64, 65, 600):
            for pages in (1, 3, 16, 64, 512):
                s = latent_splits(n_seqs, rows, pages, n_sm)
                blocks = n_seqs * ((rows + 63) // 64)
                longest = max(1, min(2 * pages // LATENT_TILES_PER_RANGE, 64))
                assert 1 <= s <= longest
                if blocks >= n_sm:
                    assert s == 1
                    continue
                # no other count within the bounds does the walk in fewer wave-lengths, the merge's share counted
                def cost(k):
                    return -(-blocks * k // n_sm) / k * (1.0 if k == 1 else 1.0 + 0.02 * k)
                assert all(cost(s) <= cost(k) + 1e-9 for k in range(1, longest + 1)), (n_seqs, rows, pages, s)
    # 64 sequences on 148 SMs: two ranges are one wave of half walks; three would be two waves of thirds
    assert latent_splits(64, 16, 64, n_sm) == 2
    # a single sequence is cut as far as its length allows
    assert latent_splits(1, 16, 512, n_sm) == 64 and latent_splits(1, 16, 8, n_sm) == 16 // LATENT_TILES_PER_RANGE
    assert latent_splits(1, 16, 1, n_sm) == 1
