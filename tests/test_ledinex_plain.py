"""The plain Ledinex implementation against closed forms, and what needs no GPU of the engine's side:
the configuration reader, the tensor lists, the cache layout of layers with several needs."""
import copy
import json
import math

import numpy as np
import pytest

import plain_ledinex as P
from ledinex_helpers import CONFIGS, LX_A, LX_B, LX_C, RANK, file_config, random_config, random_weights, tensor_shapes

RNG = np.random.default_rng(5)


def r(*shape, std=1.0):
    return RNG.standard_normal(shape) * std


# ----------------------------------------------------------------------------- the oracle's mechanisms

def test_input_convolution_by_hand_and_norm_around_zero():
    x, w = r(5, 3), r(3, 3)
    y = P.input_convolution(x, w)
    assert np.allclose(y[0], x[0] + w[:, 2] * x[0])
    assert np.allclose(y[1], x[1] + w[:, 2] * x[1] + w[:, 1] * x[0])
    assert np.allclose(y[4], x[4] + w[:, 2] * x[4] + w[:, 1] * x[3] + w[:, 0] * x[2])
    one = P.input_convolution(x, r(3, 1) * 0.0)
    assert np.allclose(one, x)                                       # one tap of weight zero: the stream itself
    assert np.allclose(P.norm_one_plus(x, np.zeros(3), 1e-5), P.rms_norm(x, None, 1e-5))
    assert np.allclose(P.norm_one_plus(x, np.full(3, 0.5), 0.0), 1.5 * x / np.sqrt((x * x).mean(1, keepdims=True)))


def test_rotation_layout_scalings_and_distance_only_scores():
    x = r(6, 2, 10)
    pos = np.arange(6) + 3
    f = P.plain_frequencies(6, 100.0)
    y = P.rotate_half(x, pos, 6, f)
    a = 4 * f[1]                                                     # token 1 stands at position 4
    assert np.allclose(y[1, 0, 1], x[1, 0, 1] * math.cos(a) - x[1, 0, 4] * math.sin(a))
    assert np.allclose(y[1, 0, 4], x[1, 0, 4] * math.cos(a) + x[1, 0, 1] * math.sin(a))
    assert np.allclose(y[..., 6:], x[..., 6:])                       # channels from dims on pass
    assert np.allclose(P.rotate_half(y, pos, 6, f, sign=-1.0), x)    # turned back
    lf, mag = P.frequencies_of({"base": 100.0, "dims": 6, "scaling": {"factor": 4.0}})
    assert np.allclose(lf, f / 4.0) and mag == 1.0
    sf, mag = P.frequencies_of({"base": 100.0, "dims": 6, "scaling": {"factor": 1.0, "original": 32, "fast": 4.0, "slow": 1.0}})
    assert np.allclose(sf, f) and mag == 1.0
    sc = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
    sf, mag = P.frequencies_of({"base": 10000.0, "dims": 32, "scaling": sc})
    f32 = P.plain_frequencies(32, 10000.0)
    assert np.isclose(mag, 0.1 * math.log(8.0) + 1.0)
    assert np.isclose(sf[0], f32[0]) and np.isclose(sf[-1], f32[-1] / 8.0)
    ratio = f32 / sf
    assert np.all(np.diff(ratio) >= -1e-12) and 1.0 < ratio[len(ratio) // 3] <= 8.0 + 1e-9
    q, k = r(1, 1, 6), r(1, 1, 6)
    dots = [float(np.sum(P.rotate_half(q, [p + 5], 6, f) * P.rotate_half(k, [p], 6, f))) for p in (0, 9, 40)]
    assert np.allclose(dots, dots[0])


def test_mask_cap_and_grouping():
    m = P.visible(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True] and m[1].tolist() == [True, True] + [False] * 4
    assert P.visible(4, 0)[3].all() and P.visible(4, 1)[3].tolist() == [False, False, False, True]
    q, k, v = r(5, 4, 3), r(5, 2, 3), r(5, 2, 2)
    o = P.softmax_attention(q, k, v, 0.7)
    s = q[4, 3] @ k[:, 1].T * 0.7                                     # head 3 reads key head 1
    p = np.exp(s - s.max())
    assert np.allclose(o[4, 3], (p / p.sum()) @ v[:, 1])
    capped = P.softmax_attention(100 * q, k, v, 0.7, softcap=1e-3)   # every score within +-0.001: an average
    assert np.allclose(capped[4, 0], v[:, 0].mean(0), atol=2e-3)
    assert np.allclose(P.softmax_attention(q, k, v, 0.7, softcap=1e6), o, atol=1e-6)


def _attn_weights(H, heads, kv, d, dv, own):
    W = {"q": r(heads * d, H), "k": r(kv * d, H), "q.norm": 1 + 0.1 * r(heads * d), "k.norm": 1 + 0.1 * r(kv * d),
         "o": r(H, heads * dv)}
    if own:
        W["v"] = r(kv * dv, H)
    else:
        W.update({"q.b": r(heads * d), "k.b": r(kv * d)})
    return W


def test_capped_attention_rotated_values_come_back():
    H, c = 7, {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "softcap": 5.0,
               "rot": {"base": 50.0, "dims": 4, "scaling": {"factor": 2.0}}}
    W = _attn_weights(H, 2, 1, 4, 6, True)
    h = r(5, H)
    out = P.capped_attention(h, W, c, 1e-5)
    # the first token attends to itself alone: its value turned by 0 and back
    v0 = h[0] @ W["v"].T
    assert np.allclose(out[0], np.concatenate([v0, v0]) @ W["o"].T)
    # what one value contributes arrives turned by the DISTANCE: moving the whole sequence changes nothing
    # (checked through a second run with a token prepended whose key no query can prefer)
    one = P.capped_attention(h[:1], W, c, 1e-5)
    assert np.allclose(one[0], out[0])


def test_window_attention_values_are_raw_keys():
    H, c = 6, {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.4, "mask": {"size": 2},
               "rot": {"base": 50.0, "dims": 2, "scaling": {"factor": 4.0, "original": 8, "fast": 2.0, "slow": 1.0}}}
    W = _attn_weights(H, 2, 2, 4, 4, False)
    h = r(4, H)
    out = P.window_attention(h, W, c, 1e-5)
    k0 = h[0] @ W["k"].T + W["k.b"]
    assert np.allclose(out[0], k0 @ W["o"].T)                         # alone: the key as projected, with its bias
    wider = P.window_attention(h, W, dict(c, mask={"size": 3}), 1e-5)
    assert np.allclose(wider[:2], out[:2]) and not np.allclose(wider[2:], out[2:])


def test_recurrent_branches_by_hand():
    H = 5
    h = r(4, H)
    # lightning: decay 0 keeps nothing, decay 1 keeps all
    c = {"heads": 2, "dim": 3, "vdim": 2, "decay": [0.0, 1.0]}
    W = {"q": r(6, H), "k": r(6, H), "v": r(4, H), "g": r(4, H), "norm": 1 + 0.1 * r(4), "o": r(H, 4)}
    q, k, v = (P.silu(h @ W[n].T) for n in "qkv")
    o = np.zeros((4, 4))
    for t in range(4):
        o[t, :2] = (q[t, :3] @ k[t, :3]) * v[t, :2]
        o[t, 2:] = sum((q[t, 3:] @ k[j, 3:]) * v[j, 2:] for j in range(t + 1))
    want = (P.rms_norm(o, W["norm"], 1e-5) * P.sigmoid(h @ W["g"].T)) @ W["o"].T
    assert np.allclose(P.lightning(h, W, c, 1e-5), want)
    # generalized delta: the first token writes k v^T; a second token with the same key and full removal and
    # no decay takes the first one's value out again before it writes its own
    c = {"heads": 1, "dim": 3}
    W = {n: r(3, H) for n in ("r", "k", "v", "a", "g")}
    W.update({"a.b": np.full(3, 40.0), "w1": r(2, H), "w2": np.zeros((3, 2)), "w0": np.full(3, -40.0), "norm": np.ones(3),
              "o": np.eye(H, 3)})
    h2 = np.stack([h[0], h[0]])
    out = P.generalized_delta(h2, W, c, 0.0)
    rr, kk, vv = (h[0] @ W[n].T for n in "rkv")
    u = kk / np.sqrt(kk @ kk + 1e-6)
    S1 = np.outer(kk, vv)
    S2 = S1 - np.outer(u, u @ S1) + np.outer(kk, vv)                 # w = 1 (sigmoid(-40) = 0), a = 1
    g = P.sigmoid(h[0] @ W["g"].T)
    for S, row in ((S1, out[0]), (S2, out[1])):
        o = S.T @ rr
        assert np.allclose(row[:3], o / np.sqrt(np.mean(o * o)) * g)
    assert np.allclose(S2, S1, atol=1e-4)                             # what was removed is what is written again
    # gated delta: the first token by hand
    c = {"heads": 2, "kv_heads": 1, "dim": 3, "vdim": 2, "conv": 2}
    W = {"q": r(3, H), "k": r(3, H), "v": r(4, H), "q.conv": r(3, 2), "k.conv": r(3, 2), "v.conv": r(4, 2), "b": r(2, H),
         "a": r(2, H), "A_log": r(2), "dt_bias": r(2), "g": r(4, H), "norm": 1 + 0.1 * r(2), "o": r(H, 4)}
    out = P.gated_delta(h, W, c, 1e-5)
    q0 = P.silu((h[0] @ W["q"].T) * W["q.conv"][:, 1])
    k0 = P.silu((h[0] @ W["k"].T) * W["k.conv"][:, 1])
    v0 = P.silu((h[0] @ W["v"].T) * W["v.conv"][:, 1]).reshape(2, 2)
    q0 = q0 / np.sqrt(q0 @ q0 + 1e-6) * 3 ** -0.5
    k0 = k0 / np.sqrt(k0 @ k0 + 1e-6)
    beta = P.sigmoid(h[0] @ W["b"].T)
    o = np.stack([(q0 @ k0) * beta[i] * v0[i] for i in range(2)])     # S starts at zero: the decay has nothing to act on
    want = (P.rms_norm(o, W["norm"], 1e-5).reshape(4) * P.silu(h[0] @ W["g"].T)) @ W["o"].T
    assert np.allclose(out[0], want)


def test_router_and_mixture():
    H, E = 6, 5
    h, Wr = r(7, H), r(E, H)
    ids, w, s = P.route(h, Wr, 2)
    assert np.allclose(w.sum(1), 1.0) and np.allclose(s.sum(1), 1.0)
    assert all(set(ids[t]) == set(np.argsort(-s[t])[:2]) for t in range(7))
    ids_all, w_all, _ = P.route(h, Wr, E)
    assert np.allclose(np.sort(w_all, 1), np.sort(s, 1))              # all chosen: the scores themselves
    tie_ids, _, _ = P.route(np.zeros((1, H)), Wr, 2)
    assert tie_ids[0].tolist() == [0, 1]                              # ties go to the lower index
    W = {"router": Wr, "shared.up": r(4, H), "shared.down": r(H, 4)}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = r(3, H), r(H, 3)
    c = {"router": {"experts": E, "top": E}, "shared": {"ff": 4}}
    want = sum(s[:, e:e + 1] * (np.maximum(h @ W[f"e{e}.up"].T, 0) ** 2) @ W[f"e{e}.down"].T for e in range(E))
    want = want + (np.maximum(h @ W["shared.up"].T, 0) ** 2) @ W["shared.down"].T
    assert np.allclose(P.mixture(h, W, c), want)


@pytest.mark.parametrize("which", list(CONFIGS))
def test_the_model_runs_and_prefixes_agree(which):
    cfg = CONFIGS[which]
    w = {k: v.astype(np.float64) for k, v in random_weights(cfg, 1).items()}
    toks = np.random.default_rng(3).integers(0, cfg["vocab"], size=12).tolist()
    layers = []
    full = P.forward(cfg, w, toks, layers)
    assert full.shape == (12, cfg["vocab"]) and len(layers) == len(cfg["layers"]) and np.isfinite(full).all()
    assert np.allclose(P.forward(cfg, w, toks[:7]), full[:7])         # causal throughout


# ----------------------------------------------------------------------------- the engine's side, without a GPU

class _RT:
    precise = True
    device = "cpu"
    stream_max_rows = 16

    def __init__(self):
        import torch
        self.dtype = torch.float32

    def buffer(self, *a, **k):
        raise AssertionError("no scratch at build time")


def _model(cfg):
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.registry import get_architecture
    from mlxforge_b200.models.decoder import DecoderModel
    c = config_from_json(json.loads(json.dumps(file_config(cfg)))).with_tensor_shapes(dict(tensor_shapes(cfg)))
    return c, DecoderModel(get_architecture("Ledinex").build_spec(c), _RT())


def test_config_reader_defaults_errors_and_round_trip():
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.model_config import ConfigError
    from mlxforge_b200.config.registry import registered_architectures
    assert "Ledinex" in registered_architectures()
    c = config_from_json(json.loads(json.dumps(LX_B)))
    assert (c.taps, c.embedding_scale, c.logit_scale) == (0, 1.0, 1.0)
    left = c.layers[0]["mixer"]["left"]
    assert left["rot"] is None and left["window"] == 0 and left["softcap"] == 0.0
    assert c.layers[4]["mixer"]["left"]["rot"]["scaling"] == {"factor": 1.0}
    a = config_from_json(json.loads(json.dumps(LX_A)))
    assert a.layers[0]["mixer"]["left"]["rot"]["scaling"] == {"factor": 4.0, "original": 16.0, "fast": 6.0, "slow": 1.5}
    assert a.layers[1]["mlp"] is None and a.layers[2]["mixer"]["right"]["decay"] == [0.9, 0.5]
    again = config_from_json(json.loads(json.dumps(a.to_json())))
    assert again.layers == a.layers and (again.vocab, again.width, again.taps, again.logit_scale) == (101, 40, 3, 1.5)

    def broken(edit, text):
        j = copy.deepcopy(LX_A)
        edit(j)
        with pytest.raises(ConfigError, match=text):
            config_from_json(j)
    broken(lambda j: j.pop("width"), "missing required field 'width'")
    broken(lambda j: j["layers"][0].update(type="parallel_3"), "is not supported")
    broken(lambda j: j["layers"][2]["mixer"]["right"].update(decay=[0.5]), "one per head")
    broken(lambda j: j["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple of")
    broken(lambda j: j["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "must be even")
    broken(lambda j: j["layers"][0]["mixer"]["left"].update(vdim=8), "keys' size")
    broken(lambda j: j["layers"][0]["mlp"]["router"].update(top=9), "cannot give a token")
    broken(lambda j: j["layers"][0]["mlp"].update(kind="dense"), "is not supported")
    broken(lambda j: j["canon"].update(taps=0), "must be positive")


@pytest.mark.parametrize("cfg", [LX_A, LX_B, LX_C])
def test_tensor_lists_agree_with_the_description(cfg):
    from mlxforge_b200.config.registry import get_architecture
    c, model = _model(cfg)
    specs = {k: tuple(v.shape) for k, v in model.tensor_specs().items()}
    assert specs == {n: tuple(s) for n, s in tensor_shapes(cfg)}
    listed = {n: tuple(s) for n, s, _ in get_architecture("Ledinex").random_tensors(c)}
    assert listed == specs
    assert model.graph_safe


def test_the_low_rank_comes_from_the_tensor_shapes():
    c, _ = _model(LX_A)
    assert [l["mixer"]["right"].get(RANK) for l in c.layers if l["type"] == "parallel_2"] == [5, 3]


def test_cache_layout_of_layers_with_several_needs():
    import torch
    from mlxforge_b200.cache.manager import CacheManager
    from mlxforge_b200.parts.base import FixedState, PagedKV
    _, model = _model(LX_A)
    layout = model.cache_layout
    assert {(g.need, g.n_lanes) for g in layout.paged} == {(PagedKV(2, 12, 11), 1), (PagedKV(3, 8, 0, v_head_dim=12), 1),
                                                           (PagedKV(1, 20, 37), 1)}
    tags = sorted((g.need.tag, g.need.shape[0], g.n_lanes) for g in layout.state)
    # layer 1 has no feed-forward: one convolution's rows; the others two (taps - 1 = 2 rows of 40 each)
    assert ("conv_read", 80, 1) in tags and ("conv_read", 160, 4) in tags
    assert ("generalized_delta", 3 * 10 * 10, 1) in tags and ("generalized_delta", 14 * 14, 1) in tags
    assert ("retention", 2 * 10 * 6, 1) in tags
    assert ("channel_delta", 4 * 6 * 10 + 2 * (2 * 2 * 6 + 4 * 10), 1) in tags
    first = layout.item_lane[0]
    assert [w[0] for w in first] == ["paged", "state", "state"] and [w[0] for w in layout.item_lane[1]] == ["state", "state"]
    cache = CacheManager(layout, page_size=16, max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu")
    lanes = cache.lane(0)
    assert isinstance(lanes, tuple) and len(lanes) == 3 and lanes[0].need == PagedKV(2, 12, 11)
    assert isinstance(lanes[2].need, FixedState) and lanes[2].tensor.shape == (2, 160)
    seq = cache.open_sequence()
    cache.reserve([(seq, 50)])
    cache.commit(seq, 50)
    assert [len([b for b in blocks if b >= 0]) for blocks in seq.blocks] == [2, 4, 4]     # windows 11, none, 37
    cache.close(seq)
    cache.check()


def test_configurations_drawn_at_random_are_read():
    for seed in range(30):
        cfg = random_config(seed, seed % 2 == 0)
        _, model = _model(cfg)
        assert {k: tuple(v.shape) for k, v in model.tensor_specs().items()} == {n: tuple(s) for n, s in tensor_shapes(cfg)}
