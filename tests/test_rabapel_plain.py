"""The plain Rabapel implementation against closed forms, and the host side of the engine for this
architecture: the configuration reader, the tensor lists, the model description, the cache layout and
the pages a sliding window gives back.  No GPU."""
import json
import math

import numpy as np
import pytest

import plain_rabapel as P
from rabapel_helpers import CONFIGS, RB_A, RB_B, RB_C, random_weights, tensor_shapes


# ----------------------------------------------------------------------------- the oracle's mechanisms

def test_stretched_frequencies():
    base, dims = 10000.0, 16
    plain, one = P.yarn_frequencies(dims, base, None)
    assert one == 1.0 and np.allclose(plain, [base ** (-2 * i / dims) for i in range(8)])
    # a factor of 1 changes nothing
    f, mag = P.yarn_frequencies(dims, base, {"factor": 1.0, "original": 64, "fast": 8.0, "slow": 1.0})
    assert mag == 1.0 and np.allclose(f, plain)
    # pairs that turn often over the trained context stay, pairs that turn rarely are divided, a ramp between
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    f, mag = P.yarn_frequencies(dims, base, sc)
    assert np.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    where = lambda t: dims * math.log(64 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), dims - 1)
    assert 0 <= lo < hi
    for i in range(8):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert np.isclose(f[i], plain[i] * (1 - ramp) + plain[i] / 4.0 * ramp)
    assert np.isclose(f[lo], plain[lo]) and np.isclose(f[-1], plain[-1] / 4.0)
    # both ends at one pair: the ramp is a step (the 0.001 keeps the division defined)
    f, _ = P.yarn_frequencies(4, 10.0, {"factor": 2.0, "original": 8, "fast": 1.2, "slow": 1.1})
    assert np.all(np.isfinite(f))


def test_rotation_of_adjacent_pairs():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2, 10))
    freqs = np.array([1.0, 0.1, 0.01])
    y = P.rotate_pairs(x, [0, 1, 2, 7, 100], 6, freqs, 1.0)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 6:], x[..., 6:])          # position 0; channels beyond dims
    a = 7 * 0.1
    assert np.isclose(y[3, 1, 2], x[3, 1, 2] * math.cos(a) - x[3, 1, 3] * math.sin(a))
    assert np.isclose(y[3, 1, 3], x[3, 1, 3] * math.cos(a) + x[3, 1, 2] * math.sin(a))
    # a rotation keeps lengths; the magnitude scales them
    assert np.allclose(np.linalg.norm(y[..., :6], axis=-1), np.linalg.norm(x[..., :6], axis=-1))
    z = P.rotate_pairs(x, [0, 1, 2, 7, 100], 6, freqs, 1.3)
    assert np.allclose(z[..., :6], 1.3 * y[..., :6]) and np.allclose(z[..., 6:], x[..., 6:])
    # scores of rotated queries and keys depend on the distance only
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    s1 = P.rotate_pairs(q, [13], 6, freqs) @ P.rotate_pairs(k, [4], 6, freqs)[0, 0]
    s2 = P.rotate_pairs(q, [109], 6, freqs) @ P.rotate_pairs(k, [100], 6, freqs)[0, 0]
    assert np.allclose(s1, s2)


def test_window_mask():
    m = P.window_mask(6, 3)
    for i in range(6):
        assert [j for j in range(6) if m[i, j]] == list(range(max(0, i - 2), i + 1))
    assert np.array_equal(P.window_mask(4, 1), np.eye(4, dtype=bool))
    assert np.array_equal(P.window_mask(5, 0), np.tril(np.ones((5, 5), dtype=bool)))
    assert np.array_equal(P.window_mask(5, 50), P.window_mask(5, 0))


def _mixer_weights(rng, H, m):
    nh, d, r, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    return {"q": rng.standard_normal((nh * (d + r), H)) * H ** -0.5, "dkv": rng.standard_normal((kr + r, H)) * H ** -0.5,
            "dkv.norm": 1 + 0.1 * rng.standard_normal(kr), "uk": rng.standard_normal((nh * d, kr)) * kr ** -0.5,
            "uv": rng.standard_normal((nh * dv, kr)) * kr ** -0.5, "g": rng.standard_normal((nh, H)) * H ** -0.5,
            "o": rng.standard_normal((H, nh * dv)) * (nh * dv) ** -0.5}


def test_latent_attention_by_hand():
    """One query position worked out from the definitions, channel by channel, against the function."""
    rng = np.random.default_rng(1)
    H, T, eps = 12, 9, 1e-5
    m = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "scale": 0.37, "mask": {"size": 4},
         "rot": {"base": 50.0, "dims": 4, "scaling": {"factor": 3.0, "original": 8, "fast": 2.0, "slow": 0.5}}}
    w = _mixer_weights(rng, H, m)
    h = rng.standard_normal((T, H))
    out = P.latent_window_attention(h, w, m, eps)
    freqs, mag = P.yarn_frequencies(4, 50.0, m["rot"]["scaling"])

    def turn(v, p):
        r = v.copy()
        for i in range(2):
            c, s = math.cos(p * freqs[i]) * mag, math.sin(p * freqs[i]) * mag
            r[2 * i], r[2 * i + 1] = v[2 * i] * c - v[2 * i + 1] * s, v[2 * i + 1] * c + v[2 * i] * s
        return r
    i = 7
    heads = []
    for hd in range(2):
        q = w["q"][hd * 10:(hd + 1) * 10] @ h[i]
        qn, qr = q[:6], turn(q[6:], i)
        scores, values = [], []
        for j in range(i - 3, i + 1):                         # the window: itself and the three before
            down = w["dkv"] @ h[j]
            c = down[:7] / math.sqrt(np.mean(down[:7] ** 2) + eps) * w["dkv.norm"]
            k = w["uk"][hd * 6:(hd + 1) * 6] @ c
            scores.append((qn @ k + qr @ turn(down[7:], j)) * 0.37)
            values.append(w["uv"][hd * 5:(hd + 1) * 5] @ c)
        p = np.exp(np.array(scores) - max(scores))
        p /= p.sum()
        o = sum(pj * v for pj, v in zip(p, values))
        heads.append(o / (1 + math.exp(-(w["g"][hd] @ h[i]))))
    assert np.allclose(out[i], w["o"] @ np.concatenate(heads), atol=1e-12)
    # the absorbed form (the query mapped into the latent, values expanded after the attention) is the same
    # function: the first position attends to itself alone
    down = w["dkv"] @ h[0]
    c = down[:7] / math.sqrt(np.mean(down[:7] ** 2) + eps) * w["dkv.norm"]
    first = np.concatenate([(w["uv"][hd * 5:(hd + 1) * 5] @ c) / (1 + math.exp(-(w["g"][hd] @ h[0]))) for hd in range(2)])
    assert np.allclose(out[0], w["o"] @ first, atol=1e-12)


def test_feed_forwards_and_router():
    rng = np.random.default_rng(2)
    H, T = 10, 6
    h = rng.standard_normal((T, H))
    up, down = rng.standard_normal((7, H)), rng.standard_normal((H, 7))
    want = (np.maximum(h @ up.T, 0) ** 2) @ down.T
    assert np.allclose(P.relu2_ff(h, {"up": up, "down": down}), want)
    assert np.allclose(P.relu2_ff(-np.abs(h), {"up": np.abs(up), "down": down}), 0.0)       # nothing passes the rectifier
    # the router: the correction steers the choice, the weights are the scores without it and are not renormalised
    router = rng.standard_normal((5, H))
    corr = np.array([0.0, 0.0, 10.0, 0.0, -10.0])
    ids, wts = P.route_softmax(h, router, corr, 2)
    z = h @ router.T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert np.all(ids[:, 0] == 2) and not np.any(ids == 4)
    assert np.allclose(wts[:, 0], s[:, 2]) and np.all(wts.sum(-1) < 1.0)
    ids0, _ = P.route_softmax(h, router, None, 2)
    assert np.array_equal(ids0, np.argsort(-s, axis=-1)[:, :2])
    # ties go to the lower index
    ids_t, w_t = P.route_softmax(np.zeros((1, H)), router, None, 3)
    assert ids_t.tolist() == [[0, 1, 2]] and np.allclose(w_t, 0.2)
    # the mixture: identity experts return their input, the shared expert is gated by one number per token
    mlp = {"router": {"experts": 2, "identity": 3, "top": 2}}
    w = {"router": router, "correction": corr}
    for e in range(2):
        w.update({f"e{e}.gate": rng.standard_normal((4, H)), f"e{e}.up": rng.standard_normal((4, H)),
                  f"e{e}.down": rng.standard_normal((H, 4))})
    out = P.mixture_ff(h, w, mlp)
    ids, wts = P.route_softmax(h, router, corr, 2)
    for t in range(T):
        want = np.zeros(H)
        for e, a in zip(ids[t], wts[t]):
            want += a * (h[t] if e >= 2 else (P.silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])) @ w[f"e{e}.down"].T)
        assert np.allclose(out[t], want)
    w.update({"shared.gate": rng.standard_normal((3, H)), "shared.up": rng.standard_normal((3, H)),
              "shared.down": rng.standard_normal((H, 3)), "shared.sg": rng.standard_normal((1, H))})
    with_shared = P.mixture_ff(h, w, mlp)
    sh = (P.silu(h @ w["shared.gate"].T) * (h @ w["shared.up"].T)) @ w["shared.down"].T
    assert np.allclose(with_shared - out, P.sigmoid(h @ w["shared.sg"].T) * sh)


def test_whole_model_runs_and_layers_are_reported():
    for which, cfg in CONFIGS.items():
        w = {k: v.astype(np.float64) for k, v in random_weights(cfg, 2).items()}
        layers = []
        toks = [1, 5, 3, 0, 7, 7, 2] * 4
        logits = P.forward(cfg, w, toks, layers)
        assert logits.shape == (len(toks), cfg["vocab"]) and len(layers) == len(cfg["layers"]) and np.isfinite(logits).all()
        # causal: a prefix gives the same logits
        assert np.allclose(P.forward(cfg, w, toks[:9])[:9], logits[:9], atol=1e-9)
        # the head reads the table itself: the embedding's scale moves the input only
        x0 = w["embed"][toks] * cfg["embedding"]["scale"]
        h = P.rms_norm(x0, w["l0.norm1"], cfg["norm"]["eps"])
        delta = P.latent_window_attention(h, P._sub(w, "l0.mix."), cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
        mlp = cfg["layers"][0]["mlp"]
        delta = delta + P.relu2_ff(h, P._sub(w, "l0.mlp."))
        assert mlp["kind"] == "dense" and np.allclose(layers[0], x0 + delta, atol=1e-9)


# ----------------------------------------------------------------------------- configuration and tensors

def test_configuration_reader_defaults_errors_and_round_trip():
    from mlxforge_b200.config import ConfigError, config_from_json
    from mlxforge_b200.config.registry import get_architecture
    arch = get_architecture("Rabapel")
    for cfg in (RB_A, RB_B, RB_C):
        c = config_from_json(json.loads(json.dumps(cfg)))
        assert c.architecture == "Rabapel" and len(c.layers) == len(cfg["layers"])
        assert config_from_json(c.to_json()).layers == c.layers
        assert config_from_json(c.to_json()).to_json() == c.to_json()
        assert [(n, tuple(s)) for n, s, _ in arch.random_tensors(c)] == [(n, tuple(s)) for n, s in tensor_shapes(cfg)]
        spec = arch.build_spec(c)
        assert spec.embedding.params["scale"] == cfg["embedding"]["scale"] and spec.head.params["tensor"] == "embed"
        for i, layer in enumerate(cfg["layers"]):
            assert (spec.layers[i].feed_forward is None) == (layer["mlp"] is None)
            assert spec.layers[i].block == "parallel_shared_norm" and spec.layers[i].feed_forward_norm is None
            p = spec.layers[i].mixer.params
            assert p["window"] == (layer["mixer"].get("mask") or {}).get("size", 0)
            assert p["softmax_scale"] == layer["mixer"]["scale"] and p["pairing"] == "pairs" and p["gate_per_head"]
            if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
                f = spec.layers[i].feed_forward.params
                assert f["n_identity"] == layer["mlp"]["router"]["identity"] and f["scoring"] == "softmax"
                assert (f["shared"] is None) == ("shared" not in layer["mlp"])
    # what a file may leave out
    j = json.loads(json.dumps(RB_A))
    del j["embedding"], j["layers"][0]["mixer"]["scale"], j["layers"][0]["mixer"]["vdim"]
    del j["layers"][0]["mixer"]["rot"]["dims"], j["layers"][1]["mlp"]["router"]["identity"]
    c = config_from_json(j)
    m0 = c.layers[0]["mixer"]
    assert c.embedding_scale == 1.0 and m0["vdim"] == 8 and m0["rot_dims"] == 4 and np.isclose(m0["scale"], 12 ** -0.5)
    assert c.layers[1]["mlp"]["identity"] == 0 and c.layers[2]["mixer"]["window"] == 0
    assert c.layers[2]["mixer"]["rot_scaling"] is None

    def broken(path, value):
        j = json.loads(json.dumps(RB_A))
        o = j
        for k in path[:-1]:
            o = o[k]
        if value is None:
            del o[path[-1]]
        else:
            o[path[-1]] = value
        return j
    for path, value, text in [(("width",), None, "'width'"), (("vocab",), 0, "vocab"), (("norm", "eps"), None, "'norm.eps'"),
                              (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
                              (("layers", 0, "type"), "conv", "not supported"),
                              (("layers", 0, "mlp", "kind"), "gated", "not supported"),
                              (("layers", 0, "mixer", "rot_dim"), 3, "rot_dim"),
                              (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
                              (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0, "factor"),
                              (("layers", 0, "mixer", "rot", "scaling", "slow"), None, "slow"),
                              (("layers", 0, "mixer", "mask", "size"), -1, "mask.size"),
                              (("layers", 1, "mlp", "router", "top"), 8, "cannot give"),
                              (("layers", 1, "mlp", "expert"), None, "expert"),
                              (("layers", 1, "mlp", "shared", "ff"), 0, "shared.ff"),
                              (("layers",), [], "layers")]:
        with pytest.raises(ConfigError, match=text):
            config_from_json(broken(path, value))


class _RT:
    precise = True
    device = "cpu"
    stream_max_rows = 16

    def __init__(self):
        import torch
        self.dtype = torch.float32

    def buffer(self, *a, **k):
        raise AssertionError("no scratch at build time")


def test_model_description_declares_the_files_tensors():
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.registry import get_architecture
    from mlxforge_b200.models.decoder import DecoderModel
    for cfg in (RB_A, RB_B, RB_C):
        c = config_from_json(json.loads(json.dumps(cfg)))
        model = DecoderModel(get_architecture("Rabapel").build_spec(c), _RT())
        specs = {k: tuple(v.shape) for k, v in model.tensor_specs().items()}
        assert specs == {n: tuple(s) for n, s in tensor_shapes(cfg)}


def test_cache_layout_groups_by_lane_and_window_and_gives_pages_back():
    import torch
    from mlxforge_b200.cache.manager import CacheManager
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.registry import get_architecture
    from mlxforge_b200.models.decoder import DecoderModel
    from mlxforge_b200.parts.base import PagedKV
    c = config_from_json(json.loads(json.dumps(RB_A)))
    model = DecoderModel(get_architecture("Rabapel").build_spec(c), _RT())
    layout = model.cache_layout
    needs = {(g.need, g.n_lanes) for g in layout.paged}
    # layers 0 and 3 are alike and share a group; only the latent and the shared key part are cached
    assert needs == {(PagedKV(1, 28, 11, v_head_dim=24, values_in_keys=True), 2),
                     (PagedKV(1, 28, 37, v_head_dim=20, values_in_keys=True), 1),
                     (PagedKV(1, 18, 0, v_head_dim=12, values_in_keys=True), 1),
                     (PagedKV(1, 32, 23, v_head_dim=30, values_in_keys=True), 1)}
    assert layout.item_lane[0][1] == layout.item_lane[3][1] and layout.item_lane[0][2] != layout.item_lane[3][2]
    assert not layout.state
    cache = CacheManager(layout, page_size=16, max_tokens=64 * 4, max_seqs=2, dtype=torch.float32, device="cpu")
    seq = cache.open_sequence()
    for n in (50, 1, 1, 30, 1, 40, 1):
        cache.reserve([(seq, n)])
        cache.commit(seq, n)
        for g, gl in enumerate(layout.paged):
            held = [b for b, p in enumerate(seq.blocks[g]) if p >= 0]
            w = gl.need.window
            first = max(0, seq.length - w + 1) // 16 if w else 0       # the next query's oldest visible key
            assert held == list(range(first, len(seq.blocks[g]))), (w, seq.length, held)
        cache.check()
    cache.close(seq)
    assert cache.free_pages() == cache.total_pages()
