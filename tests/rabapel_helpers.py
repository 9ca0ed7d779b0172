"""Small Rabapel configurations that differ in every size and option, random weights for them (made
here, not by the engine's random-weights mode) and model folders written by the tests' own writer."""
from __future__ import annotations

import numpy as np

from helpers import bf16_round, write_model_dir


def _mixer(heads, dim, rot, vdim, rank, base, window=0, scale=None, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
         "scale": (dim + rot) ** -0.5 if scale is None else scale, "rot": {"base": base, "dims": rot}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top, shared=0):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# odd sizes everywhere: a lane 28 wide, key, rotated and value sizes that all differ, a window shorter than
# a page and one that is no multiple of anything, a layer without a mask, one without a feed-forward, a
# mixture without a shared expert in which every expert is chosen, a stretched table whose ramp lies
# inside the pairs
RB_A = {"architecture": "Rabapel", "vocab": 101, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.75},
        "layers": [_layer(_mixer(3, 8, 4, 12, 24, 5000.0, window=11, scale=0.3, scaling=(4.0, 16, 6.0, 1.5)), _dense(20)),
                   _layer(_mixer(2, 16, 8, 8, 20, 90.0, window=37, scaling=(2.5, 24, 3.0, 0.5)), _moe(12, 5, 2, 2, shared=20)),
                   _layer(_mixer(5, 4, 6, 10, 12, 300.0), None),
                   _layer(_mixer(3, 8, 4, 12, 24, 5000.0, window=11, scale=0.3, scaling=(4.0, 16, 6.0, 1.5)), _moe(28, 3, 0, 3)),
                   _layer(_mixer(1, 24, 2, 16, 30, 10000.0, window=23), _dense(36))]}
# everything that can be 1, equal or absent: one head, all four head sizes equal, a window of one token
# (a query sees itself only) and one of exactly one page, a scale of 1 on the embedding, a stretch factor
# of 1, one expert beside one identity expert with one choice, identity experts only beside the experts
# never chosen by the correction
RB_B = {"architecture": "Rabapel", "vocab": 64, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
        "layers": [_layer(_mixer(1, 16, 16, 16, 16, 10000.0, window=1), _dense(32)),
                   _layer(_mixer(2, 8, 8, 8, 8, 50.0, window=16, scaling=(1.0, 32, 4.0, 1.0)), _moe(16, 1, 1, 1, shared=16)),
                   _layer(_mixer(1, 16, 16, 16, 16, 10000.0), _moe(8, 2, 3, 2)),
                   _layer(_mixer(2, 8, 8, 8, 8, 50.0, window=16, scaling=(1.0, 32, 4.0, 1.0)), None)]}
# still small, with the sizes the tensor-core kernels take: lanes 64, 128 and 160 wide, windows longer than
# a tile of keys and shorter than a split, prompts of hundreds of tokens, enough tokens and experts for the
# sorted path of the mixture
RB_C = {"architecture": "Rabapel", "vocab": 320, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25},
        "layers": [_layer(_mixer(4, 32, 16, 32, 48, 100000.0, window=80, scaling=(8.0, 64, 16.0, 2.0)), _dense(256)),
                   _layer(_mixer(6, 16, 32, 48, 96, 20000.0, window=200, scaling=(4.0, 128, 32.0, 1.0)),
                          _moe(64, 8, 2, 3, shared=96)),
                   _layer(_mixer(2, 64, 32, 64, 128, 500000.0, window=130, scaling=(16.0, 32, 8.0, 1.0)), _dense(256)),
                   _layer(_mixer(4, 32, 16, 32, 48, 100000.0, scaling=(8.0, 64, 16.0, 2.0)), _moe(64, 6, 0, 2, shared=64))]}
CONFIGS = {"A": RB_A, "B": RB_B, "C": RB_C}


def random_config(seed, big):
    """A configuration drawn from a seed: two kinds of mixer with sizes, window, base, scale and stretch drawn
    apart, two to five layers that take either, each with a dense feed-forward, a mixture (1 to 16 experts, 0
    to 4 identity experts, 1 to 6 chosen, with or without a shared expert) or none.  ``big``: sizes that the
    tensor-core kernels take among others; else small and odd ones."""
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]

    def mixer():
        heads = pick([1, 2, 3, 4, 6, 8])
        dim = pick([16, 32, 48, 64] if big else [4, 8, 12, 20])
        rot = pick([16, 32, 64] if big else [2, 4, 6, 8])
        vdim = pick([16, 24, 32, 48, 64, 80] if big else [4, 6, 10, 16])
        rank = pick([32, 48, 64, 96, 112, 128, 192] if big else [6, 12, 20, 28])
        window = pick([0, 1, 17, 64, 96, 100, 128, 200, 257])
        scaling = None if rng.random() < 0.2 else (float(pick([2.0, 4.0, 8.0, 16.0])), int(pick([32, 64, 512, 2048])),
                                                   float(pick([8.0, 32.0])), float(pick([0.5, 1.0, 2.0])))
        return _mixer(heads, dim, rot, vdim, rank, float(pick([100.0, 10000.0, 250000.0, 1e6])), window=window,
                      scale=float(pick([0.05, 0.125, 0.2, (dim + rot) ** -0.5])), scaling=scaling)

    width = pick([64, 96, 128, 160, 192, 256, 384] if big else [24, 40, 56, 72, 100])
    mixers = [mixer(), mixer()]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        r = rng.random()
        if r < 0.4:
            mlp = _dense(pick([64, 136, 256, 512] if big else [10, 24, 36]))
        elif r < 0.9:
            e, ident = int(rng.integers(1, 17)), int(rng.integers(0, 5))
            mlp = _moe(pick([32, 64, 96, 136] if big else [8, 12, 20]), e, ident, int(rng.integers(1, min(e + ident, 6) + 1)),
                       shared=pick([0, 64, 128] if big else [0, 12, 16]))
        else:
            mlp = None
        layers.append(_layer(dict(mixers[int(rng.integers(2))]), mlp))
    return {"architecture": "Rabapel", "vocab": int(pick([50, 101, 256, 1000])), "width": width,
            "norm": {"eps": float(pick([1e-6, 1e-5]))}, "embedding": {"scale": float(pick([0.5, 1.0, 2.0, 0.3]))},
            "layers": layers}


def tensor_shapes(cfg):
    H = cfg["width"]
    out = [("embed", (cfg["vocab"], H))]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        nh, d, r, dv, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        out += [(p + "norm1", (H,)), (p + "mix.q", (nh * (d + r), H)), (p + "mix.dkv", (kr + r, H)),
                (p + "mix.dkv.norm", (kr,)), (p + "mix.uk", (nh * d, kr)), (p + "mix.uv", (nh * dv, kr)),
                (p + "mix.g", (nh, H)), (p + "mix.o", (H, nh * dv))]
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out += [(p + "mlp.up", (mlp["ff"], H)), (p + "mlp.down", (H, mlp["ff"]))]
            continue
        ff, r_ = mlp["expert"]["ff"], mlp["router"]
        for e in range(r_["experts"]):
            out += [(p + f"mlp.e{e}.gate", (ff, H)), (p + f"mlp.e{e}.up", (ff, H)), (p + f"mlp.e{e}.down", (H, ff))]
        n_out = r_["experts"] + r_.get("identity", 0)
        out += [(p + "mlp.router", (n_out, H)), (p + "mlp.correction", (n_out,))]
        if mlp.get("shared"):
            fs = mlp["shared"]["ff"]
            out += [(p + "mlp.shared.gate", (fs, H)), (p + "mlp.shared.up", (fs, H)), (p + "mlp.shared.down", (H, fs)),
                    (p + "mlp.shared.sg", (1, H))]
    out.append(("final.norm", (H,)))
    return out


def random_weights(cfg, seed, qk_gain=1.0):
    """float32 arrays, exact in bfloat16.  ``qk_gain`` scales what makes queries and keys (``q`` and ``uk``) so
    that the softmax is peaked and a wrong or missing key shows.  The router's rows are large enough for
    clear choices, its correction large enough to change some of them."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg):
        n = lambda std: rng.standard_normal(shape).astype(np.float32) * np.float32(std)
        leaf = name.split(".")[-1]
        if name == "embed":
            a = n(0.5)
        elif leaf in ("norm1", "norm"):
            a = 1.0 + n(0.1)
        elif leaf == "correction":
            a = n(0.15)
        elif leaf == "router":
            a = n(3.0 / np.sqrt(shape[1]))
        else:
            a = n(1.2 / np.sqrt(shape[1]))
            if leaf in ("q", "uk"):
                a = a * np.float32(qk_gain)
        w[name] = bf16_round(a.astype(np.float32))
    return w


def make_model(tmp_path, which, seed=0, qk_gain=1.0):
    cfg = CONFIGS[which]
    w = random_weights(cfg, seed, qk_gain)
    d = write_model_dir(str(tmp_path / f"rabapel_{which}_{seed}_{qk_gain}"), cfg, w, "bfloat16")
    return d, cfg, {k: v.astype(np.float64) for k, v in w.items()}


def prompt(cfg, n, seed):
    return np.random.default_rng(7000 + seed).integers(0, cfg["vocab"], size=n).tolist()
