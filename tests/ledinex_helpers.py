"""Small Ledinex configurations that differ in every size and option, random weights for them (made
here, not by the engine's random-weights mode) and model folders written by the tests' own writer."""
from __future__ import annotations

import numpy as np

from helpers import bf16_round, write_model_dir

RANK = "decay_rank"     # the low rank of a parallel_2 layer's decay: in the tensors' shapes, not in config.json


def _rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = {"factor": scaling[0]} if len(scaling) == 1 else dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _attn(heads, kv, dim, vdim, scale, rot=None, window=0, softcap=0.0):
    a = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        a["rot"] = rot
    if window:
        a["mask"] = {"size": window}
    if softcap:
        a["softcap"] = softcap
    return a


def _par(left, heads, dim, vdim, decay, ls=1.0, rs=1.0):
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
                                          "left_scale": ls, "right_scale": rs}}


def _par2(left, heads, dim, rank, ls=1.0, rs=1.0):
    return {"type": "parallel_2", "mixer": {"left": left, "right": {"heads": heads, "dim": dim, RANK: rank},
                                            "left_scale": ls, "right_scale": rs}}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _moe(ff, experts, top, shared=0):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


# odd sizes everywhere: key, value and rotated sizes that all differ (values wider than keys in one layer),
# windows shorter than a page and no multiple of anything, a layer without a feed-forward, a mixture in which
# every expert is chosen and one without a shared expert, three taps
LX_A = {"architecture": "Ledinex", "vocab": 101, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
        "logit_scale": 1.5, "canon": {"taps": 3},
        "layers": [_with(_par2(_attn(4, 2, 12, 12, 0.3, _rot(5000.0, 8, (4.0, 16, 6.0, 1.5)), window=11), 3, 10, 5, 0.8, 0.9),
                         _moe(12, 5, 2, shared=20)),
                   _with(_delta(4, 2, 6, 10, 3), None),
                   _with(_par(_attn(6, 3, 8, 12, 0.35, _rot(300.0, 6, (2.5,)), softcap=7.0), 2, 10, 6, [0.9, 0.5], 1.2, 0.7),
                         _moe(28, 3, 3)),
                   _with(_par2(_attn(2, 1, 20, 20, 0.2, _rot(90.0, 20, (2.5, 24, 3.0, 0.5)), window=37), 1, 14, 3, 0.5, 1.1),
                         _moe(12, 4, 1, shared=8)),
                   _with(_delta(3, 3, 10, 4, 2), _moe(8, 6, 2))]}
# everything that can be 1, equal or absent: no convolution on the inputs, scales of 1, one head, equal head sizes,
# a window of one token and one of exactly a page, no soft cap, no rotation in one layer, a factor of 1, one
# expert, decays of 1 and 0, a convolution of one tap in the delta mixer
LX_B = {"architecture": "Ledinex", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
        "layers": [_with(_par(_attn(1, 1, 16, 16, 0.25), 2, 16, 16, [1.0, 0.0]), _moe(16, 1, 1)),
                   _with(_par2(_attn(1, 1, 16, 16, 0.25, _rot(10000.0, 16), window=1), 1, 16, 1), None),
                   _with(_delta(1, 1, 16, 16, 1), _moe(8, 2, 2, shared=16)),
                   _with(_par2(_attn(2, 2, 8, 8, 0.3, _rot(50.0, 8, (1.0, 32, 4.0, 1.0)), window=16), 2, 8, 2), _moe(8, 2, 1)),
                   _with(_par(_attn(2, 1, 8, 8, 0.3, _rot(50.0, 8, (1.0,))), 1, 8, 8, [0.5]), None)]}
# still small, with the sizes the tensor-core kernels take: head sizes 64 and 128, values narrower than keys,
# windows longer than a tile of keys and shorter than a split, prompts of hundreds of tokens, enough tokens
# and experts for the sorted path of the mixture, four taps
LX_C = {"architecture": "Ledinex", "vocab": 320, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 12.0},
        "logit_scale": 0.5, "canon": {"taps": 4},
        "layers": [_with(_par2(_attn(4, 2, 64, 64, 0.11, _rot(100000.0, 32, (8.0, 64, 16.0, 2.0)), window=80), 3, 64, 16, 0.8, 0.9),
                         _moe(64, 8, 3, shared=96)),
                   _with(_delta(4, 2, 64, 64, 4), _moe(64, 6, 2, shared=64)),
                   _with(_par(_attn(4, 1, 128, 64, 0.08, _rot(250000.0, 128, (8.0,)), softcap=30.0), 4, 32, 64,
                              [0.6, 0.88, 0.97, 0.999], 0.7, 1.1), _moe(64, 8, 3, shared=96)),
                   _with(_par2(_attn(2, 2, 128, 128, 0.09, _rot(20000.0, 64, (4.0, 128, 32.0, 1.0)), window=200), 2, 32, 8),
                         None)]}
CONFIGS = {"A": LX_A, "B": LX_B, "C": LX_C}


def random_config(seed, big):
    """A configuration drawn from a seed: two to five layers of the three types with sizes, windows, bases,
    scales, caps, decays and taps drawn apart, each with a mixture (with or without a shared expert) or none.
    ``big``: sizes that the tensor-core kernels take among others; else small and odd ones."""
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]

    def attn(own_values):
        kv = pick([1, 2, 3])
        heads = kv * pick([1, 2, 3])
        dim = pick([32, 64, 96, 128] if big else [4, 8, 12, 20])
        vdim = pick([dim, dim // 2, 32] if big else [dim, 6, 10]) if own_values else dim
        dims = pick([dim, dim // 2, 0] if big else [dim, 2, 4])
        if own_values:
            vdim += vdim % 2
            sc = pick([None, (2.0,), (4.0,)])
        else:
            sc = pick([None, (4.0, 2048, 32.0, 1.0), (2.5, 64, 8.0, 0.5), (16.0, 512, 32.0, 2.0)])
        rot = _rot(float(pick([100.0, 10000.0, 250000.0])), dims, sc) if dims else None
        return _attn(heads, kv, dim, vdim, float(pick([0.05, 0.125, 0.2, dim ** -0.5])), rot,
                     window=0 if own_values else pick([1, 17, 40, 64, 100, 129]),
                     softcap=float(pick([0.0, 5.0, 50.0])) if own_values else 0.0)

    def layer():
        r = rng.random()
        ls, rs = float(pick([1.0, 0.8, 0.5])), float(pick([1.0, 0.9, 1.3]))
        if r < 0.4:
            return _par2(attn(False), pick([1, 2, 6]), pick([16, 32, 64] if big else [4, 10, 12]), pick([1, 4, 16]), ls, rs)
        if r < 0.7:
            h = pick([1, 2, 4])
            return _par(attn(True), h, pick([16, 32, 64] if big else [4, 10]), pick([16, 32, 64] if big else [6, 8]),
                        [float(pick([0.5, 0.9, 0.97, 0.999, 1.0])) for _ in range(h)], ls, rs)
        kv = pick([1, 2])
        return _delta(kv * pick([1, 2]), kv, pick([16, 32, 64] if big else [4, 6, 12]), pick([16, 32, 64] if big else [4, 10]),
                      pick([1, 2, 4]))

    width = pick([64, 96, 128, 192, 256] if big else [24, 40, 56, 72])
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        e = int(rng.integers(1, 17))
        mlp = None if rng.random() < 0.15 else _moe(pick([32, 64, 96] if big else [8, 12, 20]), e,
                                                    int(rng.integers(1, min(e, 4) + 1)), shared=pick([0, 64, 128] if big else [0, 12]))
        layers.append(_with(layer(), mlp))
    return {"architecture": "Ledinex", "vocab": int(pick([50, 101, 256, 1000])), "width": width,
            "norm": {"eps": float(pick([1e-6, 1e-5]))}, "embedding": {"scale": float(pick([1.0, 4.0, 16.0]))},
            "logit_scale": float(pick([1.0, 2.0, 0.3])), **({"canon": {"taps": int(pick([1, 2, 3, 4]))}} if rng.random() < 0.9 else {}), "layers": layers}


def tensor_shapes(cfg):
    H, taps = cfg["width"], (cfg.get("canon") or {}).get("taps", 0)      # no canon: no convolution, no tensors
    out = [("embed", (cfg["vocab"], H))]
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        out += [(p + "norm1", (H,))] + ([(p + "canon1", (H, taps))] if taps else [])
        if kind == "delta":
            nqk, nv, nh = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"]
            out += [(p + "mix.q", (nqk, H)), (p + "mix.q.conv", (nqk, m["conv"])), (p + "mix.k", (nqk, H)),
                    (p + "mix.k.conv", (nqk, m["conv"])), (p + "mix.v", (nv, H)), (p + "mix.v.conv", (nv, m["conv"])),
                    (p + "mix.b", (nh, H)), (p + "mix.a", (nh, H)), (p + "mix.A_log", (nh,)), (p + "mix.dt_bias", (nh,)),
                    (p + "mix.g", (nv, H)), (p + "mix.norm", (m["vdim"],)), (p + "mix.o", (H, nv))]
        else:
            a, r, q = m["left"], m["right"], p + "mix.left."
            nq, nk = a["heads"] * a["dim"], a["kv_heads"] * a["dim"]
            out += [(q + "q", (nq, H)), (q + "k", (nk, H)), (q + "q.norm", (nq,)), (q + "k.norm", (nk,)),
                    (q + "o", (H, a["heads"] * a["vdim"]))]
            if kind == "parallel":
                out += [(q + "v", (a["kv_heads"] * a["vdim"], H))]
            else:
                out += [(q + "q.b", (nq,)), (q + "k.b", (nk,))]
            q, n = p + "mix.right.", r["heads"] * r["dim"]
            if kind == "parallel":
                nv = r["heads"] * r["vdim"]
                out += [(q + "q", (n, H)), (q + "k", (n, H)), (q + "v", (nv, H)), (q + "g", (nv, H)), (q + "norm", (nv,)),
                        (q + "o", (H, nv))]
            else:
                out += [(q + t, (n, H)) for t in ("r", "k", "v", "a", "g")]
                out += [(q + "a.b", (n,)), (q + "w1", (r[RANK], H)), (q + "w2", (n, r[RANK])), (q + "w0", (n,)),
                        (q + "norm", (n,)), (q + "o", (H, n))]
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out += [(p + "norm2", (H,))] + ([(p + "canon2", (H, taps))] if taps else [])
        out += [(p + "mlp.router", (mlp["router"]["experts"], H))]
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            out += [(p + f"mlp.e{e}.up", (ff, H)), (p + f"mlp.e{e}.down", (H, ff))]
        if mlp.get("shared"):
            out += [(p + "mlp.shared.up", (mlp["shared"]["ff"], H)), (p + "mlp.shared.down", (H, mlp["shared"]["ff"]))]
    out.append(("final.norm", (H,)))
    return out


def random_weights(cfg, seed, qk_gain=1.0):
    """float32 arrays, exact in bfloat16.  ``qk_gain`` scales the attention's query and key norm weights so
    that the softmax is peaked and a wrong or missing key shows.  The router's rows are large enough for clear
    choices."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg):
        n = lambda std: rng.standard_normal(shape).astype(np.float32) * np.float32(std)
        parts = name.split(".")
        leaf = parts[-1]
        if name == "embed":
            a = n(0.5)
        elif leaf in ("norm1", "norm2") or name == "final.norm":
            a = n(0.2)                          # stored around zero: 1 + w multiplies
        elif leaf in ("canon1", "canon2"):
            a = n(0.3)
        elif leaf == "norm" and parts[-2] in ("q", "k"):
            a = (1.0 + n(0.1)) * np.float32(qk_gain)
        elif leaf == "norm":
            a = 1.0 + n(0.1)
        elif leaf == "conv":
            a = n(0.5)
        elif leaf in ("A_log", "dt_bias", "w0", "b") and len(shape) == 1:
            a = n(0.7)
        elif leaf == "router":
            a = n(3.0 / np.sqrt(shape[1]))
        else:
            a = n(1.2 / np.sqrt(shape[-1]))
        w[name] = bf16_round(a.astype(np.float32))
    return w


def make_model(tmp_path, which, seed=0, qk_gain=1.0):
    cfg = CONFIGS[which]
    w = random_weights(cfg, seed, qk_gain)
    d = write_model_dir(str(tmp_path / f"ledinex_{which}_{seed}_{qk_gain}"), file_config(cfg), w, "bfloat16")
    return d, cfg, {k: v.astype(np.float64) for k, v in w.items()}


def file_config(cfg):
    """The configuration as a file has it: without the sizes that only the tensors' shapes say."""
    import copy
    c = copy.deepcopy(cfg)
    for layer in c["layers"]:
        if layer["type"] == "parallel_2":
            layer["mixer"]["right"].pop(RANK, None)
    return c


def prompt(cfg, n, seed):
    return np.random.default_rng(9000 + seed).integers(0, cfg["vocab"], size=n).tolist()
