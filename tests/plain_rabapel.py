"""A plain, slow implementation of the Rabapel decoder in NumPy float64: whole sequences, no cache,
no batching, one function per mechanism.  It shares no code with the engine and is the oracle its
kernels are compared with.

Notation.  ``W`` of a linear map is stored ``[out, in]`` and applied as ``x @ W.T``.  A sequence is
``T`` tokens at positions ``0 .. T-1``.  A layer is ``x + mixer(n(x)) + ff(n(x))`` with ONE norm
``n`` whose output both branches read.

* ``rms_norm``              ``x / sqrt(mean(x^2) + eps) * w``
* ``yarn_frequencies``      the rotary frequencies after the blend between stretched and plain ones,
                            and the factor on cosine and sine
* ``rotate_pairs``          channel ``2i`` with ``2i + 1`` over the first ``dims`` channels of a head
* ``window_mask``           query i sees key j iff ``0 <= i - j < size`` (size 0: plain causal)
* ``latent_window_attention``  queries projected directly, keys and values expanded from a normed
                            latent all heads share, one rotated key part all heads share, sliding
                            window, one gate number per head
* ``relu2_ff``              ``W_d relu(W_u x)^2``
* ``route_softmax``         softmax scores, choice by score plus a correction, weights without it
* ``expert_ff``             ``W_d (silu(W_g x) * (W_u x))``
* ``mixture_ff``            routed experts, identity experts, the gated shared expert
"""
from __future__ import annotations

import math

import numpy as np

ROUND = None          # a function applied to activations where a bfloat16 engine rounds; None = exact


def _r(x):
    return x if ROUND is None else ROUND(x)


def round_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint32) << 16
    return u.view(np.float32).astype(np.float64)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def rms_norm(x, w, eps):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


# ----------------------------------------------------------------------------- rotary positions

def yarn_frequencies(dims, base, scaling):
    """(frequency of every pair [dims/2], factor on cos and sin).  ``scaling`` None: the plain
    frequencies ``base^(-2i/dims)`` and 1.  Else a dict with ``factor, original, fast, slow``: pairs
    that turn fast keep their frequency, pairs that turn slowly get it divided by ``factor``, with a
    linear ramp over the pair index between the two turning counts."""
    half = dims // 2
    f = np.array([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, dims, freqs, magnitude=1.0):
    """x [T, heads, d]: channels (2i, 2i+1), i < dims/2, turned by ``position * freqs[i]``; cosine
    and sine both times ``magnitude``; channels from ``dims`` on unchanged."""
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * np.asarray(freqs)[None, None, :]
    c, s = np.cos(a) * magnitude, np.sin(a) * magnitude
    out = np.array(x, dtype=np.float64, copy=True)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mask

def window_mask(T, size):
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    d = i - j
    return (d >= 0) & ((d < size) if size > 0 else True)


# ----------------------------------------------------------------------------- mixer

def latent_window_attention(h, w, m, eps, positions=None):
    """``h`` [T, H] (the normed input); ``w``: dict of the mixer's tensors (``q, dkv, dkv.norm, uk,
    uv, g, o``); ``m``: the mixer's sizes and constants.  Keys and values are expanded per head."""
    T = h.shape[0]
    nh, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", r))
    pos = np.arange(T) if positions is None else np.asarray(positions)
    freqs, mag = yarn_frequencies(dims, rot.get("base", 10000.0), rot.get("scaling")) if dims else (np.zeros(0), 1.0)
    q = _r(h @ w["q"].T).reshape(T, nh, d + r)
    q_plain, q_rot = q[..., :d], _r(rotate_pairs(q[..., d:], pos, dims, freqs, mag))
    down = _r(h @ w["dkv"].T)
    c = _r(rms_norm(down[:, :rank], w["dkv.norm"], eps))
    k_rot = _r(rotate_pairs(down[:, None, rank:], pos, dims, freqs, mag))[:, 0]       # [T, r], one for all heads
    k_plain = _r(c @ w["uk"].T).reshape(T, nh, d)
    v = _r(c @ w["uv"].T).reshape(T, nh, dv)
    s = (np.einsum("ihd,jhd->hij", q_plain, k_plain) + np.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    mask = window_mask(T, int((m.get("mask") or {}).get("size", 0)))
    s = np.where(mask[None], s, -np.inf)
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    p = p / p.sum(axis=-1, keepdims=True)
    o = np.einsum("hij,jhv->ihv", p, v)
    if "g" in w:
        o = o * sigmoid(h @ w["g"].T)[:, :, None]            # one number per (token, head)
    return _r(o).reshape(T, nh * dv) @ w["o"].T


# ----------------------------------------------------------------------------- feed-forwards

def relu2_ff(h, w):
    a = np.maximum(h @ w["up"].T, 0.0)
    return _r(a * a) @ w["down"].T


def expert_ff(h, gate, up, down):
    return _r(silu(h @ gate.T) * (h @ up.T)) @ down.T


def route_softmax(h, router, correction, top):
    """(chosen [T, top] in the order of the choice, their weights [T, top]).  Ties go to the lower index."""
    z = h @ router.T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s if correction is None else s + correction
    order = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def choice_margin(h, router, correction, top):
    """[T]: how far the last chosen expert's choice score lies above the first one left out (infinite when
    every output is chosen).  A small margin is a close call that rounding may turn the other way."""
    z = h @ router.T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s = s / s.sum(axis=-1, keepdims=True)
    c = -np.sort(-(s if correction is None else s + correction), axis=-1)
    return c[:, top - 1] - c[:, top] if c.shape[1] > top else np.full(h.shape[0], np.inf)


def mixture_ff(h, w, mlp):
    """``w``: the feed-forward's tensors (``router, correction, e<i>.gate|up|down, shared.gate|up|down|sg``);
    ``mlp``: its configuration.  The router has ``experts + identity`` outputs; the last ``identity`` of
    them stand for experts that return their input."""
    n_real = int(mlp["router"]["experts"])
    top = int(mlp["router"]["top"])
    ids, weights = route_softmax(h, w["router"], w.get("correction"), top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(ids[t, k])
            y = h[t] if e >= n_real else expert_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            out[t] += weights[t, k] * y
    if "shared.gate" in w:
        out = out + sigmoid(h @ w["shared.sg"].T) * expert_ff(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


# ----------------------------------------------------------------------------- the model

def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one whole sequence.  ``tensors``: name -> float64 array.  ``layers_out``: a
    list that receives the residual stream after every layer; ``margins_out``: a list that receives every
    mixture layer's ``choice_margin`` [T]."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"][np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _r(rms_norm(x, tensors[p + "norm1"], eps))
        delta = _r(latent_window_attention(h, _sub(tensors, p + "mix."), layer["mixer"], eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            w = _sub(tensors, p + "mlp.")
            if margins_out is not None and mlp["kind"] != "dense":
                margins_out.append(choice_margin(h, w["router"], w.get("correction"), int(mlp["router"]["top"])))
            delta = delta + _r(relu2_ff(h, w) if mlp["kind"] == "dense" else mixture_ff(h, w, mlp))
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.copy())
    hn = _r(rms_norm(x, tensors["final.norm"], eps))
    return hn @ tensors["embed"].T
