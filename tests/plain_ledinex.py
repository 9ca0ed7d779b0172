"""A plain, slow implementation of the Ledinex decoder in NumPy float64: whole sequences, no cache,
no batching, one function per mechanism.  It shares no code with the engine and is the oracle its
kernels are compared with.

Notation.  ``W`` of a linear map is stored ``[out, in]`` and applied as ``x @ W.T``.  A sequence is
``T`` tokens at positions ``0 .. T-1``.  A layer is ``x + n1(mixer(c1(x)))`` followed by
``x + n2(ff(c2(x)))``: the norms sit on the sublayers' outputs, and what a sublayer reads is the
stream itself plus a short causal convolution of it (``c(x) = x + conv(x)``).

* ``rms_norm`` / ``norm_one_plus``  ``x / sqrt(mean(x^2) + eps)`` times ``w`` / times ``1 + w``
* ``input_convolution``     ``x_t + sum_j w[:, j] x_(t - taps + 1 + j)``, zeros before the start
* ``causal_convolution``    the sum alone (the delta mixer's short convolutions)
* ``linear_frequencies`` / ``stretched_frequencies``  rotary frequencies divided by a factor / blended
                            between stretched and plain ones with a factor on cosine and sine
* ``rotate_half``           channel ``i`` with ``i + dims/2`` over the first ``dims`` channels of a head
* ``softmax_attention``     grouped queries, scale, soft cap, causal or sliding window
* ``capped_attention``      the left branch of ``parallel``: whole-projection norms, rotated values
* ``window_attention``      the left branch of ``parallel_2``: biases, values that are the raw keys
* ``lightning``             the right branch of ``parallel``: a state with a fixed decay per head
* ``generalized_delta``     the right branch of ``parallel_2``: decay and removal per key channel
* ``gated_delta``           the ``delta`` mixer: one decay per head, short convolutions
* ``route`` / ``mixture``   softmax router, renormalised weights, squared-rectifier experts
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


def round_f32(x):
    return np.asarray(x, dtype=np.float32).astype(np.float64)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def lin(x, W, b=None):
    y = _r(x) @ np.asarray(W, dtype=np.float64).T
    return y if b is None else y + np.asarray(b, dtype=np.float64)


def rms_norm(x, w, eps):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def norm_one_plus(x, w, eps):
    return rms_norm(x, 1.0 + np.asarray(w, dtype=np.float64), eps)


# ----------------------------------------------------------------------------- convolutions over time

def causal_convolution(x, w):
    """x [T, C], w [C, taps]: ``y_t = sum_j w[:, j] x_(t - taps + 1 + j)``, zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * w[:, j]
    return y


def input_convolution(x, w):
    return x + causal_convolution(x, np.asarray(w, dtype=np.float64))


# ----------------------------------------------------------------------------- rotary positions

def plain_frequencies(dims, base):
    return np.array([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def linear_frequencies(dims, base, factor):
    return plain_frequencies(dims, base) / float(factor), 1.0


def stretched_frequencies(dims, base, scaling):
    """(frequency of every pair, factor on cosine and sine) with ``factor, original, fast, slow``."""
    f = plain_frequencies(dims, base)
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def frequencies_of(rot):
    """From a ``rot`` object ``{base, dims, scaling}``: no scaling, a factor alone, or the stretched form."""
    dims, base, sc = int(rot["dims"]), float(rot["base"]), rot.get("scaling")
    if not sc:
        return plain_frequencies(dims, base), 1.0
    if "original" in sc:
        return stretched_frequencies(dims, base, sc)
    return linear_frequencies(dims, base, sc["factor"])


def rotate_half(x, positions, dims, freqs, magnitude=1.0, sign=1.0):
    """x [T, heads, d]: channels (i, i + dims/2), i < dims/2, turned by ``sign * position * freqs[i]``."""
    half = dims // 2
    a = sign * np.asarray(positions, dtype=np.float64)[:, None, None] * np.asarray(freqs)[None, None, :]
    c, s = np.cos(a) * magnitude, np.sin(a) * magnitude
    y = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    y[..., :half] = u * c - v * s
    y[..., half:dims] = v * c + u * s
    return y


# ----------------------------------------------------------------------------- softmax attention

def visible(T, window):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    m = j <= i
    if window:
        m &= (i - j) < window
    return m


def softmax_attention(q, k, v, scale, softcap=0.0, window=0):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query head h reads key head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    mask = visible(T, window)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def _heads(x, n):
    return x.reshape(x.shape[0], n, -1)


def capped_attention(h, W, c, eps):
    """Left branch of ``parallel``.  ``W``: tensors by their names behind the branch's prefix."""
    T = h.shape[0]
    H, G, d, dv = int(c["heads"]), int(c.get("kv_heads") or c["heads"]), int(c["dim"]), int(c.get("vdim") or c["dim"])
    pos = np.arange(T)
    q = rms_norm(lin(h, W["q"]), W["q.norm"], eps)
    k = rms_norm(lin(h, W["k"]), W["k.norm"], eps)
    v = _heads(lin(h, W["v"]), G)
    rot = c.get("rot")
    q, k = _heads(q, H), _heads(k, G)
    if rot:
        f, mag = frequencies_of(rot)
        q = rotate_half(q, pos, int(rot["dims"]), f, mag)
        k = rotate_half(k, pos, int(rot["dims"]), f, mag)
    fv = plain_frequencies(dv, float((rot or {}).get("base", 10000.0)))
    v = rotate_half(v, pos, dv, fv)
    o = softmax_attention(_r(q), _r(k), _r(v), float(c["scale"]), float(c.get("softcap") or 0.0),
                          int((c.get("mask") or {}).get("size") or 0))
    o = rotate_half(o, pos, dv, fv, sign=-1.0)
    return lin(o.reshape(T, H * dv), W["o"])


def window_attention(h, W, c, eps):
    """Left branch of ``parallel_2``: the values are the keys as projected (with their bias)."""
    T = h.shape[0]
    H, G, d = int(c["heads"]), int(c.get("kv_heads") or c["heads"]), int(c["dim"])
    pos = np.arange(T)
    q0 = lin(h, W["q"], W["q.b"])
    k0 = lin(h, W["k"], W["k.b"])
    v = _heads(k0, G)
    q = rms_norm(q0, W["q.norm"], eps)
    k = rms_norm(k0, W["k.norm"], eps)
    rot = c.get("rot")
    q, k = _heads(q, H), _heads(k, G)
    if rot:
        f, mag = frequencies_of(rot)
        q = rotate_half(q, pos, int(rot["dims"]), f, mag)
        k = rotate_half(k, pos, int(rot["dims"]), f, mag)
    o = softmax_attention(_r(q), _r(k), _r(v), float(c["scale"]), float(c.get("softcap") or 0.0),
                          int((c.get("mask") or {}).get("size") or 0))
    return lin(o.reshape(T, -1), W["o"])


# ----------------------------------------------------------------------------- recurrent branches

def lightning(h, W, c, eps):
    """Right branch of ``parallel``: ``S <- decay_h S + k v^T``, ``o = S^T q`` per head."""
    T = h.shape[0]
    H, d = int(c["heads"]), int(c["dim"])
    dv = int(c.get("vdim") or d)
    q = _heads(silu(lin(h, W["q"])), H)
    k = _heads(silu(lin(h, W["k"])), H)
    v = _heads(silu(lin(h, W["v"])), H)
    o = np.zeros((T, H, dv))
    for hd in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = float(c["decay"][hd]) * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    y = rms_norm(o.reshape(T, H * dv), W["norm"], eps) * sigmoid(lin(h, W["g"]))
    return lin(y, W["o"])


def generalized_delta(h, W, c, eps):
    """Right branch of ``parallel_2``: ``S <- diag(w) S - (a u)(u^T S) + k v^T`` (both terms read the old
    state), ``o = S^T r``."""
    T = h.shape[0]
    H, d = int(c["heads"]), int(c["dim"])
    r = _heads(lin(h, W["r"]), H)
    k = _heads(lin(h, W["k"]), H)
    v = _heads(lin(h, W["v"]), H)
    w = np.exp(-math.exp(-0.5) * sigmoid(lin(np.tanh(lin(h, W["w1"])), W["w2"]) + W["w0"]))
    w = _heads(w, H)
    a = _heads(sigmoid(lin(h, W["a"], W["a.b"])), H)
    u = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    o = np.zeros((T, H, d))
    for hd in range(H):
        S = np.zeros((d, d))
        for t in range(T):
            S = w[t, hd][:, None] * S - np.outer(a[t, hd] * u[t, hd], u[t, hd] @ S) + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ r[t, hd]
    o = rms_norm(o, None, eps)
    y = o.reshape(T, H * d) * W["norm"] * sigmoid(lin(h, W["g"]))
    return lin(y, W["o"])


def gated_delta(h, W, c, eps):
    """The ``delta`` mixer: ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``."""
    T = h.shape[0]
    H, G, d, dv = int(c["heads"]), int(c["kv_heads"]), int(c["dim"]), int(c["vdim"])
    q = _heads(silu(causal_convolution(lin(h, W["q"]), W["q.conv"])), G)
    k = _heads(silu(causal_convolution(lin(h, W["k"]), W["k.conv"])), G)
    v = _heads(silu(causal_convolution(lin(h, W["v"]), W["v.conv"])), H)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(lin(h, W["b"]))
    g = np.exp(-np.exp(W["A_log"]) * softplus(lin(h, W["a"]) + W["dt_bias"]))
    o = np.zeros((T, H, dv))
    for hd in range(H):
        kv = hd // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            o[t, hd] = S.T @ q[t, kv]
    o = rms_norm(o, W["norm"], eps)
    y = o.reshape(T, H * dv) * silu(lin(h, W["g"]))
    return lin(y, W["o"])


# ----------------------------------------------------------------------------- feed-forward

def relu2_ff(h, up, down):
    return lin(np.maximum(lin(h, up), 0.0) ** 2, down)


def route(h, Wr, top):
    """(ids [T, top], weights [T, top], scores [T, E]): the largest scores, ties to the lower index."""
    z = lin(h, Wr)
    e = np.exp(z - z.max(axis=1, keepdims=True))
    s = e / e.sum(axis=1, keepdims=True)
    ids = np.argsort(-s, axis=1, kind="stable")[:, :top]
    w = np.take_along_axis(s, ids, axis=1)
    return ids, w / (w.sum(axis=1, keepdims=True) + 1e-20), s


def choice_margins(h, Wr, top):
    """Per token, how far the router's last chosen logit lies above the first rejected one, relative to the
    largest logit; infinite where every expert is chosen or where the expert in question would get a
    weight below a thousandth either way (then the choice moves nothing)."""
    z = lin(h, Wr)
    if z.shape[1] <= top:
        return np.full(z.shape[0], np.inf)
    zs = -np.sort(-z, axis=1)
    e = np.exp(zs - zs[:, :1])
    weight = e[:, top - 1] / e[:, :top].sum(axis=1)
    m = (zs[:, top - 1] - zs[:, top]) / np.maximum(1.0, np.abs(z).max(axis=1))
    return np.where(weight < 1e-3, np.inf, m)


def mixture(h, W, c):
    """``W``: tensors by name behind the feed-forward's prefix (``router``, ``e<i>.up`` ...)."""
    ids, w, _ = route(h, W["router"], int(c["router"]["top"]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += w[t, j] * relu2_ff(h[t:t + 1], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if c.get("shared"):
        out += relu2_ff(h, W["shared.up"], W["shared.down"])
    return out


# ----------------------------------------------------------------------------- the model

def _sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: np.asarray(v, dtype=np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def mixer_forward(h, layer, W, eps):
    kind, c = layer["type"], layer["mixer"]
    if kind == "delta":
        return gated_delta(h, W, c, eps)
    L, R = _sub(W, "left."), _sub(W, "right.")
    if kind == "parallel":
        left, right = capped_attention(h, L, c["left"], eps), lightning(h, R, c["right"], eps)
    elif kind == "parallel_2":
        left, right = window_attention(h, L, c["left"], eps), generalized_delta(h, R, c["right"], eps)
    else:
        raise ValueError(f"unknown layer type {kind}")
    return float(c["left_scale"]) * left + float(c["right_scale"]) * right


def forward(config, tensors, tokens, layers_out=None, choices_out=None):
    """Logits [T, vocab] of one sequence.  ``tensors``: name -> array.  ``layers_out``: a list that gets
    the stream after every layer.  ``choices_out``: a list that gets, per layer with experts, the margin of
    every token's choice (``choice_margins``)."""
    eps = float(config["norm"]["eps"])
    E = np.asarray(tensors["embed"], dtype=np.float64)
    x = E[np.asarray(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = _r(input_convolution(x, tensors[p + "canon1"]) if p + "canon1" in tensors else x)
        x = x + norm_one_plus(mixer_forward(h, layer, _sub(tensors, p + "mix."), eps), tensors[p + "norm1"], eps)
        if layer.get("mlp"):
            h = _r(input_convolution(x, tensors[p + "canon2"]) if p + "canon2" in tensors else x)
            W = _sub(tensors, p + "mlp.")
            x = x + norm_one_plus(mixture(h, W, layer["mlp"]), tensors[p + "norm2"], eps)
            if choices_out is not None:
                choices_out.append(choice_margins(h, W["router"], int(layer["mlp"]["router"]["top"])))
        if layers_out is not None:
            layers_out.append(x.copy())
    hn = norm_one_plus(x, tensors["final.norm"], eps)
    return lin(hn, E) * float(config.get("logit_scale", 1.0))
