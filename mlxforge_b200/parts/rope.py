"""Rotary position encoding with the reference's frequency schedules.

``freqs[i] = theta ** (2i / rotary_dim)`` in float32, then the llama3 or linear
rescaling (src/model/decoder_model.cpp:44-49, :65-70, :116-146); an angle is
``position / freqs[i]`` and pairs are half-split, ``(i, i + rotary_dim/2)``
(``traditional=false``, :220-228).  Keys are cached after rotation, values are
never rotated (:255-258).  The kernel that rotates also writes keys and values
into their pages, so the encoding owns that step of the mixer.

``"none"`` is the encoding without positions: the same kernel with nothing
rotated.

``"rotary"`` is the plain rotation with its constants as parameters: ``base``, how many leading
channels of a head rotate (``rotary_dim``) and the pairing (``"half"``: channel i with
i + rotary_dim/2; ``"pairs"``: channel 2i with 2i + 1).  Pair i turns by
``position * base^(-2i/rotary_dim)``; the angle is a 32-bit product on the bfloat16 path and a
double one on the 32-bit path.  It can also fill the value pages with the keys as they were
before the rotation, for mixers whose values are their keys.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..config.model_config import RopeScaling, validate_rope_scaling
from ..csrc import ops
from .base import PositionEncoding, register_position

_TWO_PI = np.float32(6.283185307179586)   # src/model/decoder_model.cpp:21


def rope_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    """float32 [rotary_dim/2], computed in float32 as the reference does."""
    if rotary_dim <= 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
    idx = np.arange(0, rotary_dim, 2, dtype=np.float32)
    freqs = np.power(np.float32(theta), idx / np.float32(rotary_dim)).astype(np.float32)
    if scaling is None:
        return freqs
    rs = scaling if isinstance(scaling, RopeScaling) else RopeScaling.from_json(scaling)
    validate_rope_scaling(rs)
    if rs.rope_type == "default":
        return freqs
    factor = np.float32(rs.factor)
    if rs.rope_type == "linear":
        return (freqs * factor).astype(np.float32)
    low_ff, high_ff = np.float32(rs.low_freq_factor), np.float32(rs.high_freq_factor)
    old_ctx = np.float32(rs.original_max_position_embeddings)
    low_wl, high_wl = old_ctx / low_ff, old_ctx / high_ff
    wavelens = (_TWO_PI * freqs).astype(np.float32)
    scaled = np.where(wavelens > low_wl, freqs * factor, freqs).astype(np.float32)
    medium = (wavelens > high_wl) & (wavelens < low_wl)      # strict on both sides
    smooth = ((old_ctx / wavelens - low_ff) / (high_ff - low_ff)).astype(np.float32)
    denom = ((np.float32(1.0) - smooth) / factor + smooth).astype(np.float32)
    return np.where(medium, (scaled / denom).astype(np.float32), scaled).astype(np.float32)


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        self.freqs_host = rope_frequencies(self.rotary_dim, float(params["theta"]), params.get("scaling"))
        self.freqs = torch.from_numpy(self.freqs_host).to(runtime.device)

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache):
        ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, batch.block_table(lane.group),
                          lane.page_size, self.freqs, q_out, lane.k, lane.v, n_heads, n_kv_heads,
                          self.head_dim, self.rotary_dim, writes_cache, self.rt.precise)


@register_position("none")
class NoPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache):
        ops.rope_kv_write(qkv, batch.positions, batch.seq_of_token, batch.block_table(lane.group),
                          lane.page_size, None, q_out, lane.k, lane.v, n_heads, n_kv_heads,
                          self.head_dim, 0, writes_cache, self.rt.precise)


def inverse_wavelengths(rotary_dim: int, base: float, device):
    """``base^(-2i/rotary_dim)``, i < rotary_dim/2, worked out in double: (float32 tensor, float64 tensor)."""
    if rotary_dim < 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be even and not negative, got {rotary_dim}")
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    inv = np.power(float(base), -2.0 * i / max(rotary_dim, 1))
    return (torch.from_numpy(inv.astype(np.float32)).to(device), torch.from_numpy(inv).to(device))


def stretched_inverse_wavelengths(rotary_dim: int, base: float, scaling, device):
    """Inverse wavelengths of a rotation whose slow pairs are stretched for contexts longer than the ones
    trained on (the YaRN schedule), and the factor that goes with it on cosine and sine:
    (float32 tensor, float64 tensor, factor).

    ``scaling`` has ``factor``, ``original`` (the trained context), ``fast`` and ``slow`` (turns over that
    context).  With ``w_i = base^(-2i/dims)`` and ``p(t) = dims ln(original / (2 pi t)) / (2 ln base)`` the
    pair index at which a pair makes ``t`` turns over the trained context: pairs up to
    ``lo = max(floor(p(fast)), 0)`` keep ``w_i``, pairs from ``hi = min(ceil(p(slow)), dims - 1)`` on get
    ``w_i / factor``, and between them the two are blended linearly in the pair index (a ramp over
    ``max(hi - lo, 0.001)``).  Cosine and sine are multiplied by ``0.1 ln(factor) + 1``.  ``scaling`` None:
    the plain table and 1.  Worked out in double."""
    if rotary_dim < 0 or rotary_dim % 2:
        raise ValueError(f"rotary_dim must be even and not negative, got {rotary_dim}")
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    inv = np.power(float(base), -2.0 * i / max(rotary_dim, 1))
    magnitude = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])
        fast, slow = float(scaling["fast"]), float(scaling["slow"])
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and base > 1):
            raise ValueError("stretched rotation: factor, original, fast and slow must be positive, base above 1")

        def pair_of(turns: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), rotary_dim - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        inv = inv / factor * ramp + inv * (1.0 - ramp)
        magnitude = 0.1 * math.log(factor) + 1.0
    return (torch.from_numpy(inv.astype(np.float32)).to(device), torch.from_numpy(inv).to(device), magnitude)


@register_position("rotary")
class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.pairing = str(params.get("pairing", "half"))
        if self.pairing not in ("half", "pairs"):
            raise ValueError(f"rotary: pairing must be 'half' or 'pairs', got '{self.pairing}'")
        if self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        self.inv_f, inv_d = inverse_wavelengths(self.rotary_dim, float(params["base"]), runtime.device)
        self.inv_d = inv_d if runtime.precise else None      # the 32-bit path takes its angles in double

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache, values_from_keys=False,
                         ld=None):
        """``values_from_keys``: the rows hold queries and keys only, and the value pages get the keys as
        projected.  ``ld``: elements between rows of ``qkv`` (it may hold further columns behind the heads)."""
        ops.rope_store(qkv, batch.positions, batch.seq_of_token, batch.block_table(lane.group), lane.page_size,
                       self.inv_f, self.inv_d, q_out, lane.k, lane.v, n_heads, n_kv_heads, self.head_dim,
                       self.rotary_dim, self.pairing == "pairs", writes_cache, values_from_keys, ld)
