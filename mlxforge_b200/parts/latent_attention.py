"""Attention over a compressed latent: every token keeps one normed latent vector ``c`` [kv_rank]
and one rotated key part ``r`` [rot_dim] that all heads share, instead of keys and values per head.

    c_q = rmsnorm(W_dq x) ;  q_h = (n_h | p_h) = rows of W_uq c_q, ``dim`` plain and ``rot_dim`` rotated
        (``q_rank`` 0: no query latent, q_h = rows of W_q x)
    (c' | r') = W_dkv x ;    c = rmsnorm(c') ;  r = rotate(r')         (kept in the cache, per token)
    k_h = (W_uk,h c | r) ;   v_h = W_uv,h c
    s_h = (n_h . W_uk,h c + rotate(p_h) . r) * softmax_scale ;  causal softmax ;  o_h = sum_j p_j v_h,j
    out = W_o (concat_h(o_h) * sigmoid(W_g x))

The engine never expands keys or values: ``n_h . (W_uk,h c) = (W_uk,h^T n_h) . c``, so the query of a
head becomes ``(W_uk,h^T n_h | rotate(p_h))``, ``kv_rank + rot_dim`` wide, the cached rows are its
keys, their first ``kv_rank`` channels its values (one key head shared by all query heads, no value
pool), and ``W_uv,h`` is applied to the attended latent.  A layer with ``shares_cache`` has no
``W_dkv``: it reads the lane of the layer it names in the schedule and writes nothing.

Options, all parameters: ``window`` > 0 (query i sees key j iff ``0 <= i - j < window``); ``pairing`` of the
rotation (``"half"``: channel i with i + dims/2; ``"pairs"``: channel 2i with 2i + 1) over the first
``rot_dims`` channels of the rotated part; ``rope_scaling`` (a stretched frequency table with its factor on
cosine and sine, see ``rope.stretched_inverse_wavelengths``; the softmax scale is used as given); the
gate as one number per output channel (``W_g`` [heads * v_head_dim, H]) or, with ``gate_per_head``, one
per head (``W_g`` [heads, H]).  Norms, angles, scores and the softmax are 32-bit.  ``names`` maps the
tensors' roles to their names behind the prefix.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Mixer, PagedKV, TensorSpec, register_mixer
from .rope import stretched_inverse_wavelengths

_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
          "uv": "uv", "g": "g", "o": "o"}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["head_dim"])
        self.rot = int(p["rot_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.q_rank = int(p.get("q_rank") or 0)          # 0: the queries are projected from the input directly
        self.rank = int(p["kv_rank"])
        self.scale = float(p["softmax_scale"])
        self.eps = float(p["eps"])
        self.has_gate = bool(p.get("gate", True))
        self.gate_per_head = bool(p.get("gate_per_head", False))
        self.shares_cache = bool(p.get("shares_cache", False))
        self.window = int(p.get("window", 0) or 0)
        self.pairing = str(p.get("pairing", "half"))
        self.rot_dims = int(p["rot_dims"]) if p.get("rot_dims") is not None else self.rot
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if self.pairing not in ("half", "pairs"):
            raise ValueError(f"latent_attention: pairing must be 'half' or 'pairs', got '{self.pairing}'")
        if self.rot_dims % 2 or not (0 <= self.rot_dims <= self.rot):
            raise ValueError(f"latent_attention: rot_dims must be even and at most rot_dim, got {self.rot_dims}")
        if min(self.n_heads, self.dim, self.vdim, self.rank) <= 0 or self.rot < 0 or self.q_rank < 0 or self.window < 0:
            raise ValueError("latent_attention: sizes must be positive")
        self.inv_f, inv_d, self.magnitude = stretched_inverse_wavelengths(
            self.rot_dims, float(p.get("rope_base", 10000.0)), p.get("rope_scaling"), runtime.device)
        self.inv_d = inv_d if runtime.precise else None
        self.w_in = self.w_uq = self.w_ukT = self.w_uv = self.w_o = self.q_norm = self.kv_norm = None
        self.kv_off = self.g_off = 0

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    @property
    def kv_width(self) -> int:
        return self.rank + self.rot

    @property
    def gate_rows(self) -> int:
        return self.n_heads if self.gate_per_head else self.n_heads * self.vdim

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        H, nh = self.hidden, self.n_heads
        specs = {
            self._n("uk"): TensorSpec((nh * self.dim, self.rank)),
            self._n("uv"): TensorSpec((nh * self.vdim, self.rank)),
            self._n("o"): TensorSpec((H, nh * self.vdim)),
        }
        if self.q_rank:
            specs[self._n("dq")] = TensorSpec((self.q_rank, H))
            specs[self._n("dq_norm")] = TensorSpec((self.q_rank,), role="vector")
            specs[self._n("uq")] = TensorSpec((nh * (self.dim + self.rot), self.q_rank))
        else:
            specs[self._n("q")] = TensorSpec((nh * (self.dim + self.rot), H))
        if not self.shares_cache:
            specs[self._n("dkv")] = TensorSpec((self.kv_width, H))
            specs[self._n("dkv_norm")] = TensorSpec((self.rank,), role="vector")
        if self.has_gate:
            specs[self._n("g")] = TensorSpec((self.gate_rows, H))
        return specs

    def bind(self, tensors) -> None:
        dt, f32 = self.rt.dtype, torch.float32
        # every projection of the input is one product: [queries or their latent | key/value latent and the
        # shared key part | gate], padded with zero rows to whole 16-byte rows of bfloat16 output
        roles = ("dq" if self.q_rank else "q",) + (() if self.shares_cache else ("dkv",)) + (("g",) if self.has_gate else ())
        blocks = [tensors[self._n(r)].to(dt) for r in roles]
        rows = [b.shape[0] for b in blocks]
        self.kv_off = rows[0]
        self.g_off = sum(rows) - (rows[-1] if self.has_gate else 0)
        pad = -sum(rows) % 8
        if pad:
            blocks.append(torch.zeros((pad, self.hidden), dtype=dt, device=blocks[0].device))
        self.w_in = torch.cat(blocks, dim=0).contiguous()
        if self.q_rank:
            self.w_uq = tensors[self._n("uq")].to(dt).contiguous()
            self.q_norm = tensors[self._n("dq_norm")].to(f32).contiguous()
        # [heads, kv_rank, dim]: head h's key expansion, transposed, so that it maps a query to the latent
        self.w_ukT = tensors[self._n("uk")].to(dt).view(self.n_heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[self._n("uv")].to(dt).view(self.n_heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        if not self.shares_cache:
            self.kv_norm = tensors[self._n("dkv_norm")].to(f32).contiguous()

    def weight_bytes(self) -> int:
        ws = [w for w in (self.w_in, self.w_uq, self.w_ukT, self.w_uv, self.w_o) if w is not None]
        return sum(w.numel() for w in ws) * self.w_in.element_size()

    def cache_need(self):
        return PagedKV(1, self.kv_width, window=self.window, v_head_dim=self.rank, values_in_keys=True)

    def attend(self, q_full, batch, cache, out):
        latent_paged_attention(self.rt, batch, q_full, cache, out, self)

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T, nh = self.rt, x.shape[0], self.n_heads
        qw = self.dim + self.rot
        pairs = self.pairing == "pairs"
        proj = rt.linear(x, self.w_in, rt.buffer("lat.in", (T, self.w_in.shape[0])))
        cq = rt.buffer("lat.cq", (T, self.q_rank)) if self.q_rank else None
        ops.latent_prepare(proj, self.q_rank, self.kv_off, self.rank, self.rot, self.q_norm, self.kv_norm, self.eps,
                           batch.positions, batch.seq_of_token, batch.block_table(cache.group), cache.page_size,
                           self.inv_f, self.inv_d, cq, cache.k, writes_cache and not self.shares_cache, pairs,
                           self.rot_dims, self.magnitude)
        if self.q_rank:
            q, q_ld = rt.linear(cq, self.w_uq, rt.buffer("lat.q", (T, nh * qw))), nh * qw
        else:
            q, q_ld = proj, proj.shape[1]          # the queries are the first columns of the input's product
        q_full = rt.buffer("lat.q_full", (T, nh * self.kv_width))
        rt.head_linear(q, q_ld, qw, self.w_ukT, q_full, nh * self.kv_width, self.kv_width, T)
        ops.latent_query(q, nh, self.dim, self.rot, self.rank, batch.positions, self.inv_f, self.inv_d, q_full, q_ld,
                         pairs, self.rot_dims, self.magnitude)
        o_lat = rt.buffer("lat.o_lat", (T, nh * self.rank))
        self.attend(q_full, batch, cache, o_lat)
        o = rt.buffer("lat.o", (T, nh * self.vdim))
        gate = proj[:, self.g_off:] if self.has_gate else None
        rt.head_linear(o_lat, nh * self.rank, self.rank, self.w_uv, o, nh * self.vdim, self.vdim, T, gate,
                       proj.shape[1], self.gate_per_head)
        return rt.linear(o, self.w_o, rt.buffer("lat.delta", (T, self.hidden)))


def latent_paged_attention(rt, batch, q, lane, out, m: LatentAttention) -> None:
    """Causal attention (within the mixer's window, if it has one) of queries ``kv_rank + rot_dim`` wide over
    the lane's one key head, the values being the keys' first ``kv_rank`` channels: the attention kernels'
    option ``values_in_keys``."""
    from .attention import options_paged_attention
    options_paged_attention(rt, batch, q, lane, out, m.n_heads, m.scale, m.window)
