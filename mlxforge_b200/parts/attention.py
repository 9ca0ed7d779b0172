"""Grouped-query attention over the paged cache.

``q = x Wq^T, k = x Wk^T, v = x Wv^T`` (weights ``(out, in)``, no bias; head ``h``
is output rows ``[h*hd, (h+1)*hd)``), position encoding on q and k, keys and
values appended to the cache, ``softmax(q k^T * scale) v`` with the causal mask
aligned to the end of the keys, query head ``h`` reading KV head
``h // (n_heads / n_kv_heads)``, then the output projection
(src/model/decoder_model.cpp:234-275, :315-328; src/model/sdpa.cpp:27,44-46,71-95).
The three projections are one matrix here (stacked at load time), which changes
no number.  ``window`` > 0 limits every query to the last ``window`` keys.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import POSITIONS, Mixer, PagedKV, PartSpec, TensorSpec, build_part, register_mixer


def paged_attention(rt, batch, q, lane, out, n_heads: int, scale: float, window: int) -> None:
    """Attention of the step's queries over ``lane``; the kernel is chosen by dtype and by how
    many tokens each sequence brings.  bfloat16: the sequences that bring one token (the batch
    lays them out first: ``batch.n_decode``) go to the split-key decode kernel, the others to the
    prefill kernel.  float32: the generic kernel for all."""
    need = lane.need
    table = batch.block_table(lane.group)
    nd = batch.n_decode if q.dtype == torch.bfloat16 else 0
    if nd > 0:
        # contexts of very unequal length (the host knows them, the launcher does not): said to the
        # kernel's launcher, which then avoids dealing many items of unequal size out in turn
        lens = batch.ctx_len[:nd]
        unequal = nd >= 8 and max(lens) * nd > 1.3 * sum(lens)
        n_o, n_ml = ops.attention_decode_scratch(nd, n_heads, need.head_dim, batch.max_ctx)
        ops.attention_decode(q[:nd], lane.k, lane.v, out[:nd],
                             rt.buffer("attn.part_o", (n_o,), torch.float32),
                             rt.buffer("attn.part_ml", (n_ml,), torch.float32),
                             batch.positions[:nd], batch.seq_of_token[:nd], table, lane.page_size, n_heads,
                             need.n_kv_heads, need.head_dim, scale, window, batch.max_ctx, unequal)
    if nd < batch.n_tokens and q.dtype == torch.bfloat16:
        ops.attention_prefill(q, lane.k, lane.v, out, batch.seq_q_start[nd:], batch.seq_q_len[nd:],
                              batch.seq_ctx_len[nd:], nd, max(batch.q_len[nd:]), table, lane.page_size,
                              n_heads, need.n_kv_heads, need.head_dim, scale, window)
    elif nd < batch.n_tokens:
        ops.attention_generic(q[nd:], lane.k, lane.v, out[nd:], batch.positions[nd:],
                              batch.seq_of_token[nd:], table, lane.page_size, n_heads, need.n_kv_heads,
                              need.head_dim, scale, window)


@register_mixer("attention")
class AttentionMixer(Mixer):
    """``forward`` is four steps, each a method of its own, so that a variant (a norm on queries
    and keys, a gate on the output, another kernel) overrides one step and keeps the rest."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.scale = float(p["softmax_scale"])
        self.window = int(p.get("window", 0) or 0)
        if self.n_heads % self.n_kv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.hd % 16 or not (16 <= self.hd <= 256):
            raise ValueError(f"attention: head_dim {self.hd} is not a multiple of 16 in [16, 256]")
        self.position = build_part(POSITIONS, p["position"], runtime)
        self.w_qkv = None
        self.w_o = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, kv = self.n_heads * self.hd, self.n_kv * self.hd
        specs = {
            self.prefix + "q_proj.weight": TensorSpec((q, self.hidden)),
            self.prefix + "k_proj.weight": TensorSpec((kv, self.hidden)),
            self.prefix + "v_proj.weight": TensorSpec((kv, self.hidden)),
            self.prefix + "o_proj.weight": TensorSpec((self.hidden, q)),
        }
        specs.update(self.position.tensor_specs())      # a position encoding may have tensors of its own
        return specs

    def bind(self, tensors) -> None:
        self.position.bind(tensors)
        dt = self.rt.dtype
        self.w_qkv = torch.cat([tensors[self.prefix + n + "_proj.weight"].to(dt) for n in ("q", "k", "v")],
                               dim=0).contiguous()
        self.w_o = tensors[self.prefix + "o_proj.weight"].to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_need(self):
        return PagedKV(self.n_kv, self.hd, self.window)

    def project(self, x):
        """[T, H] -> queries, keys and values side by side, [T, (n_heads + 2 n_kv) * head_dim]."""
        T = x.shape[0]
        return self.rt.linear(x, self.w_qkv, self.rt.buffer("attn.qkv", (T, (self.n_heads + 2 * self.n_kv) * self.hd)))

    def encode_and_store(self, qkv, batch, cache, writes_cache: bool):
        """Position-encode queries and keys, append keys and values to the cache; returns the queries."""
        q = self.rt.buffer("attn.q", (qkv.shape[0], self.n_heads * self.hd))
        self.position.rotate_and_store(qkv, batch, q, cache, self.n_heads, self.n_kv, writes_cache)
        return q

    def attend(self, q, batch, cache):
        o = self.rt.buffer("attn.o", (q.shape[0], self.n_heads * self.hd))
        paged_attention(self.rt, batch, q, cache, o, self.n_heads, self.scale, self.window)
        return o

    def output(self, o):
        return self.rt.linear(o, self.w_o, self.rt.buffer("attn.delta", (o.shape[0], self.hidden)))

    def forward(self, x, batch, cache, writes_cache: bool = True):
        qkv = self.project(x)
        q = self.encode_and_store(qkv, batch, cache, writes_cache)
        return self.output(self.attend(q, batch, cache))


def options_paged_attention(rt, batch, q, lane, out, n_heads: int, scale: float, window: int = 0, keep_first: int = 0,
                            sink=None, gate=None, gate_ld: int = 0) -> None:
    """Attention over ``lane`` with the options beyond a window: values of their own width or inside the
    keys (the lane's need says which), kept first keys, a sink, a gate on the output.  bfloat16 with sizes
    the tensor-core kernels take: the sequences that bring one token (the batch lays them out first) go to
    the split-key decode kernel, portions of prompts to the prefill kernel; the 32-bit path and other sizes
    take the block-per-token kernel."""
    need = lane.need
    table = batch.block_table(lane.group)
    vd, in_k = need.value_dim, need.values_in_keys
    if q.dtype != torch.bfloat16 or not ops.attention_tc_ok(need.head_dim, vd, lane.page_size):
        ops.attention_generic_ex(q, lane.k, lane.v, out, batch.positions, batch.seq_of_token, table, lane.page_size,
                                 n_heads, need.n_kv_heads, need.head_dim, scale, window, vd,
                                 need.head_dim if in_k else vd, keep_first, sink, gate, gate_ld)
        return
    nd = batch.n_decode
    if nd > 0:
        n_o, n_ml = ops.attention_decode_scratch(nd, n_heads, need.head_dim, batch.max_ctx, window)
        ops.attention_decode_ex(q[:nd], lane.k, lane.v, out[:nd], rt.buffer("attn.part_o", (n_o,), torch.float32),
                                rt.buffer("attn.part_ml", (n_ml,), torch.float32), batch.positions[:nd],
                                batch.seq_of_token[:nd], table, lane.page_size, n_heads, need.n_kv_heads,
                                need.head_dim, scale, window, batch.max_ctx, vd, in_k, keep_first, sink, gate, gate_ld)
    if nd < batch.n_tokens:
        ops.attention_prefill_ex(q, lane.k, lane.v, out, batch.seq_q_start[nd:], batch.seq_q_len[nd:],
                                 batch.seq_ctx_len[nd:], nd, max(batch.q_len[nd:]), table, lane.page_size, n_heads,
                                 need.n_kv_heads, need.head_dim, scale, window, vd, in_k, keep_first, sink, gate,
                                 gate_ld)


_SINK_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "sink": "sink"}


@register_mixer("sink_attention")
class SinkAttention(AttentionMixer):
    """Grouped-query attention with four options, each a parameter:

    * ``values``: ``"keys"`` — there is no value projection; the values are the keys as projected,
      before the rotation (the value pages are filled beside the key pages) — or ``"own"``;
    * ``window`` with ``keep_first``: query i sees key j if ``j <= i`` and (``i - j < window`` or
      ``j < keep_first``); the kept keys stay at their own positions;
    * ``sink``: a learned number per query head whose exponential joins the softmax denominator; it has
      no key and no value and is not scaled;
    * ``gate``: the concatenated heads are multiplied by ``sigmoid(Wg x)`` before the output projection.

    All projections that read the mixer's input are one product.  ``names`` maps the tensors' roles to
    their names behind the prefix."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        p = dict(params)
        p.setdefault("position", PartSpec("none", {"head_dim": int(p["head_dim"])}))
        Mixer.__init__(self, p, prefix, runtime)
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.scale = float(p["softmax_scale"])
        self.window = int(p.get("window", 0) or 0)
        self.keep_first = int(p.get("keep_first", 0) or 0) if self.window else 0
        self.values = str(p.get("values", "own"))
        self.has_sink = bool(p.get("sink", False))
        self.has_gate = bool(p.get("gate", False))
        self.names = dict(_SINK_NAMES, **(p.get("names") or {}))
        if self.values not in ("own", "keys"):
            raise ValueError(f"sink_attention: values must be 'own' or 'keys', got '{self.values}'")
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.window < 0 or self.keep_first < 0:
            raise ValueError("sink_attention: window and keep_first must not be negative")
        self.position = build_part(POSITIONS, p["position"], runtime)
        self.w_in = self.w_o = self.sink = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def _roles(self):
        return ("q", "k") + (("v",) if self.values == "own" else ()) + (("g",) if self.has_gate else ())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        q, kv = self.n_heads * self.hd, self.n_kv * self.hd
        rows = {"q": q, "k": kv, "v": kv, "g": q}
        specs = {self._n(r): TensorSpec((rows[r], self.hidden)) for r in self._roles()}
        specs[self._n("o")] = TensorSpec((self.hidden, q))
        if self.has_sink:
            specs[self._n("sink")] = TensorSpec((self.n_heads,), role="vector")
        specs.update(self.position.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        self.position.bind(tensors)
        dt = self.rt.dtype
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in self._roles()], dim=0).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        if self.has_sink:
            self.sink = tensors[self._n("sink")].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return PagedKV(self.n_kv, self.hd, self.window, keep_first=self.keep_first)

    def project(self, x):
        """[T, H] -> queries, keys, (values,) (gates) side by side."""
        return self.rt.linear(x, self.w_in, self.rt.buffer("sattn.in", (x.shape[0], self.w_in.shape[0])))

    def encode_and_store(self, proj, batch, cache, writes_cache: bool):
        q = self.rt.buffer("sattn.q", (proj.shape[0], self.n_heads * self.hd))
        self.position.rotate_and_store(proj, batch, q, cache, self.n_heads, self.n_kv, writes_cache,
                                       values_from_keys=self.values == "keys", ld=proj.shape[1])
        return q

    def forward(self, x, batch, cache, writes_cache: bool = True):
        proj = self.project(x)
        q = self.encode_and_store(proj, batch, cache, writes_cache)
        o = self.rt.buffer("sattn.o", (q.shape[0], self.n_heads * self.hd))
        gate = proj[:, proj.shape[1] - self.n_heads * self.hd:] if self.has_gate else None
        options_paged_attention(self.rt, batch, q, cache, o, self.n_heads, self.scale, self.window, self.keep_first,
                                self.sink, gate, proj.shape[1])
        return self.rt.linear(o, self.w_o, self.rt.buffer("sattn.delta", (o.shape[0], self.hidden)))


_NORMED_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "q_norm": "q.norm",
                 "k_norm": "k.norm"}


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    """Grouped-query attention whose queries and keys are normalised over their WHOLE projections (one root
    mean square over all heads' rows of q, one over k's, each with a plain weight of that size) before they
    are rotated.  Every option is a parameter:

    * ``bias``: q and k projections have biases (added in 32-bit before the norm);
    * ``qk_norm``: ``"whole"`` or None;
    * ``rotary``: ``{"dims", "base", "scaling"}`` - half-split pairs over the first ``dims`` channels of a head;
      ``scaling`` None, ``{"factor"}`` (every frequency divided by it) or ``{"factor", "original", "fast",
      "slow"}`` (the stretched table, cosine and sine times ``0.1 ln(factor) + 1``);
    * ``values``: ``"own"`` (a value projection, ``v_head_dim`` wide per head) or ``"keys"`` (the keys as
      projected, with their bias, before norm and rotation);
    * ``rotate_values``: the value of position j is turned by j over all its channels (half-split pairs, pair m
      by ``j * base^(-2m/v_head_dim)``, no scaling) before it is cached, and a head's output at position i is
      turned back by i;
    * ``softmax_scale``, ``softcap`` (``cap * tanh(score / cap)``), ``window`` (0: causal);
    * ``out_f32``: the output projection is written in 32-bit."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.scale = float(p["softmax_scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = int(p.get("window", 0) or 0)
        self.values = str(p.get("values", "own"))
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.eps = float(p.get("eps", 1e-6))
        self.rotate_values = bool(p.get("rotate_values", False))
        self.out_f32 = bool(p.get("out_f32", False))
        self.names = dict(_NORMED_NAMES, **(p.get("names") or {}))
        if self.values not in ("own", "keys"):
            raise ValueError(f"normed_attention: values must be 'own' or 'keys', got '{self.values}'")
        if self.qk_norm not in (None, "whole"):
            raise ValueError(f"normed_attention: qk_norm must be 'whole' or None, got '{self.qk_norm}'")
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.values == "keys" and self.vd != self.hd:
            raise ValueError("normed_attention: values that are the keys have the keys' size")
        if self.rotate_values and self.vd % 2:
            raise ValueError("normed_attention: rotated values need an even v_head_dim")
        from .rope import inverse_wavelengths, stretched_inverse_wavelengths
        rot = p.get("rotary") or {}
        self.rot = int(rot.get("dims", 0) or 0)
        if self.rot % 2 or self.rot > self.hd:
            raise ValueError(f"normed_attention: rotary dims {self.rot} must be even and at most head_dim")
        base, sc = float(rot.get("base", 10000.0)), rot.get("scaling") or None
        self.magnitude = 1.0
        if sc and "original" in sc:
            inv_f, inv_d, self.magnitude = stretched_inverse_wavelengths(self.rot, base, sc, runtime.device)
        else:
            inv_f, inv_d = inverse_wavelengths(self.rot, base, runtime.device)
            if sc:
                inv_d = inv_d / float(sc["factor"])
                inv_f = inv_d.to(torch.float32)
        self.inv_f, self.inv_d = inv_f, (inv_d if runtime.precise else None)
        self.vinv_f = self.vinv_d = None
        if self.rotate_values:
            vf, vd = inverse_wavelengths(self.vd, base, runtime.device)
            self.vinv_f, self.vinv_d = vf, (vd if runtime.precise else None)
        self.w_in = self.w_o = self.b_in = self.q_w = self.k_w = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def _roles(self):
        return ("q", "k") + (("v",) if self.values == "own" else ())

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nq, nk, nv = self.n_heads * self.hd, self.n_kv * self.hd, self.n_kv * self.vd
        rows = {"q": nq, "k": nk, "v": nv}
        specs = {self._n(r): TensorSpec((rows[r], self.hidden)) for r in self._roles()}
        specs[self._n("o")] = TensorSpec((self.hidden, self.n_heads * self.vd))
        if self.bias:
            specs[self._n("q_bias")] = TensorSpec((nq,), role="vector")
            specs[self._n("k_bias")] = TensorSpec((nk,), role="vector")
        if self.qk_norm:
            specs[self._n("q_norm")] = TensorSpec((nq,), role="vector")
            specs[self._n("k_norm")] = TensorSpec((nk,), role="vector")
        return specs

    def bind(self, tensors) -> None:
        dt, f32 = self.rt.dtype, torch.float32
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in self._roles()], dim=0).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        if self.bias:
            b = [tensors[self._n("q_bias")].to(f32), tensors[self._n("k_bias")].to(f32)]
            if self.values == "own":
                b.append(torch.zeros(self.n_kv * self.vd, dtype=f32, device=b[0].device))
            self.b_in = torch.cat(b).contiguous()
        if self.qk_norm:
            self.q_w = tensors[self._n("q_norm")].to(f32).contiguous()
            self.k_w = tensors[self._n("k_norm")].to(f32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return PagedKV(self.n_kv, self.hd, self.window, v_head_dim=0 if self.vd == self.hd else self.vd)

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T = self.rt, x.shape[0]
        # the projections feed 32-bit norms: they are written in 32-bit and rounded once, after norm and rotation
        proj = rt.linear(x, self.w_in, rt.buffer("nattn.in", (T, self.w_in.shape[0]), torch.float32))
        q = rt.buffer("nattn.q", (T, self.n_heads * self.hd))
        table = batch.block_table(cache.group)
        ops.qk_norm_rope(proj, self.n_heads, self.n_kv, self.hd, self.vd, self.rot, self.values == "keys", self.eps,
                         self.magnitude, self.b_in, self.q_w, self.k_w, self.inv_f, self.inv_d, self.vinv_f, self.vinv_d,
                         batch, table, cache.page_size, q, cache.k, cache.v, writes_cache)
        o = rt.buffer("nattn.o", (T, self.n_heads * self.vd))
        softcap_attention(rt, batch, q, cache, o, self.n_heads, self.scale, self.window, self.softcap)
        if self.rotate_values:
            ops.rotate_rows(o, self.n_heads, self.vd, self.vd, batch.positions, self.vinv_f, self.vinv_d, -1.0)
        return rt.linear(o, self.w_o, rt.buffer("nattn.delta", (T, self.hidden), torch.float32 if self.out_f32 else None))


def softcap_attention(rt, batch, q, lane, out, n_heads: int, scale: float, window: int, softcap: float) -> None:
    """Attention over ``lane`` (values of their own width in a pool of their own) with a window and a soft cap
    on the scaled scores; kernels chosen as in ``options_paged_attention``."""
    need = lane.need
    table = batch.block_table(lane.group)
    vd = need.value_dim
    if q.dtype != torch.bfloat16 or not ops.attention_tc_ok(need.head_dim, vd, lane.page_size):
        ops.attention_generic_ex(q, lane.k, lane.v, out, batch.positions, batch.seq_of_token, table, lane.page_size,
                                 n_heads, need.n_kv_heads, need.head_dim, scale, window, vd, vd, 0, None, None, 0,
                                 softcap)
        return
    nd = batch.n_decode
    if nd > 0:
        n_o, n_ml = ops.attention_decode_scratch(nd, n_heads, need.head_dim, batch.max_ctx, window)
        ops.attention_decode_ex(q[:nd], lane.k, lane.v, out[:nd], rt.buffer("attn.part_o", (n_o,), torch.float32),
                                rt.buffer("attn.part_ml", (n_ml,), torch.float32), batch.positions[:nd],
                                batch.seq_of_token[:nd], table, lane.page_size, n_heads, need.n_kv_heads,
                                need.head_dim, scale, window, batch.max_ctx, vd, False, 0, None, None, 0, softcap)
    if nd < batch.n_tokens:
        ops.attention_prefill_ex(q, lane.k, lane.v, out, batch.seq_q_start[nd:], batch.seq_q_len[nd:],
                                 batch.seq_ctx_len[nd:], nd, max(batch.q_len[nd:]), table, lane.page_size, n_heads,
                                 need.n_kv_heads, need.head_dim, scale, window, vd, False, 0, None, None, 0, softcap)
