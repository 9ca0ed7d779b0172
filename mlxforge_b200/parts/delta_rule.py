"""Gated delta rule with a decay per head and key channel ("channel delta"), a recurrent mixer.

Per head, with a 32-bit state ``S`` [head_dim, v_head_dim] per request, token after token:

    S <- diag(g_t) S ;   u = beta_t (v_t - S^T k_t) ;   S <- S + k_t u^T ;   o_t = S^T q_t

``q, k`` (``n_kv_heads`` heads) and ``v`` (``n_heads`` heads) are projections of the input, each
through a short causal convolution over time per channel (``conv`` taps, the last one the current
token's, zeros before the start) and SiLU; ``q`` and ``k`` are made unit vectors per head
(``x / sqrt(sum x^2 + 1e-6)``), ``q`` also times ``head_dim^-1/2``; head ``h`` uses q/k head
``h // (n_heads / n_kv_heads)``.  ``beta = sigmoid(Wb x)`` per head;
``g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 x) + dt_bias))`` per head and key channel.  The read-out of
every head is divided by its root mean square over ``v_head_dim`` (``eps``), multiplied by a weight
shared by the heads and by ``sigmoid(Wg2 (Wg1 x))``, then projected by ``Wo``.

Options: ``decay_rank`` 0 makes the decay's logit a direct projection ``Wa x`` (tensor role ``a``), and with
``decay_per_head`` it is one number per head that all its key channels share (``dt_bias`` then has one entry
per head); ``gate_rank`` 0 makes the gate a direct projection ``Wg x`` (role ``g``); ``gate_act`` is
``"sigmoid"`` or ``"silu"``; ``out_f32`` writes the output projection in 32-bit.

``generalized_delta`` (below) is the rule with a removal term beside the decay.

The request's slot keeps ``S`` of every head and the last ``conv - 1`` inputs of every convolution,
so a step goes on from where the step before ended, however the prompt was cut.  All projections
that read the mixer's input are one product; the two low-rank second factors are one product with a
block-diagonal matrix.  Everything after the projections is 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FixedState, Mixer, TensorSpec, register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "beta": "b", "A_log": "A_log", "dt_bias": "dt_bias",
          "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2", "a": "a", "g": "g", "norm": "norm", "o": "o"}


@register_mixer("channel_delta")
class ChannelDeltaMixer(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.decay_rank = int(p.get("decay_rank") or 0)
        self.gate_rank = int(p.get("gate_rank") or 0)
        self.decay_per_head = bool(p.get("decay_per_head", False))
        self.gate_act = str(p.get("gate_act", "sigmoid"))
        self.out_f32 = bool(p.get("out_f32", False))
        if self.decay_per_head and self.decay_rank:
            raise ValueError("channel_delta: one decay per head is a direct projection (decay_rank 0)")
        if self.gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"channel_delta: gate_act must be 'sigmoid' or 'silu', got '{self.gate_act}'")
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError("channel_delta: n_heads must be a multiple of n_kv_heads")
        if self.taps < 1:
            raise ValueError("channel_delta: conv must be at least 1 tap")
        if self.dim > 256:
            raise ValueError(f"channel_delta: head_dim {self.dim} is larger than the recurrence kernel's 256")
        self.channels = 2 * self.n_kv * self.dim + self.n_heads * self.vdim
        self.state_floats = self.n_heads * self.dim * self.vdim
        self.w_in = self.w_low = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nqk, nv, H = self.n_kv * self.dim, self.n_heads * self.vdim, self.hidden
        c = self.names["conv"]
        specs = {
            self._n("q"): TensorSpec((nqk, H)), self._n("k"): TensorSpec((nqk, H)), self._n("v"): TensorSpec((nv, H)),
            self._n("q") + c: TensorSpec((nqk, self.taps), role="vector"),
            self._n("k") + c: TensorSpec((nqk, self.taps), role="vector"),
            self._n("v") + c: TensorSpec((nv, self.taps), role="vector"),
            self._n("beta"): TensorSpec((self.n_heads, H)),
            self._n("A_log"): TensorSpec((self.n_heads,), role="vector"),
            self._n("dt_bias"): TensorSpec((self.n_decay_in,), role="vector"),
            self._n("norm"): TensorSpec((self.vdim,), role="vector"),
            self._n("o"): TensorSpec((H, nv)),
        }
        if self.decay_rank:
            specs[self._n("a1")] = TensorSpec((self.decay_rank, H))
            specs[self._n("a2")] = TensorSpec((self.n_heads * self.dim, self.decay_rank))
        else:
            specs[self._n("a")] = TensorSpec((self.n_decay_in, H))
        if self.gate_rank:
            specs[self._n("g1")] = TensorSpec((self.gate_rank, H))
            specs[self._n("g2")] = TensorSpec((nv, self.gate_rank))
        else:
            specs[self._n("g")] = TensorSpec((nv, H))
        return specs

    @property
    def n_decay_in(self) -> int:
        """Decay logits per token: one per head, or one per head and key channel."""
        return self.n_heads if self.decay_per_head else self.n_heads * self.dim

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        f32 = torch.float32
        c = self.names["conv"]
        # columns of the one input product: q | k | v | beta | low-rank first factors | direct decay | direct gate
        roles = ["q", "k", "v", "beta"] + (["a1"] if self.decay_rank else []) + (["g1"] if self.gate_rank else []) \
            + ([] if self.decay_rank else ["a"]) + ([] if self.gate_rank else ["g"])
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in roles], dim=0).contiguous()
        n_a2 = self.n_heads * self.dim if self.decay_rank else 0
        n_g2 = self.n_heads * self.vdim if self.gate_rank else 0
        if n_a2 + n_g2:
            low = torch.zeros((n_a2 + n_g2, self.decay_rank + self.gate_rank), dtype=dt, device=self.w_in.device)
            if n_a2:
                low[:n_a2, :self.decay_rank] = tensors[self._n("a2")].to(dt)
            if n_g2:
                low[n_a2:, self.decay_rank:] = tensors[self._n("g2")].to(dt)
            self.w_low = low.contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        self.conv_w = torch.cat([tensors[self._n(r) + c].to(f32) for r in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = tensors[self._n("A_log")].to(f32).contiguous()
        self.dt_bias = tensors[self._n("dt_bias")].to(f32).contiguous()
        self.norm_w = tensors[self._n("norm")].to(f32).contiguous()

    def weight_bytes(self) -> int:
        low = self.w_low.numel() if self.w_low is not None else 0
        return (self.w_in.numel() + low + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return FixedState((self.state_floats + (self.taps - 1) * self.channels,), tag="channel_delta")

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T = self.rt, x.shape[0]
        f32 = torch.float32
        nh, nkv, d, dv = self.n_heads, self.n_kv, self.dim, self.vdim
        state = cache.tensor                                       # [slots, S of every head | convolution tails]
        proj = rt.linear(x, self.w_in, rt.buffer("delta.proj", (T, self.w_in.shape[0]), f32))
        qkv = rt.buffer("delta.qkv", (T, self.channels), f32)
        beta = rt.buffer("delta.beta", (T, nh), f32)
        n_low = self.decay_rank + self.gate_rank
        low = rt.buffer("delta.low", (T, max(n_low, 1)))[:, :n_low]
        ops.delta_prepare(proj, self.conv_w, self.taps, state, self.state_floats, batch, qkv, beta, low, nh, nkv, d, dv)
        ag = rt.buffer("delta.ag", (T, nh * d + nh * dv), f32)
        if self.decay_rank and self.gate_rank and not self.decay_per_head and self.gate_act == "sigmoid":
            rt.linear(low, self.w_low, ag)
            ops.delta_gates(ag, self.a_log, self.dt_bias, nh, d, nh * dv)
        else:
            # logits of decays and gates from wherever they were projected: behind the low-rank second
            # factors, or columns of the input product
            second = rt.linear(low, self.w_low, rt.buffer("delta.low2", (T, self.w_low.shape[0]), f32)) if n_low else None
            direct = self.channels + nh + n_low
            if self.decay_rank:
                decay_in, decay_ld = second, second.shape[1]
            else:
                decay_in, decay_ld = proj[:, direct:], proj.shape[1]
            if self.gate_rank:
                gate_in, gate_ld = second[:, nh * d if self.decay_rank else 0:], second.shape[1]
            else:
                gate_in, gate_ld = proj[:, direct + (0 if self.decay_rank else self.n_decay_in):], proj.shape[1]
            ops.delta_gates_ex(decay_in, decay_ld, self.decay_per_head, 0, 0.0, self.a_log, self.dt_bias, gate_in, gate_ld,
                               self.gate_act, ag, nh, d, nh * dv)
        o = rt.buffer("delta.o", (T, nh * dv), f32)
        ops.delta_recurrence(qkv, beta, ag, state, batch, o, nh, nkv, d, dv)
        og = rt.buffer("delta.og", (T, nh * dv))
        ops.delta_output(o, ag[:, nh * d:], ag.shape[1], self.norm_w, self.eps, og, nh, dv)
        return rt.linear(og, self.w_o, rt.buffer("delta.delta", (T, self.hidden), f32 if self.out_f32 else None))


_G_NAMES = {"r": "r", "k": "k", "v": "v", "a": "a", "a_bias": "a.b", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0",
            "norm": "norm", "o": "o"}


@register_mixer("generalized_delta")
class GeneralizedDelta(Mixer):
    """Generalized delta rule: a decay and a removal rate per head and key channel, both acting on the OLD
    state.  Per head, with a 32-bit state ``S`` [head_dim, head_dim] per request:

        S <- diag(w_t) S - (a_t * u_t) (u_t^T S) + k_t v_t^T ;   o_t = S^T r_t

    ``r, k, v`` are projections of the input (``n_heads`` heads of ``head_dim``), ``u = k / sqrt(sum k^2 + 1e-6)``
    the head's unit key, ``w = exp(-decay_scale * sigmoid(W2 tanh(W1 x) + w0))`` (``decay_scale`` a parameter;
    ``e^-1/2`` by default), ``a = sigmoid(Wa x + a_bias)``.  A head's read-out is divided by its root mean square
    (``eps``), the heads are concatenated, multiplied by a plain weight over all heads and by
    ``sigmoid(Wg x)``, then projected by ``Wo``.  All projections that read the input are one product (written
    in 32-bit: everything after them is 32-bit); the slot keeps ``S`` of every head."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["head_dim"])
        self.rank = int(p["decay_rank"])
        self.eps = float(p["eps"])
        self.decay_scale = float(p.get("decay_scale", 0.6065306597126334))
        self.out_f32 = bool(p.get("out_f32", False))
        self.names = dict(_G_NAMES, **(p.get("names") or {}))
        if self.dim > 128:
            raise ValueError(f"generalized_delta: head_dim {self.dim} is larger than the recurrence kernel's 128")
        if self.rank < 1:
            raise ValueError("generalized_delta: decay_rank must be at least 1")
        self.w_in = self.w2 = self.w_o = self.w0 = self.a_bias = self.norm_w = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, H = self.n_heads * self.dim, self.hidden
        specs = {self._n(r): TensorSpec((n, H)) for r in ("r", "k", "v", "a", "g")}
        specs.update({self._n("a_bias"): TensorSpec((n,), role="vector"), self._n("w1"): TensorSpec((self.rank, H)),
                      self._n("w2"): TensorSpec((n, self.rank)), self._n("w0"): TensorSpec((n,), role="vector"),
                      self._n("norm"): TensorSpec((n,), role="vector"), self._n("o"): TensorSpec((H, n))})
        return specs

    def bind(self, tensors) -> None:
        dt, f32 = self.rt.dtype, torch.float32
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in ("r", "k", "v", "a", "g", "w1")], dim=0).contiguous()
        self.w2 = tensors[self._n("w2")].to(dt).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        self.w0 = tensors[self._n("w0")].to(f32).contiguous()
        self.a_bias = tensors[self._n("a_bias")].to(f32).contiguous()
        self.norm_w = tensors[self._n("norm")].to(f32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w2.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return FixedState((self.n_heads * self.dim * self.dim,), tag="generalized_delta")

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T, nh, d = self.rt, x.shape[0], self.n_heads, self.dim
        n, f32 = nh * d, torch.float32
        proj = rt.linear(x, self.w_in, rt.buffer("gdelta.proj", (T, self.w_in.shape[0]), f32))
        operands = rt.buffer("gdelta.ops", (T, 4 * n), f32)
        low = rt.buffer("gdelta.low", (T, self.rank))
        ops.gdelta_prepare(proj, self.a_bias, operands, low, 5 * n, nh, d)
        wl = rt.linear(low, self.w2, rt.buffer("gdelta.wl", (T, n), f32))
        ag = rt.buffer("gdelta.ag", (T, 2 * n), f32)
        ops.delta_gates_ex(wl, n, False, 1, self.decay_scale, None, self.w0, proj[:, 4 * n:], proj.shape[1], "sigmoid",
                           ag, nh, d, n)
        o = rt.buffer("gdelta.o", (T, n), f32)
        ops.gdelta_recurrence(operands, ag, 2 * n, proj[:, 2 * n:], proj.shape[1], cache.tensor, batch, o, nh, d)
        og = rt.buffer("gdelta.og", (T, n))
        ops.delta_output(o, ag[:, n:], 2 * n, self.norm_w, self.eps, og, nh, d, weight_per_head=True)
        return rt.linear(og, self.w_o, rt.buffer("gdelta.delta", (T, self.hidden), f32 if self.out_f32 else None))
