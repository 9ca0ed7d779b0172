"""Retention: linear attention with a fixed decay per head, a recurrent mixer without softmax.

Per head, with a 32-bit state ``S`` [head_dim, v_head_dim] per request that starts at zero, token
after token:

    S <- decay_h S + k_t v_t^T ;   o_t = S^T q_t

``q, k`` (``n_heads`` heads of ``head_dim``) and ``v`` (``n_heads`` heads of ``v_head_dim``) are
projections of the input; q and k are rotated by position (the ``rotary`` encoding's constants:
``rotary_dim`` leading channels, half-split pairs), k is then multiplied by ``head_dim^-1/2``.
Every head's read-out is divided by its root mean square over ``v_head_dim`` (``eps``, no weight),
the heads are concatenated, multiplied by ``silu(W_g x)`` and projected by ``W_o``.

Options, each a parameter: ``activation: "silu"`` passes q, k and v through SiLU first ("lightning" attention
is this with ``rotary_dim`` 0 and ``key_scale`` 1); ``output_norm: "whole"`` divides the concatenated heads by
ONE root mean square over all of them instead of one per head; ``norm_weight`` names a plain weight
[n_heads * v_head_dim] that multiplies the normalised read-out; ``gate_act: "sigmoid"`` replaces the gate's
SiLU; ``out_f32`` writes the output projection in 32-bit.

The request's slot keeps ``S`` of every head, so a step goes on from where the step before ended,
however the prompt was cut.  All projections that read the mixer's input are one product;
everything after them is 32-bit.  ``names`` maps the tensors' roles to their names.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FixedState, Mixer, TensorSpec, register_mixer
from .rope import inverse_wavelengths

_NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}


@register_mixer("retention")
class Retention(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.rot = int(p.get("rotary_dim", self.dim))
        self.eps = float(p["eps"])
        self.decay_host = [float(d) for d in p["decay"]]
        self.k_scale = float(p.get("key_scale", self.dim ** -0.5))
        self.names = dict(_NAMES, **(p.get("names") or {}))
        self.activation = p.get("activation")
        self.output_norm = str(p.get("output_norm", "head"))
        self.norm_weight_name = p.get("norm_weight")
        self.gate_act = str(p.get("gate_act", "silu"))
        self.out_f32 = bool(p.get("out_f32", False))
        if self.activation not in (None, "silu"):
            raise ValueError(f"retention: activation must be 'silu' or None, got '{self.activation}'")
        if self.output_norm not in ("head", "whole") or self.gate_act not in ("silu", "sigmoid"):
            raise ValueError("retention: output_norm is 'head' or 'whole', gate_act 'silu' or 'sigmoid'")
        self.norm_w = None
        if len(self.decay_host) != self.n_heads:
            raise ValueError(f"retention: {len(self.decay_host)} decays for {self.n_heads} heads")
        if self.rot % 2 or self.rot > self.dim:
            raise ValueError(f"retention: rotary_dim {self.rot} must be even and at most head_dim")
        if self.dim > 512:
            raise ValueError(f"retention: head_dim {self.dim} is larger than the recurrence kernel's 512")
        self.inv_f, inv_d = inverse_wavelengths(self.rot, float(p.get("rope_base", 10000.0)), runtime.device)
        self.inv_d = inv_d if runtime.precise else None
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32, device=runtime.device)
        self.w_in = self.w_o = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nqk, nv, H = self.n_heads * self.dim, self.n_heads * self.vdim, self.hidden
        specs = {self._n("q"): TensorSpec((nqk, H)), self._n("k"): TensorSpec((nqk, H)),
                 self._n("v"): TensorSpec((nv, H)), self._n("g"): TensorSpec((nv, H)),
                 self._n("o"): TensorSpec((H, nv))}
        if self.norm_weight_name:
            specs[self.prefix + self.norm_weight_name] = TensorSpec((nv,), role="vector")
        return specs

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        if self.norm_weight_name:
            self.norm_w = tensors[self.prefix + self.norm_weight_name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return FixedState((self.n_heads * self.dim * self.vdim,), tag="retention")

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T, nh, d, dv = self.rt, x.shape[0], self.n_heads, self.dim, self.vdim
        f32 = torch.float32
        proj = rt.linear(x, self.w_in, rt.buffer("ret.in", (T, self.w_in.shape[0])))
        ld = proj.shape[1]
        qk = rt.buffer("ret.qk", (T, 2 * nh * d), f32)
        if self.activation:
            # the values pass the activation too: they go on in 32-bit beside the queries and keys
            v = rt.buffer("ret.v", (T, nh * dv), f32)
            ops.retention_prepare(proj, nh, d, self.rot, self.k_scale, batch.positions, self.inv_f, self.inv_d, qk,
                                  True, v, 2 * nh * d)
            v_ld = nh * dv
        else:
            ops.retention_prepare(proj, nh, d, self.rot, self.k_scale, batch.positions, self.inv_f, self.inv_d, qk)
            v, v_ld = proj[:, 2 * nh * d:], ld
        o = rt.buffer("ret.o", (ops.retention_parts(d, dv, v, v_ld), T, nh * dv), f32)
        ops.retention_recurrence(qk, v, v_ld, self.decay, cache.tensor, batch, o, nh, d, dv)
        og = rt.buffer("ret.og", (T, nh * dv))
        ops.retention_output(o, proj[:, 2 * nh * d + nh * dv:], ld, self.eps, og, nh, dv, self.norm_w,
                             self.output_norm == "whole", self.gate_act)
        return rt.linear(og, self.w_o, rt.buffer("ret.delta", (T, self.hidden), f32 if self.out_f32 else None))
