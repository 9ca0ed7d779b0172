"""Mixture of experts: a router that scores the experts, the chosen experts' gated feed-forwards,
their weighted sum.

Router (32-bit), by ``scoring``: ``s = sigmoid(Wr x)`` or ``s = softmax(Wr x)`` over all router outputs.
The ``n_experts`` experts may form ``n_groups`` equal groups of neighbours; a group's score is the sum of
its two largest ``s``, and only experts of the ``keep_groups`` best groups can be chosen (``n_groups`` = 0:
any expert).  Each token uses the ``top`` allowed experts with the largest ``s`` (plus ``choice_bias``, a
tensor with one number per router output that steers the choice and nothing else), weighted by
``s * route_scale`` (not renormalised); ties go to the lower index.  Expert ``e``:

    g = min(Wg_e x, limit) ;  u = clamp(Wu_e x, -limit, limit) ;  y = Wd_e (g sigmoid(alpha g) (u + up_offset))

(no ``limit``, ``alpha`` 1 and ``up_offset`` 0 make it ``Wd (silu(Wg x) * (Wu x))``).

``renormalize``: the chosen experts' weights are divided by their sum (+ 1e-20).  ``expert_act`` (``"relu2"``,
``"silu"``, ``"gelu_tanh"``): the experts have no gate, ``y = Wd_e act(Wu_e x)``, and no ``gate`` tensors.

``n_identity`` further router outputs, after the experts', stand for experts without matrices that return
their input: a token that chooses one gets ``weight * x``.  ``shared`` (a feed-forward part's spec) is a
branch every token takes; it is added times ``sigmoid(w_sg . x)`` where ``shared_gate`` names that row
vector (its product rides along with the router's), else as it is.

The experts' matrices are stacked at load time (``[E, 2, ff, H]`` gate rows then up rows, and
``[E, H, ff]``).  Few tokens (and the 32-bit path) take the kernel with a block per (token, chosen
expert), which streams that expert's matrices once; many tokens in bfloat16 are sorted by expert
and go through the library's grouped product (as the engine's other many-row products go through
the library) with this engine's gather, activation and weighted-sum kernels around it, or, where
nothing may be allocated (a CUDA graph being recorded), the library lacks it, or the backend is
``tcgen05``/``MLXFORGE_MOE_TILES=1``, through this engine's own tensor-core tiles.  Either way a
token's chosen experts are added in the order of the choice, so its result does not depend on what
else is in the batch.
"""
from __future__ import annotations

import math
import os
from typing import Dict

import torch

from ..csrc import ops
from .base import FEED_FORWARDS, FeedForward, TensorSpec, build_part, register_feed_forward

_NAMES = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.ff = int(p["intermediate_size"])
        self.n_experts = int(p["n_experts"])
        self.n_identity = int(p.get("n_identity") or 0)
        self.top = int(p["top"])
        self.n_groups = int(p.get("n_groups") or 0)
        self.keep = int(p.get("keep_groups") or 0)
        self.route_scale = float(p.get("route_scale", 1.0))
        self.scoring = str(p.get("scoring", "sigmoid"))
        self.limit = float(p["limit"]) if p.get("limit") is not None else math.inf
        self.alpha = float(p.get("alpha", 1.702))
        self.up_offset = float(p.get("up_offset", 1.0))
        self.renormalize = bool(p.get("renormalize", False))
        self.expert_act = p.get("expert_act")
        if self.expert_act is not None:
            ops.activation_code(self.expert_act)
        self.choice_bias_name = p.get("choice_bias")
        self.shared_gate_name = p.get("shared_gate")
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if self.scoring not in ("sigmoid", "softmax"):
            raise ValueError(f"routed_experts: scoring must be 'sigmoid' or 'softmax', got '{self.scoring}'")
        if self.n_experts < 0 or self.n_identity < 0 or not (1 <= self.top <= self.n_outputs):
            raise ValueError(f"routed_experts: top {self.top} of {self.n_experts} experts and {self.n_identity} "
                             f"identity experts")
        if self.n_groups:
            if self.n_identity:
                raise ValueError("routed_experts: groups of experts and identity experts do not go together")
            if self.n_experts % self.n_groups or not (1 <= self.keep <= self.n_groups):
                raise ValueError(f"routed_experts: {self.n_experts} experts, {self.n_groups} groups, keep {self.keep}")
            if self.keep * (self.n_experts // self.n_groups) < self.top:
                raise ValueError("routed_experts: the kept groups hold fewer experts than a token uses")
        self.shared = build_part(FEED_FORWARDS, p["shared"], runtime) if p.get("shared") is not None else None
        if self.shared_gate_name and self.shared is None:
            raise ValueError("routed_experts: a shared gate without a shared branch")
        # tokens from which the sorted, tiled path is taken (bfloat16 only)
        self.grouped_min_tokens = int(p.get("grouped_min_tokens", 64))
        self.w_router = self.w_gu = self.w_down = self.choice_bias = None

    @property
    def n_outputs(self) -> int:
        """Outputs of the router: the experts and the identity experts."""
        return self.n_experts + self.n_identity

    def _e(self, e: int, role: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.names["router"]: TensorSpec((self.n_outputs, self.hidden))}
        for e in range(self.n_experts):
            if self.expert_act is None:
                specs[self._e(e, "gate")] = TensorSpec((self.ff, self.hidden))
            specs[self._e(e, "up")] = TensorSpec((self.ff, self.hidden))
            specs[self._e(e, "down")] = TensorSpec((self.hidden, self.ff))
        if self.choice_bias_name:
            specs[self.prefix + self.choice_bias_name] = TensorSpec((self.n_outputs,), role="vector")
        if self.shared_gate_name:
            specs[self.prefix + self.shared_gate_name] = TensorSpec((1, self.hidden))
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        rows = [tensors[self.prefix + self.names["router"]].to(dt)]
        if self.shared_gate_name:        # the shared branch's gate logit is one more column of the router's product
            rows.append(tensors[self.prefix + self.shared_gate_name].to(dt).view(1, self.hidden))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        first = ("gate", "up") if self.expert_act is None else ("up",)
        if self.n_experts:
            self.w_gu = torch.stack([torch.stack([tensors[self._e(e, r)].to(dt) for r in first])
                                     for e in range(self.n_experts)]).contiguous()     # [E, 2, ff, H]; [E, 1, ff, H] ungated
            self.w_down = torch.stack([tensors[self._e(e, "down")].to(dt) for e in range(self.n_experts)]).contiguous()
        else:
            self.w_gu = torch.zeros((0, len(first), self.ff, self.hidden), dtype=dt, device=self.w_router.device)
            self.w_down = torch.zeros((0, self.hidden, self.ff), dtype=dt, device=self.w_router.device)
        if self.choice_bias_name:
            self.choice_bias = tensors[self.prefix + self.choice_bias_name].to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def weight_bytes(self) -> int:
        # a step reads the router and, per token, `top` experts; at most all of them
        per = (3 if self.expert_act is None else 2) * self.ff * self.hidden * self.w_gu.element_size()
        shared = self.shared.weight_bytes() if self.shared is not None else 0
        return self.w_router.numel() * self.w_router.element_size() + self.n_experts * per + shared

    def route(self, x):
        """(ids [T, top], weights [T, top], z): the choice, and the router's product with the shared gate's
        logit in its last column where there is one."""
        T = x.shape[0]
        z = self.rt.linear(x, self.w_router, self.rt.buffer("moe.z", (T, self.w_router.shape[0]), torch.float32))
        ids = self.rt.buffer("moe.ids", (T, self.top), torch.int32)
        weights = self.rt.buffer("moe.weights", (T, self.top), torch.float32)
        ops.moe_route(z, self.n_groups, self.keep, self.top, self.route_scale, ids, weights, self.n_outputs,
                      self.scoring == "softmax", self.choice_bias, self.renormalize)
        return ids, weights, z

    def _combine(self, y, weights, slot_of, out, slices, ids, x, z, shared):
        """The weighted sum with what the plain one does not have: identity experts and the shared branch."""
        gate = z[:, self.n_outputs:] if self.shared_gate_name else None
        ops.moe_combine(y, weights, slot_of, out, slices, ids if self.n_identity else None, self.n_experts,
                        x if self.n_identity else None, shared, gate, z.shape[1])

    def forward(self, x, batch):
        rt, T = self.rt, x.shape[0]
        ids, weights, z = self.route(x)
        shared = self.shared.forward(x, batch) if self.shared is not None else None
        out = rt.buffer("moe.delta", (T, self.hidden))
        if (x.dtype == torch.bfloat16 and T >= self.grouped_min_tokens and self.n_experts
                and ops.moe_grouped_ok(self.hidden, self.ff, self.n_experts)):
            return self.forward_grouped(x, ids, weights, out, z, shared)
        slices = ops.moe_rows_slices(self.ff)
        y = rt.buffer("moe.y", (T, self.top * slices, self.hidden), torch.float32)
        if self.n_experts:
            ops.moe_rows(x, self.w_gu, self.w_down, ids, y, self.limit, self.alpha, self.up_offset, self.expert_act)
        self._combine(y, weights, None, out, slices, ids, x, z, shared)
        return out

    def _library_grouped(self) -> bool:
        """Whether the two products of the sorted pairs go through the library's grouped product."""
        if os.environ.get("MLXFORGE_MOE_TILES", "0") == "1" or getattr(self.rt, "gemm_backend", "auto") == "tcgen05":
            return False
        return hasattr(torch, "_grouped_mm") and not torch.cuda.is_current_stream_capturing()

    def forward_grouped(self, x, ids, weights, out, z, shared):
        """Many tokens: pairs ordered by expert, the two products over the sorted rows, the weighted sum in
        the order of the choice."""
        rt, T = self.rt, x.shape[0]
        i32, n = torch.int32, T * self.top
        slot_of = rt.buffer("moe.slot_of", (n,), i32)
        row_token = rt.buffer("moe.row_token", (n,), i32)
        meta = rt.buffer("moe.meta", (4,), i32)
        tiles = rt.buffer("moe.tiles", (3 * ops.moe_grouped_max_tiles(T, self.top, self.n_experts),), i32)
        ends = rt.buffer("moe.ends", (self.n_experts,), i32)
        ops.moe_sort(ids, self.n_experts, slot_of, row_token, meta, tiles, ends)
        act = rt.buffer("moe.act", (n, self.ff))
        if self._library_grouped():
            xg = rt.buffer("moe.xg", (n, self.hidden))
            ops.moe_gather_rows(x, row_token, xg)
            gu = torch._grouped_mm(xg, self.w_gu.view(self.n_experts, -1, self.hidden).transpose(1, 2), offs=ends)
            if self.expert_act is None:
                ops.moe_activation(gu, act, self.limit, self.alpha, self.up_offset)
            else:
                ops.unary_act(gu, act, self.expert_act)
            y = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=ends)
            self._combine(y, weights, slot_of, out, 1, ids, x, z, shared)
            return out
        ops.moe_grouped_up(x, self.w_gu, row_token, meta, tiles, act, self.top, self.limit, self.alpha, self.up_offset,
                           self.expert_act)
        y = rt.buffer("moe.y", (n, self.hidden), torch.float32)
        ops.moe_grouped_down(act, self.w_down, meta, tiles, y, T, self.top)
        self._combine(y, weights, slot_of, out, 1, ids, x, z, shared)
        return out
