"""Dense feed-forwards.  Gated: ``down( act(gate(x)) * up(x) )`` with ``act`` = SiLU
(src/model/decoder_model.cpp:277-282) or, as a parameter (``activation: "gelu_tanh"``), the tanh
form of GELU; ``names`` maps the three roles to tensor names behind the prefix.  Gate and up are one matrix here, their
rows interleaved in groups of 8 (8 gate rows, then the matching 8 up rows) so a
kernel that owns 16 consecutive output rows holds both halves of a product;
when the intermediate size is no multiple of 8 the two are simply stacked.

Without a gate (``dense_mlp``): ``down( act(up(x)) )`` with ``act`` one of the same activations or
``"relu2"``, the square of the rectified value; ``names`` maps the two roles to tensor names."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.group = 8 if self.inter % 8 == 0 else self.inter
        self.act = str(params.get("activation", "silu"))
        ops.activation_code(self.act)
        n = params.get("names") or {}
        self.names = {"gate": n.get("gate", "gate_proj.weight"), "up": n.get("up", "up_proj.weight"),
                      "down": n.get("down", "down_proj.weight")}
        self.w_gu = None
        self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self.prefix + self.names["gate"]: TensorSpec((self.inter, self.hidden)),
            self.prefix + self.names["up"]: TensorSpec((self.inter, self.hidden)),
            self.prefix + self.names["down"]: TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        g = tensors[self.prefix + self.names["gate"]].to(dt)
        u = tensors[self.prefix + self.names["up"]].to(dt)
        n = self.inter // self.group
        gu = torch.stack([g.view(n, self.group, self.hidden), u.view(n, self.group, self.hidden)], dim=1)
        self.w_gu = gu.reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors[self.prefix + self.names["down"]].to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_gu.numel() + self.w_down.numel()) * self.w_gu.element_size()

    def forward(self, x, batch):
        rt = self.rt
        T = x.shape[0]
        act = rt.linear_swiglu(x, self.w_gu, self.group, rt.buffer("ffn.act", (T, self.inter)), self.act)
        return rt.linear(act, self.w_down, rt.buffer("ffn.delta", (T, self.hidden)))


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """``down(act(up(x)))``: two products and an activation between them, applied in 32-bit to the first
    product's sums before they are rounded (in that product's epilogue where its kernel has one)."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.act = str(params.get("activation", "relu2"))
        ops.activation_code(self.act)
        n = params.get("names") or {}
        self.names = {"up": n.get("up", "up"), "down": n.get("down", "down")}
        self.w_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.prefix + self.names["up"]: TensorSpec((self.inter, self.hidden)),
                self.prefix + self.names["down"]: TensorSpec((self.hidden, self.inter))}

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        self.w_up = tensors[self.prefix + self.names["up"]].to(dt).contiguous()
        self.w_down = tensors[self.prefix + self.names["down"]].to(dt).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_up.numel() + self.w_down.numel()) * self.w_up.element_size()

    def forward(self, x, batch):
        rt, T = self.rt, x.shape[0]
        a = rt.linear_act(x, self.w_up, rt.buffer("ffn.act", (T, self.inter)), self.act)
        return rt.linear(a, self.w_down, rt.buffer("ffn.delta", (T, self.hidden)))
