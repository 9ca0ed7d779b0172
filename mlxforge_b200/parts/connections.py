"""Connections between a sublayer and several residual streams ("hyper-connections").

A model with ``S`` streams keeps ``x_1 .. x_S`` per token, all equal to the embedding's output at
the start.  A sublayer reads ``u = sum_s in[s] x_s``, runs on ``norm(u)``, and its result ``y`` is
written back as ``x_t <- sum_s mix[s, t] x_s + out[t] y`` (all ``t`` at once from the old streams;
``mix`` is indexed ``[from, to]``).  At the end the model's output is the sum of the streams.  With
``S = 1`` and all three weights 1 this is the ordinary residual sum.

The write-back is not done by the connection: it hands a ``StreamWrite`` on as the layer's pending
delta, and the norm of the next sublayer (``group_rmsnorm``) applies it in the kernel that also
reads and normalises, as the single stream's add is fused into the next RMSNorm.

``conv_read`` is a connection on the reading side alone: the sublayer reads the stream itself plus a
short causal convolution of it over time, per channel (``h_t = x_t + sum_j w[:, j] x_(t-taps+1+j)``,
zeros before the sequence's start).  The last ``taps - 1`` rows it has read belong to the request's
state; the arrangement gives it a place in a state slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch

from ..csrc import ops
from .base import Connection, TensorSpec, register_connection


@dataclass
class StreamWrite:
    """A sublayer's result that has not been written into the streams yet: ``delta`` [T, H] (plus
    ``bias`` [H], 32-bit, if the sublayer's last projection has one that was not added), and the
    weights of the write (None: identity mixing, out = 1)."""

    delta: Optional[Any]
    bias: Optional[Any] = None
    mix: Optional[Any] = None
    out: Optional[Any] = None


@register_connection("hyper")
class HyperConnection(Connection):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.streams = int(params["streams"])
        if not (1 <= self.streams <= 8):
            raise ValueError(f"hyper connection: {self.streams} streams (1 to 8 are supported)")
        self.w_in = self.w_out = self.w_mix = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        s = self.streams
        return {self.prefix + "in": TensorSpec((s,), role="vector"),
                self.prefix + "out": TensorSpec((s,), role="vector"),
                self.prefix + "mix": TensorSpec((s, s), role="vector")}

    def bind(self, tensors) -> None:
        self.w_in = tensors[self.prefix + "in"].to(torch.float32).contiguous()
        self.w_out = tensors[self.prefix + "out"].to(torch.float32).contiguous()
        self.w_mix = tensors[self.prefix + "mix"].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (2 * self.streams + self.streams ** 2) * 4

    def write(self, delta, bias=None) -> StreamWrite:
        return StreamWrite(delta, bias, self.w_mix, self.w_out)


@register_connection("conv_read")
class ConvRead(Connection):
    """``read(x)`` = ``x + conv(x)`` with the weight ``tensor`` [size, taps] (no bias), in 32-bit on the
    32-bit stream, rounded once to the compute dtype."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.taps = int(params["taps"])
        self.name = self.prefix + str(params.get("tensor", "conv"))
        # taps 0: no convolution and no tensor; the sublayer reads the stream's rounding (one tap of weight zero)
        self.identity = self.taps == 0
        if self.identity:
            self.taps = 1
        if self.taps < 1:
            raise ValueError(f"conv_read: {self.taps} taps (0 for none, else at least 1)")
        self.weight = None

    @property
    def state_floats(self) -> int:
        """32-bit numbers of a request's state: the last taps - 1 rows of the stream."""
        return (self.taps - 1) * self.size

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {} if self.identity else {self.name: TensorSpec((self.size, self.taps), role="vector")}

    def bind(self, tensors) -> None:
        if self.identity:
            self.weight = torch.zeros((self.size, 1), dtype=torch.float32, device=self.rt.device)
        else:
            self.weight = tensors[self.name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * self.taps * 4

    def read(self, x, batch, state, offset: int, name: str = "conv.read"):
        """``x`` [T, size] the 32-bit stream; ``state`` [slots, floats] with this connection's rows from
        ``offset`` on.  Returns [T, size] in the compute dtype; the slots' rows move on."""
        out = self.rt.buffer(name, (x.shape[0], self.size))
        ops.conv_input(x, self.weight, state, offset, batch, out)
        return out
