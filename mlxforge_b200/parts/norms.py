"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` over the last axis, the weight
multiplying directly (src/model/decoder_model.cpp:206-208).  The sum of squares,
the scaling and the residual sum it is fused with are 32-bit.

``one_plus``: the stored weight lies around zero and ``1 + w`` multiplies.  ``scale``: a constant folded into
the weight (a model whose logits are multiplied by a constant applies it to the final norm's rows, which
is the same product).  ``post_add`` is the norm on a sublayer's OUTPUT: ``residual += rms(y) * w``.

A layer whose branches run side by side on one residual hands on two deltas at once
(``DeltaPair``) and wants two norms of the same sum: ``RMSNorm.pair_forward`` adds both deltas
and applies both weights in one kernel."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import DeltaPair, Norm, ScaledPair, TensorSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = self.prefix + str(params.get("tensor", "weight"))
        self.one_plus = bool(params.get("one_plus", False))
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), role="vector")}

    def bind(self, tensors) -> None:
        w = tensors[self.name].to(torch.float32)
        if self.one_plus:
            w = w + 1.0
        if self.scale != 1.0:
            w = w * self.scale
        self.weight = w.contiguous()

    def weight_bytes(self) -> int:
        return self.size * 4

    def forward(self, x, out=None):
        return self.add_forward(x, None, out)

    def post_add(self, residual, y) -> None:
        """``residual += rms(y) * weight`` in 32-bit, in place; ``y`` [T, size] is a sublayer's output (32-bit or
        the compute dtype) or a ``ScaledPair`` of two branches' outputs, whose weighted sum is normalised."""
        if isinstance(y, ScaledPair):
            ops.postnorm_add(residual, y.first, y.first_scale, y.second, y.second_scale, self.weight, self.eps)
        else:
            ops.postnorm_add(residual, y, 1.0, None, 0.0, self.weight, self.eps)

    def add_forward(self, residual, delta, out=None, rows=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = self.rt.buffer("norm.out", (n, self.size))
        if isinstance(delta, DeltaPair):
            ops.add_rmsnorm_pair(residual, delta.first, delta.second, self.weight, None, self.eps, out, None, rows)
        else:
            ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out

    def pair_forward(self, residual, delta, other: "RMSNorm" = None):
        """``residual += delta`` (a tensor, a ``DeltaPair`` or None), then this norm of the sum and, with
        ``other``, that norm (same size and eps, its own weight) of the same sum: (out, out_other)."""
        if other is not None and (other.size != self.size or other.eps != self.eps):
            raise ValueError("pair_forward: the two norms must agree in size and eps")
        pair = delta if isinstance(delta, DeltaPair) else DeltaPair(delta, None)
        n = residual.shape[0]
        out1 = self.rt.buffer("norm.out", (n, self.size))
        out2 = self.rt.buffer("norm.out2", (n, self.size)) if other is not None else None
        ops.add_rmsnorm_pair(residual, pair.first, pair.second, self.weight, other.weight if other is not None else None,
                             self.eps, out1, out2)
        return out1, out2


@register_norm("group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in groups: the channels are cut into ``groups`` equal consecutive parts, each divided
    by its own ``sqrt(mean(part^2) + eps)``, and the whole is multiplied by the weight (``groups`` = 1
    is RMSNorm).  It also knows models with several residual streams (``streams``): the stream tensor
    is then [T, streams * size], a pending ``StreamWrite`` (see ``connections.py``) is written back
    into the streams first, and the streams are read with the weights ``read`` (None: their plain sum)
    before the norm; all of it is one kernel."""

    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1) or 1)
        self.streams = int(params.get("streams", 1) or 1)
        self.name = self.prefix + str(params.get("tensor", "weight"))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.size} channels do not divide into {self.groups} groups")
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), role="vector")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 4

    def forward(self, x, out=None):
        return self.add_forward(x, None, out)

    def add_forward(self, residual, delta, out=None, rows=None, read=None):
        from .connections import StreamWrite
        n = residual.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = self.rt.buffer("norm.out", (n, self.size))
        w = delta if isinstance(delta, StreamWrite) else StreamWrite(delta)
        ops.hyper_update_norm(residual, w.delta, w.bias, w.mix, w.out, read, self.weight, self.eps, self.groups, out,
                              self.streams, rows)
        return out
