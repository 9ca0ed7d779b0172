"""Token embedding (``h[t] = E[token[t]]``, src/model/decoder_model.cpp:194-204;
optionally times a constant ``scale``)
into the 32-bit residual stream (into every stream, where a model has several;
optionally plus a sinusoidal position vector), and the output head (``logits = hn W^T`` with
``W = lm_head.weight`` when the checkpoint has it, else the embedding table,
:346-350), computed only for the rows that were asked for, in float32."""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

from ..csrc import ops
from .base import Part, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = self.prefix + str(params.get("tensor", "weight"))
        # "sinusoid": channel 2i gets sin(p f_i), channel 2i+1 cos(p f_i), f_i = theta^(-2i/hidden)
        self.positions = params.get("positions")
        if self.positions not in (None, "sinusoid"):
            raise ValueError(f"token_embedding: unknown positions '{self.positions}' (None or 'sinusoid')")
        self.theta = float(params.get("theta", 10000.0))
        # the row is multiplied by this on its way into the residual stream (the head, where it shares
        # the table, reads the table itself)
        self.scale = float(params.get("scale", 1.0))
        if self.scale != 1.0 and self.positions is not None:
            raise ValueError("token_embedding: a scale together with added positions is not supported")
        self.freqs = None
        self.table = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors) -> None:
        self.table = tensors[self.name].to(self.rt.dtype).contiguous()
        if self.positions == "sinusoid":
            i = np.arange((self.hidden + 1) // 2, dtype=np.float64)
            self.freqs = torch.from_numpy(np.power(self.theta, -2.0 * i / self.hidden)).to(self.rt.device)

    def weight_bytes(self) -> int:
        return 0     # a step reads one row per token, not the table

    def forward(self, tokens, out):
        ops.embed(self.table, tokens, out, self.scale)
        return out

    def embed(self, batch, out, copies: int = 1):
        """The step's tokens into ``out`` [T, copies * hidden]: every copy (residual stream) starts equal."""
        if self.positions is None and copies == 1:
            return self.forward(batch.tokens, out)
        ops.embed_positions(self.table, batch.tokens, batch.positions, self.freqs, out, copies, self.rt.precise)
        return out


@register_head("linear_head")
class LinearHead(Part):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = self.prefix + str(params.get("tensor", "weight"))
        self.tied_to = params.get("tied_to")
        self.require_own = bool(params.get("require_own", False))
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        own = TensorSpec((self.vocab, self.hidden), optional=not self.require_own and self.tied_to is not None)
        specs = {self.name: own}
        if self.tied_to and not self.require_own:
            specs[self.tied_to] = TensorSpec((self.vocab, self.hidden))
        return specs

    def bind(self, tensors) -> None:
        w = tensors.get(self.name)
        if w is None:
            w = tensors[self.tied_to]
        self.weight = w.to(self.rt.dtype).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, out):
        """x [n, H] in the compute dtype -> float32 logits [n, V]."""
        return self.rt.linear(x, self.weight, out)
