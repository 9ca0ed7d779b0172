"""Two mixers side by side on one input: ``left_scale * left(x) + right_scale * right(x)``.

Each branch is any registered mixer, built from its own ``PartSpec`` (``left`` and ``right``), with its own
tensors and its own cache need; the pair's need is the tuple of both (a branch without a need leaves no
entry) and the pair hands each branch its own lanes.  The two outputs are not added here: they travel
on as a ``ScaledPair`` so that whoever takes them (the norm on the sublayer's output) forms the weighted
sum in 32-bit in the kernel it runs anyway.

The branches depend on nothing of each other.  With many tokens in a step (``overlap_min_tokens``, 256 by
default; 0 switches it off) the right branch is launched on a second stream, forked from and joined back to
the step's stream by events, so that a branch whose kernels fill a fraction of the GPU (a recurrence that is
serial in time) runs beside the other's products and attention instead of before them.  Steps of few
tokens (decoding, which is replayed from CUDA graphs) stay on one stream.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import MIXERS, Mixer, ScaledPair, TensorSpec, build_part, count_needs, flatten_needs, register_mixer


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.left = build_part(MIXERS, params["left"], runtime)
        self.right = build_part(MIXERS, params["right"], runtime)
        self.left_scale = float(params.get("left_scale", 1.0))
        self.right_scale = float(params.get("right_scale", 1.0))
        self.n_left = count_needs(self.left.cache_need())
        self.n_right = count_needs(self.right.cache_need())
        self.overlap_min_tokens = int(params.get("overlap_min_tokens", 256))
        self._side = self._fork = self._join = None

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = dict(self.left.tensor_specs())
        specs.update(self.right.tensor_specs())
        return specs

    def bind(self, tensors) -> None:
        self.left.bind(tensors)
        self.right.bind(tensors)

    def weight_bytes(self) -> int:
        return self.left.weight_bytes() + self.right.weight_bytes()

    def cache_need(self):
        needs = flatten_needs(self.left.cache_need(), self.right.cache_need())
        return None if not needs else (needs[0] if len(needs) == 1 else needs)

    @staticmethod
    def _lanes(lanes, first: int, n: int):
        return None if n == 0 else (lanes[first] if n == 1 else tuple(lanes[first:first + n]))

    def forward(self, x, batch, cache, writes_cache: bool = True):
        lanes = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        left_lanes, right_lanes = self._lanes(lanes, 0, self.n_left), self._lanes(lanes, self.n_left, self.n_right)
        # the opt-in products with scratch of their own (partial sums shared by all calls) stay on one stream
        shared_scratch = getattr(self.rt, "mid_rows_enabled", False) or getattr(self.rt, "gemm_backend", "auto") == "tcgen05"
        if shared_scratch or not (self.overlap_min_tokens and x.shape[0] >= self.overlap_min_tokens and x.is_cuda):
            y1 = self.left.forward(x, batch, left_lanes, writes_cache)
            y2 = self.right.forward(x, batch, right_lanes, writes_cache)
            return ScaledPair(y1, self.left_scale, y2, self.right_scale)
        if self._side is None:
            self._side, self._fork, self._join = torch.cuda.Stream(), torch.cuda.Event(), torch.cuda.Event()
        main = torch.cuda.current_stream()
        self._fork.record(main)                       # x and everything before it are ready for the side stream
        self._side.wait_event(self._fork)
        with torch.cuda.stream(self._side):
            y2 = self.right.forward(x, batch, right_lanes, writes_cache)
            self._join.record(self._side)
        y1 = self.left.forward(x, batch, left_lanes, writes_cache)
        main.wait_event(self._join)                   # whoever takes the pair reads both
        return ScaledPair(y1, self.left_scale, y2, self.right_scale)
