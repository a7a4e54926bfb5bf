"""Two mixers side by side: both read the same input, and their outputs are added with a weight each,

    out = left_scale * left(h) + right_scale * right(h)

in float32.  Each of the two is a mixer of any registered kind with a cache or state of its own."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer
from .registry import lookup


class ParallelMixers(Mixer):
    """params: left, right (PartSpec of a mixer each), left_scale, right_scale."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.left = lookup("mixer", p["left"].kind)(p["left"], env)
        self.right = lookup("mixer", p["right"].kind)(p["right"], env)
        self.left_scale, self.right_scale = float(p["left_scale"]), float(p["right_scale"])

    def sub_parts(self):
        return {"left": self.left, "right": self.right}

    def tensor_specs(self):
        return self.left.tensor_specs() + self.right.tensor_specs()

    def load(self, source):
        self.left.load(source)
        self.right.load(source)

    def weight_bytes(self):
        return self.left.weight_bytes() + self.right.weight_bytes()

    def flops(self, tokens, keys=0.0):
        return self.left.flops(tokens, keys) + self.right.flops(tokens, keys)

    def forward(self, h, ctx, cache, add_to=None):
        kids = cache.children if cache is not None and cache.children else {}
        a = self.left.forward(h, ctx, kids.get("left"))
        b = self.right.forward(h, ctx, kids.get("right"))
        return ops.scaled_sum(ops.cast(a, torch.float32), self.left_scale, ops.cast(b, torch.float32),
                              self.right_scale)
