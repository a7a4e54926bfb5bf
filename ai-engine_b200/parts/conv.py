"""A short causal convolution over time in front of a sublayer: out_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j),
per channel, zeros before the sequence's start.  The last taps - 1 inputs of a request are state of the
request; a portion of a prompt or a single decoded token continues from them."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import StateRequest, TokenFilter


class CausalShortConv(TokenFilter):
    """params: size (channels), taps.  tensors: weight [size, taps] (no bias).  Input float32 rows (a norm's
    output), output in the compute dtype; the sum is float32."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size, self.taps = int(spec.params["size"]), int(spec.params["taps"])
        if self.taps < 1:
            raise ValueError(f"short convolution: taps must be >= 1, got {self.taps}")
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.tensors["weight"], (self.size, self.taps), std=0.2)]

    def load(self, source):
        self.weight = source.get(self.spec.tensors["weight"]).float().contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def flops(self, tokens, keys=0.0):
        return 2.0 * tokens * self.size * self.taps

    def state_request(self):
        return StateRequest((self.taps - 1, self.size), torch.float32)

    def forward(self, h, ctx, cache):
        return ops.short_conv(h, self.weight, cache.state, ctx, self.env.dtype)
