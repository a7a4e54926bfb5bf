"""A selective state-space mixer with one decay per token and head (the form in which a state-space layer is a
linear attention whose decay is a scalar):

    [z | x | B | C | dt] = W_in h           z, x: P heads of dv channels; B, C: G groups of N; dt: P
    (x, B, C) <- silu(causal convolution over time + bias), per channel
    dt <- softplus(dt + dt_bias);  a = exp(-exp(A_log) dt)
    S_t = a_t S_(t-1) + dt_t B_t x_t^T     (S: [N, dv] per head, float32; head p reads group p / (P / G))
    y_t = S_t^T C_t + D x_t
    out = W_o (norm(y * silu(z)) * w)      the norm divides each of `norm_groups` equal parts of the row by its own
                                           root mean square

The state and the convolution's last taps - 1 inputs live in the request's slot, so a portion of a prompt or a
decoded token continues where the previous step stopped.  Step sizes, decays, the state, the gate and the norm are
float32 in both compute dtypes.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateRequest


class ScalarDecayStateSpace(Mixer):
    """params: hidden_size, num_heads (P), value_dim (dv), state_size (N), groups (G), taps, norm_groups, eps.
    tensors: in [2 P dv + 2 G N + P, hidden], conv [P dv + 2 G N, taps], conv_bias, dt_bias [P], a_log [P],
    skip [P], norm [P dv], o [hidden, P dv]."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.P, self.dv = int(p["hidden_size"]), int(p["num_heads"]), int(p["value_dim"])
        self.N, self.G, self.taps = int(p["state_size"]), int(p["groups"]), int(p["taps"])
        self.norm_groups, self.eps = int(p.get("norm_groups") or 1), float(p["eps"])
        self.inner = self.P * self.dv
        if self.P % self.G:
            raise ValueError(f"state space: {self.P} heads are not a multiple of {self.G} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"state space: the width {self.inner} does not divide into {self.norm_groups} norm groups")
        if self.taps < 1:
            raise ValueError(f"state space: taps must be >= 1, got {self.taps}")
        self.channels = self.inner + 2 * self.G * self.N
        self.w_in = self.w_o = self.w_conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm_w = None

    def tensor_specs(self):
        t = self.spec.tensors
        return [TensorSpec(t["in"], (2 * self.inner + 2 * self.G * self.N + self.P, self.hidden)),
                TensorSpec(t["conv"], (self.channels, self.taps), std=0.4),
                TensorSpec(t["conv_bias"], (self.channels,), std=0.1),
                TensorSpec(t["dt_bias"], (self.P,), mean=-1.0, std=0.5),
                TensorSpec(t["a_log"], (self.P,), mean=-0.5, std=0.5),
                TensorSpec(t["skip"], (self.P,), mean=1.0, std=0.2),
                TensorSpec(t["norm"], (self.inner,), init="ones"),
                TensorSpec(t["o"], (self.hidden, self.inner))]

    def load(self, source):
        t = self.spec.tensors
        f32 = lambda name: source.get(t[name]).float().contiguous()
        self.w_in, self.w_o = source.get(t["in"]), source.get(t["o"])
        self.w_conv, self.conv_bias = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.skip, self.norm_w = f32("dt_bias"), f32("a_log"), f32("skip"), f32("norm")

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, tokens, keys=0.0):
        proj = 2.0 * tokens * self.hidden * (self.w_in.shape[0] + self.inner)
        return proj + 4.0 * tokens * self.P * self.N * self.dv

    def state_request(self):
        return {"tail": StateRequest((self.taps - 1, self.channels), torch.float32),
                "S": StateRequest((self.P, self.N, self.dv), torch.float32)}

    def forward(self, h, ctx, cache, add_to=None):
        inner, GN = self.inner, self.G * self.N
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)                     # [z | x B C | dt]
        xbc = ops.causal_conv(proj[:, inner:inner + self.channels], self.w_conv, self.conv_bias, cache.state["tail"],
                              ctx, torch.float32, activation="silu")
        y = ops.linear_recurrence(xbc[:, inner + GN:], xbc[:, inner:inner + GN], xbc[:, :inner], None, None, 1.0, 1.0,
                                  cache.state["S"], ctx, self.P, self.N, self.dv, heads_per_group=self.P // self.G,
                                  dt_raw=proj[:, inner + self.channels:], dt_bias=self.dt_bias, a_log=self.a_log,
                                  skip=self.skip, chunked=self.env.dtype == torch.bfloat16,
                                  wide_state=self.env.dtype == torch.float32)
        g = ops.gate_group_norm(y.view(-1, inner), proj[:, :inner], self.norm_w, self.norm_groups, self.eps, self.env.dtype)
        return ops.linear_parts(g, self.w_o, ctx.err)
