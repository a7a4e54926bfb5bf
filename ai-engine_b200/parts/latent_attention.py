"""Attention whose cache holds one compressed vector per token.

Per token the layer projects a latent c [kv_rank] (RMS-normalised with a weight) and one rotated key part
kr [rot_dim] that all heads share; only [c | kr] is cached.  Head h has the key [W_uk,h c | kr] and the
value W_uv,h c, and a query [q_plain,h | q_rot,h]; score = (q_plain . W_uk c + q_rot . kr) * scale, softmax
over the keys the mask shows (all earlier ones, or the last `window`), output W_o on the concatenated heads.

The up-projections never touch the cache: W_uk is folded into the query (qa_h = W_uk,h^T q_plain,h, so
qa_h . c = q_plain,h . W_uk,h c) and W_uv is applied to the attention-weighted sum of latents
(sum_j p_j W_uv c_j = W_uv sum_j p_j c_j).  The attention kernel then reads the cache rows as they are, as
one key/value head for all query heads, for prompts and decoded tokens alike.

A layer may read another layer's cache (`shares_cache`): it has no latent projection of its own and writes
nothing; the run order names the layer whose rows it reads.
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import KVRequest, Mixer, StepPlanner


class LatentWork(StepPlanner):
    """The work list of the tensor-core kernel: `tiles` [n, 2] = (request row, offset among the tokens it brings)
    of units of `tq` consecutive tokens of one request, which share the cache rows they gather.  A step in which
    every request brings one token has units of one token, all others units of four."""

    key = "latent"

    def plan(self, ctx):
        tq = 1 if ctx.max_q_len <= 1 else 4
        tiles = [(r, off) for r, n in enumerate(ctx.h_q_len.tolist()) for off in range(0, n, tq)]
        return dict(tiles=np.asarray(tiles, dtype=np.int32).reshape(-1, 2)), dict(tq=tq)


LATENT_WORK = LatentWork()


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (unrotated part), rot_dim, value_dim, kv_rank, scale, window
    (0 = all keys), cache_window (the window the cached rows must outlive: the widest of all layers that read
    them; default = window), eps (of the latent's norm), position_encoding (name of an interleaved rotary
    encoding over rot_dim or fewer elements), shares_cache.  tensors: q [H (d + rot), hidden], dkv [kv_rank +
    rot, hidden], dkv_norm [kv_rank], uk [H d, kv_rank], uv [H dv, kv_rank], o [hidden, H dv]."""

    adds_in_place = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.H = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.rot, self.dv, self.rank = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window") or 0)
        self.cache_window = int(p["cache_window"]) if p.get("cache_window") is not None else self.window
        self.eps = float(p["eps"])
        self.shares_cache = bool(p.get("shares_cache"))
        pe = p.get("position_encoding")
        self.rope = env.position_encodings[pe] if pe else None
        if self.rope is not None:
            if not getattr(self.rope, "interleaved", False):
                raise ValueError("latent attention rotates interleaved pairs: its encoding needs layout=interleaved")
            if self.rope.rot_dim > self.rot:
                raise ValueError("latent attention: the rotation is wider than rot_dim")
        self.w_in = self.w_ukT = self.w_uv = self.w_o = self.c_weight = self._no_rope = None

    def tensor_specs(self):
        t, dq = self.spec.tensors, self.d + self.rot
        specs = [TensorSpec(t["q"], (self.H * dq, self.hidden))]
        if not self.shares_cache:
            specs += [TensorSpec(t["dkv"], (self.rank + self.rot, self.hidden)),
                      TensorSpec(t["dkv_norm"], (self.rank,), init="ones")]
        return specs + [TensorSpec(t["uk"], (self.H * self.d, self.rank)),
                        TensorSpec(t["uv"], (self.H * self.dv, self.rank)),
                        TensorSpec(t["o"], (self.hidden, self.H * self.dv))]

    def load(self, source):
        t = self.spec.tensors
        q = source.get(t["q"])
        if self.shares_cache:
            self.w_in = q
        else:
            dkv = source.get(t["dkv"])
            dt = torch.float32 if torch.float32 in (q.dtype, dkv.dtype) else q.dtype
            self.w_in = torch.cat([q.to(dt), dkv.to(dt)], dim=0).contiguous()
            self.c_weight = source.get(t["dkv_norm"]).float().contiguous()
        # [H, kv_rank, d]: the folding product reads W_uk,h transposed
        self.w_ukT = source.get(t["uk"]).view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_uv = source.get(t["uv"]).view(self.H, self.dv, self.rank).contiguous()
        self.w_o = source.get(t["o"])
        self._no_rope = torch.zeros(0, dtype=torch.float32, device=self.env.device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_ukT, self.w_uv, self.w_o))

    def flops(self, tokens, keys=0.0):
        if self.window:
            keys = min(keys, float(self.window))
        proj = 2.0 * tokens * (self.w_in.shape[0] * self.hidden + self.H * self.dv * self.hidden
                               + self.H * self.rank * (self.d + self.dv))
        return proj + 2.0 * tokens * keys * self.H * (2 * self.rank + self.rot)

    def cache_request(self):
        return KVRequest(1, self.rank + self.rot, self.cache_window, planes=1)

    def step_planner(self):
        return LATENT_WORK

    def forward(self, h, ctx, cache, add_to=None):
        T = h.shape[0]
        rot = self.rope.rotation() if self.rope is not None else None
        inv_freq = rot[0] if rot is not None else self._no_rope
        proj = ops.linear(h, self.w_in, torch.float32, ctx.err)
        q_plain, q_full = ops.latent_prepare(proj, self.H, self.d, self.rot, self.rank, self.c_weight, self.eps,
                                             inv_freq, cache.k_pages, ctx, cache.block_table, self.env.dtype,
                                             write=cache.writes and not self.shares_cache)
        ops.head_linear(q_plain, self.w_ukT, q_full)
        mixed = ops.latent_attention(q_full, cache.k_pages, ctx, cache.block_table, self.rank, self.scale,
                                     self.window, self.env.dtype, ctx.plan(LATENT_WORK))
        a = torch.empty((T, self.H, self.dv), dtype=self.env.dtype, device=h.device)
        ops.head_linear(mixed, self.w_uv, a)
        a = a.view(T, self.H * self.dv)
        if add_to is not None and ops.linear_add(add_to, a, self.w_o):
            return None
        return ops.linear_parts(a, self.w_o, ctx.err)
