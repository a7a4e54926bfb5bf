"""A plain, slow restatement of the Zupitar design, one function per mechanism, in torch on the CPU.

It shares nothing with the engine: it reads a dict of tensors by name and the raw config.json dict, runs a
whole sequence (or continues one from a `State`), and returns logits for every token.  Everything is
computed in the dtype the caller asks for (float64 by default).

Notation: T tokens, D = width; attention: H query heads, K key/value heads, d per-head size; state-space
mixer: P heads of dv channels, N state rows, G groups.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---------------------------------------------------------------------------------------------------
# token-local pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gated_ff(h, w_gate, w_up, w_down, act):
    return (act(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def route(h, w_router, correction, top, group_count, group_keep, margins=None):
    """(chosen expert ids [T, top], weights [T, top]).  Scores are a softmax over all router outputs; the choice
    is made on score + correction among the members of the `group_keep` groups whose best member is largest;
    the weights are the plain scores of the chosen ones.  `margins`: a list that receives, per token, how far the
    choice is from turning (the last chosen value above the first one left out, for experts and for groups)."""
    s = torch.softmax(h @ w_router.T, dim=-1)
    choice = s + correction
    T, E = s.shape
    per = E // group_count
    best = choice.view(T, group_count, per).max(dim=-1).values             # [T, groups]
    kept = torch.zeros(T, group_count, dtype=torch.bool)
    kept.scatter_(1, best.topk(group_keep, dim=-1).indices, True)
    masked = torch.where(kept.repeat_interleave(per, dim=1), choice, torch.full_like(choice, -math.inf))
    ids = masked.topk(top, dim=-1).indices
    if margins is not None:
        m = torch.full((T,), math.inf, dtype=s.dtype)
        if top < per * group_keep:
            srt = masked.sort(dim=-1, descending=True).values
            m = torch.minimum(m, srt[:, top - 1] - srt[:, top])
        if group_keep < group_count:
            srt = best.sort(dim=-1, descending=True).values
            m = torch.minimum(m, srt[:, group_keep - 1] - srt[:, group_keep])
        margins.append(m)
    return ids, s.gather(1, ids)


def routed_moe(h, w_router, correction, experts, identity, top, group_count, group_keep, margins=None):
    """`experts`: list of (gate, up, down); the router's last `identity` outputs stand for experts that hand
    their input on unchanged."""
    ids, w = route(h, w_router, correction, top, group_count, group_keep, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(ids[t, j])
            y = h[t] if e >= len(experts) else gated_ff(h[t:t + 1], *experts[e], silu)[0]
            out[t] = out[t] + w[t, j] * y
    return out


def causal_conv(u, w, history, bias=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) (+ bias).  u [T, C]; w [C, taps]; `history` [taps - 1, C]: the
    inputs before u's first row (zeros at a sequence's start).  Returns (y, new history)."""
    taps = w.shape[1]
    ext = torch.cat([history, u], dim=0)
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] = y[t] + w[:, j] * ext[t + j]
    if bias is not None:
        y = y + bias
    return y, ext[ext.shape[0] - (taps - 1):].clone()


def rotate_halves(x, positions, base, dims, factor):
    """x [T, heads, d]: element i < dims/2 of each head turns with element i + dims/2 by the angle
    p * base^(-2i/dims) / factor; the elements from `dims` on pass."""
    out = x.clone()
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = base ** (-2.0 * i / dims) / factor
    ang = positions.to(x.dtype)[:, None] * f[None, :]                       # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---------------------------------------------------------------------------------------------------
# mixers
def keyed_attention(h, m, w, st, pos0):
    """Softmax attention whose values are its keys before rotation.  `st`: dict with q_hist, k_hist (conv
    histories) and keys, values (lists of earlier rows)."""
    H, K, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q, st["q_hist"] = causal_conv(h @ w["q"].T, w["q.conv"], st["q_hist"])
    k, st["k_hist"] = causal_conv(h @ w["k"].T, w["k.conv"], st["k_hist"])
    q, k = q.view(T, H, d), k.view(T, K, d)
    v = k.clone()
    pos = torch.arange(pos0, pos0 + T)
    rot = m.get("rot")
    if rot and rot.get("dims", 0) > 0:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_halves(q, pos, float(rot["base"]), int(rot["dims"]), factor)
        k = rotate_halves(k, pos, float(rot["base"]), int(rot["dims"]), factor)
    st["keys"] = torch.cat([st["keys"], k], dim=0)
    st["values"] = torch.cat([st["values"], v], dim=0)
    keys, values = st["keys"], st["values"]
    out = torch.zeros(T, H, d, dtype=h.dtype)
    per = H // K
    for t in range(T):
        n = pos0 + t + 1
        for hh in range(H):
            g = hh // per
            sc = (keys[:n, g] @ q[t, hh]) * m["scale"]
            p = torch.softmax(sc, dim=0)
            out[t, hh] = p @ values[:n, g]
    return out.reshape(T, H * d) @ w["o"].T


def state_space(h, m, w, st, eps):
    """The selective state-space mixer with a scalar decay per head.  `st`: dict with hist (conv history of
    x|B|C) and S [P, N, dv]."""
    P, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = P * dv, h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc, st["hist"] = causal_conv(xbc, w["conv"], st["hist"], w["conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].view(T, P, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                        # [T, P]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)                          # [T, P]
    y = torch.zeros(T, P, dv, dtype=h.dtype)
    S = st["S"]
    per = P // G
    for t in range(T):
        for p in range(P):
            g = p // per
            S[p] = decay[t, p] * S[p] + dt[t, p] * torch.outer(B[t, g], x[t, p])
            y[t, p] = S[p].T @ C[t, g] + w["D"][p] * x[t, p]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


# ---------------------------------------------------------------------------------------------------
class State:
    """What a sequence carries from one call to the next."""

    def __init__(self, cfg, dtype):
        self.pos = 0
        self.layers = []
        for l in cfg["layers"]:
            m = l["mixer"]
            s = {}
            if l["type"] == "parallel":
                s["left"] = self._attn(m["left"], dtype)
                s["right"] = self._ssm(m["right"], dtype)
            else:
                s = self._ssm(m, dtype)
            self.layers.append(s)

    @staticmethod
    def _attn(m, dtype):
        return dict(q_hist=torch.zeros(m["conv"] - 1, m["heads"] * m["dim"], dtype=dtype),
                    k_hist=torch.zeros(m["conv"] - 1, m["kv_heads"] * m["dim"], dtype=dtype),
                    keys=torch.zeros(0, m["kv_heads"], m["dim"], dtype=dtype),
                    values=torch.zeros(0, m["kv_heads"], m["dim"], dtype=dtype))

    @staticmethod
    def _ssm(m, dtype):
        ch = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
        return dict(hist=torch.zeros(m["conv"] - 1, ch, dtype=dtype),
                    S=torch.zeros(m["heads"], m["state"], m["vdim"], dtype=dtype))


def _sub(tensors, prefix, dtype):
    n = len(prefix)
    return {k[n:]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64,
            state: Optional[State] = None, layers_out: Optional[list] = None,
            margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [len(ids), vocab] of the tokens `ids`, continuing `state` when given (it is updated).  `layers_out`
    receives the stream after every layer, `margins_out` every router's margins (see `route`)."""
    st = state if state is not None else State(cfg, dtype)
    eps = float(cfg["norm"]["eps"])
    W = lambda name: tensors[name].to(dtype)
    x = W("embed")[torch.tensor(ids, dtype=torch.long)]
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        h = norm(x, W(p + "norm1"), eps)
        if l["type"] == "parallel":
            a = keyed_attention(h, m["left"], _sub(tensors, p + "mix.left.", dtype), st.layers[i]["left"], st.pos)
            b = state_space(h, m["right"], _sub(tensors, p + "mix.right.", dtype), st.layers[i]["right"], eps)
            y = m["left_scale"] * a + m["right_scale"] * b
        elif l["type"] == "mamba2":
            y = state_space(h, m, _sub(tensors, p + "mix.", dtype), st.layers[i], eps)
        else:
            raise ValueError(l["type"])
        x = x + norm(y, W(p + "norm1b"), eps)
        f = l.get("mlp")
        if f is not None:
            h = norm(x, W(p + "norm2"), eps)
            if f["kind"] == "dense":
                y = gated_ff(h, W(p + "mlp.gate"), W(p + "mlp.up"), W(p + "mlp.down"), torch.relu)
            else:
                r = f["router"]
                experts = [(W(f"{p}mlp.e{e}.gate"), W(f"{p}mlp.e{e}.up"), W(f"{p}mlp.e{e}.down"))
                           for e in range(r["experts"])]
                groups = r.get("groups") or dict(count=1, keep=1)
                y = routed_moe(h, W(p + "mlp.router"), W(p + "mlp.correction"), experts, r.get("identity", 0),
                               r["top"], groups["count"], groups["keep"], margins_out)
            x = x + norm(y, W(p + "norm2b"), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    st.pos += len(ids)
    logits = norm(x, W("final.norm"), eps) @ W("head").T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
