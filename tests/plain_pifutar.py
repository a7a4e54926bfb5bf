"""A plain, slow restatement of the Pifutar design, one function per mechanism, in torch on the CPU.

It shares nothing with the engine: it reads a dict of tensors by name and the raw config.json dict, runs a
whole sequence (or continues one from a `State`), and returns logits for every token.  Everything is
computed in the dtype the caller asks for (float64 by default).

Notation: T tokens, D = width, H heads; d = per-head key size, dv = per-head value size.
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


def norm_zero_centred(x, w, eps):
    """RMS norm whose stored weight is the offset from one."""
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def polynorm(z, coef, eps):
    """coef = (a, b, c, e): a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean square."""
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z ** 3, eps) + e


def dense_ff(h, w_up, w_down, coef, eps):
    return polynorm(h @ w_up.T, coef, eps) @ w_down.T


def clamped_expert(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def table_moe(h, token_ids, table, experts, limit, shared=None):
    """Experts chosen by the token's id through `table` [vocab, top]; each weighs 1/top.  `experts`:
    list of (gate, up, down).  `shared`: (gate, up, down, sg, limit) or None."""
    top = table.shape[1]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for s in range(top):
            e = int(table[int(token_ids[t]), s])
            out[t] += clamped_expert(h[t:t + 1], *experts[e], limit)[0] / top
    if shared is not None:
        g, u, d, sg, lim = shared
        out = out + clamped_expert(h, g, u, d, lim) * torch.sigmoid(h @ sg.T)
    return out


def short_conv(h, w, history):
    """h + causal convolution of h over time, per channel.  w [D, taps]; `history` [taps - 1, D]: the
    inputs before h's first row (zeros at a sequence's start).  Returns (result, new history)."""
    taps = w.shape[1]
    ext = torch.cat([history, h], dim=0)                  # row t + taps - 1 is h[t]
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * ext[t + j]                # ext[t + j] = h[t - taps + 1 + j]
    return out, ext[ext.shape[0] - (taps - 1):].clone()


def rotate_interleaved(x, positions, base, dims):
    """Pairs (2i, 2i+1) of the first `dims` elements of the last axis turn by p * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = base ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]       # [T, dims/2]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * torch.cos(a) - v * torch.sin(a)
    out[..., 1:dims:2] = v * torch.cos(a) + u * torch.sin(a)
    return out


# ---------------------------------------------------------------------------------------------------
# mixers; each takes h [T, D] of one sequence, the positions of its rows and the state so far
def latent_attention(h, positions, W, m, eps, kv):
    """m: the mixer's config dict.  W: tensors by short name (q, dkv, dkv.norm, uk, uv, o).  kv: dict with
    'c' [n, kv_rank] and 'kr' [n, rot_dim] of all earlier tokens, extended here unless W has no 'dkv'
    (then kv already holds this step's rows too, written by the layer it borrows from)."""
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ W["q"].T).view(T, H, d + dr)
    q_rot = rotate_interleaved(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"])
    if "dkv" in W:
        z = h @ W["dkv"].T
        c = rms(z[:, :rank], eps) * W["dkv.norm"]
        kr = rotate_interleaved(z[:, rank:], positions, m["rot"]["base"], m["rot"]["dims"])
        kv["c"] = torch.cat([kv["c"], c]) if kv.get("c") is not None else c
        kv["kr"] = torch.cat([kv["kr"], kr]) if kv.get("kr") is not None else kr
    c_all, kr_all = kv["c"], kv["kr"]
    n = c_all.shape[0]
    k = (c_all @ W["uk"].T).view(n, H, d)
    v = (c_all @ W["uv"].T).view(n, H, dv)
    scale = m.get("scale", (d + dr) ** -0.5)
    window = (m.get("mask") or {}).get("size", 0)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        s = (torch.einsum("hd,jhd->hj", q[t, :, :d], k[lo:p + 1])
             + torch.einsum("hd,jd->hj", q_rot[t], kr_all[lo:p + 1])) * scale
        out[t] = torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[lo:p + 1])
    return out.reshape(T, H * dv) @ W["o"].T


def linear_recurrence(q, k, v, decay, S):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T ; o_t = S_t^T q_t, per head.  q, k [T, H, d]; v [T, H, dv];
    decay [T, H, d] (broadcast for a constant); S [H, d, dv], updated in place."""
    T = q.shape[0]
    o = torch.zeros_like(v)
    for t in range(T):
        S.mul_(decay[t].unsqueeze(-1)).add_(k[t].unsqueeze(-1) * v[t].unsqueeze(-2))
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o


def retention(h, W, m, eps, S):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W["q"].T).view(T, H, d)
    k = (h @ W["k"].T).view(T, H, d) * d ** -0.5
    v = (h @ W["v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype).view(1, H, 1).expand(T, H, d)
    o = rms(linear_recurrence(q, k, v, decay, S), eps)
    g = h @ W["g"].T
    return (o.reshape(T, H * dv) * g * torch.sigmoid(g)) @ W["o"].T


def gated_linear_attention(h, W, m, eps, S):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ W["k"].T).view(T, H, d)
    v = (h @ W["v"].T).view(T, H, dv)
    z = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, d)
    o = rms(linear_recurrence(q, k, v, decay, S), eps) * W["norm"]
    g = h @ W["g"].T
    return (o.reshape(T, H * dv) * g * torch.sigmoid(g)) @ W["o"].T


# ---------------------------------------------------------------------------------------------------
class State:
    """What one sequence carries from token to token: per layer the convolution inputs of both
    sublayers, the latent cache or the recurrent state, and the number of tokens so far."""

    def __init__(self):
        self.n = 0
        self.layers: Dict[int, dict] = {}


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], token_ids, state: Optional[State] = None,
            dtype=torch.float64, streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of `token_ids`, which continue `state` (a fresh sequence when None).
    `streams`, if a list, receives the residual stream after every layer."""
    st = state if state is not None else State()
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    taps = config["canon"]["taps"]
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    T, D = ids.shape[0], config["width"]
    positions = torch.arange(st.n, st.n + T)
    x = W["embed"][ids]
    history = [x]
    for i, layer in enumerate(config["layers"]):
        L = st.layers.setdefault(i, {})
        p = f"l{i}."
        m = layer["mixer"]
        h = norm_zero_centred(x, W[p + "norm1"], eps)
        h, L["conv1"] = short_conv(h, W[p + "canon1"], L.get("conv1", torch.zeros(taps - 1, D, dtype=dtype)))
        mw = _sub(W, p + "mix.")
        if layer["type"] == "latent_attention":
            kv = st.layers[m["kv_from"]]["kv"] if "kv_from" in m else L.setdefault("kv", {})
            a = latent_attention(h, positions, mw, m, eps, kv)
        elif layer["type"] == "retention":
            S = L.setdefault("S", torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dtype))
            a = retention(h, mw, m, eps, S)
        elif layer["type"] == "gla":
            S = L.setdefault("S", torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=dtype))
            a = gated_linear_attention(h, mw, m, eps, S)
        else:
            raise ValueError(layer["type"])
        x = x + a
        ff = layer.get("mlp")
        if ff is not None:
            h = norm_zero_centred(x, W[p + "norm2"], eps)
            h, L["conv2"] = short_conv(h, W[p + "canon2"], L.get("conv2", torch.zeros(taps - 1, D, dtype=dtype)))
            fw = _sub(W, p + "mlp.")
            if ff["kind"] == "dense":
                x = x + dense_ff(h, fw["up"], fw["down"], fw["act"], eps)
            else:
                n_exp = ff["router"]["experts"]
                experts = [(fw[f"e{e}.gate"], fw[f"e{e}.up"], fw[f"e{e}.down"]) for e in range(n_exp)]
                shared = None
                if ff.get("shared"):
                    shared = (fw["shared.gate"], fw["shared.up"], fw["shared.down"], fw["shared.sg"],
                              ff["shared"]["limit"])
                x = x + table_moe(h, ids, fw["table"], experts, ff["expert"]["limit"], shared)
        history.append(x)
        dwa = W[p + "dwa"]
        x = sum(dwa[j] * history[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x.clone())
    st.n += T
    return norm_zero_centred(x, W["final.norm"], eps) @ W["embed"].T
