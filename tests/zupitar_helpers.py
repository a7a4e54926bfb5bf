"""Shared by the Zupitar tests: small configurations (none has the sizes of a published model; between them every
size, count and constant differs, some are 1 or equal where the others differ), model folders with random weights,
the plain implementation as oracle, a rig that steps one part on a real cache, and tolerances relative to the
spread of the logits."""
from __future__ import annotations

import os

import numpy as np
import torch

import plain_zupitar as pz


def _attn(heads, kv_heads, dim, conv, scale=None, rot=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, conv=conv, scale=scale if scale is not None else dim ** -0.5)
    if rot is not None:
        base, dims, factor = rot
        m["rot"] = dict(base=base, dims=dims)
        if factor is not None:
            m["rot"]["scaling"] = dict(factor=factor)
    return m


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def _par(left, right, ls, rs, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs), mlp=mlp)


def _moe(ff, experts, identity, top, count=None, keep=None):
    r = dict(experts=experts, top=top)
    if identity:
        r["identity"] = identity
    if count is not None:
        r["groups"] = dict(count=count, keep=keep)
    return dict(kind="moe", expert=dict(ff=ff), router=r)


# every kind of layer and feed-forward; odd sizes; a partial rotation with stretched positions; three groups of router
# outputs of which two are kept; a layer without rotation, with one tap and as many key heads as query heads; a layer
# without feed-forward; a router without groups, identity experts or a second choice
CFG_A = dict(architecture="Zupitar", vocab=211, width=96, norm=dict(eps=1e-4), logit_softcap=10.0, layers=[
    _par(_attn(6, 2, 32, 3, scale=0.21, rot=(1000.0, 16, 2.0)), _ssm(4, 24, 16, 2, 4, 2), 0.7, 1.3, _moe(40, 5, 1, 2, 3, 2)),
    dict(type="mamba2", mixer=_ssm(3, 40, 24, 1, 2, 3), mlp=dict(kind="dense", ff=80)),
    _par(_attn(3, 3, 16, 1), _ssm(6, 8, 40, 6, 1, 1), 1.0, 0.5, None),
    dict(type="mamba2", mixer=_ssm(2, 36, 8, 2, 3, 1), mlp=_moe(24, 3, 0, 1)),
])

# the sizes the tensor-core kernels take in bfloat16: heads of 64 and 128, experts of 128 on a width of 128 (the grouped
# tcgen05 product), a full rotation without stretching, no bound on the logits, more identity experts than real ones in a group
CFG_B = dict(architecture="Zupitar", vocab=257, width=128, norm=dict(eps=1e-5), layers=[
    _par(_attn(4, 1, 64, 2, rot=(10000.0, 64, None)), _ssm(4, 32, 64, 4, 2, 1), 1.1, 0.9, _moe(128, 6, 2, 3, 4, 2)),
    _par(_attn(2, 2, 128, 4, scale=0.05, rot=(500000.0, 32, 8.0)), _ssm(2, 64, 128, 1, 3, 2), 0.6, 0.6, dict(kind="dense", ff=256)),
    dict(type="mamba2", mixer=_ssm(8, 16, 32, 2, 4, 4), mlp=_moe(64, 2, 2, 2, 2, 1)),
])

# no attention at all (no pages, only slots); a width that is no multiple of 8; only identity experts in one router
CFG_C = dict(architecture="Zupitar", vocab=130, width=36, norm=dict(eps=1e-6), logit_softcap=4.0, layers=[
    dict(type="mamba2", mixer=_ssm(5, 12, 20, 5, 2, 5), mlp=_moe(16, 0, 3, 2)),
    dict(type="mamba2", mixer=_ssm(1, 44, 12, 1, 5, 2), mlp=dict(kind="dense", ff=52)),
    dict(type="mamba2", mixer=_ssm(4, 9, 4, 2, 3, 1), mlp=None),
])

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C}


def make_dir(tmp_path, name, seed=0, gain=4.0):
    """A model folder for configuration `name`: random weights N(0, 0.07) written by the engine's random-weights
    mode, norm weights 1 + N(0, 0.1), and the query projections of attention multiplied by `gain` so that scores
    spread and single keys stand out."""
    import ai_engine_b200 as aie
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"zupitar_{name}_{seed}_{gain}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    aie.write_random_model(aie.ZupitarConfig.from_dict(CONFIGS[name]), d, seed=seed, std=0.07, norm_std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = {}
    with safe_open(path, "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith("mix.left.q") and gain != 1.0:
                t = (t.float() * gain).to(t.dtype)
            tensors[k] = t.clone().contiguous()          # a copy: the file is written again below
    save_file(tensors, path)
    return d


def read_tensors(d):
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(d, "model.safetensors"), "pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


_REFS = {}


CLEAR = 0.03     # a router's choice stands when its last chosen value leads the first one left out by this much
AFTER = 6        # a choice that turned moves the rows behind it too (convolution tails, states), fading with distance


class Ref(np.ndarray):
    """Logits [tokens, vocab] with `clear` [tokens]: whether the router choices of the token and of the AFTER tokens
    before it are all far from turning (always true without routers).  Slicing rows keeps the flags of those rows."""

    def __new__(cls, logits, clear):
        obj = np.asarray(logits).view(cls)
        obj.clear = np.asarray(clear)
        return obj

    def __array_finalize__(self, obj):
        self.clear = getattr(obj, "clear", None)

    def __getitem__(self, item):
        out = super().__getitem__(item)
        if isinstance(out, Ref) and self.clear is not None and not isinstance(item, tuple):
            out.clear = self.clear[item]
        return out


def plain_logits(d, name, ids, dtype=torch.float64):
    """[len(ids), vocab] from the plain implementation, with the rows whose routing is clear (cached per folder and
    sequence)."""
    key = (d, tuple(ids), dtype)
    if key not in _REFS:
        margins = []
        logits = pz.forward(CONFIGS[name], read_tensors(d), ids, dtype=dtype, margins_out=margins).to(torch.float64).numpy()
        m = torch.stack(margins).min(dim=0).values.double().numpy() if margins else np.full(len(ids), np.inf)
        ok = m >= CLEAR
        clear = np.array([bool(ok[max(0, i - AFTER):i + 1].all()) for i in range(len(ids))])
        _REFS[key] = Ref(logits, clear)
    return _REFS[key]


def close(got, ref, dtype, what=""):
    """Logits agree within rounding.  The float32 engine against the float64 oracle: 2e-4 of the logits' spread at
    every element.  bfloat16 against the float32 oracle on the same weights: a router's close call may turn either
    way under rounding, and then the row (and, fading, the next ones) is another expert's.  So over all rows the
    median of the rows' worst differences must stay under 0.12 of the spread and nine rows in ten under 0.2 (a wrong
    key, state or expert moves every row by the spread itself), and at the rows whose routing is clear the worst element may differ by 0.2 of
    the spread and the mean difference must stay under 0.03 of it."""
    spread = max(float(np.std(ref)), 1e-3)
    diff = np.abs(np.asarray(got, dtype=np.float64) - np.asarray(ref))
    if dtype != "float32":
        if diff.shape[0] >= 8:
            med = float(np.median(diff.max(axis=-1)))
            assert med <= 0.12 * spread, f"{what}: median row difference {med:.3e} above {0.12 * spread:.3e}"
        if diff.shape[0] >= 100:
            p90 = float(np.percentile(diff.max(axis=-1), 90))
            assert p90 <= 0.2 * spread, f"{what}: nine rows in ten must be within {0.2 * spread:.3e}, are within {p90:.3e}"
        if getattr(ref, "clear", None) is not None:
            diff = diff[ref.clear]
            if diff.size == 0:
                return 0.0
    err = float(diff.max())
    tol = (2e-4 if dtype == "float32" else 0.2) * spread
    assert err <= tol, f"{what}: max difference {err:.3e} above {tol:.3e}"
    if dtype != "float32":
        assert float(diff.mean()) <= 0.03 * spread, f"{what}: mean difference {diff.mean():.3e} above {0.03 * spread:.3e}"
    return err


def oracle_dtype(dtype):
    return torch.float64 if dtype == "float32" else torch.float32


def ids_for(n, vocab, seed):
    return np.random.RandomState(seed).randint(0, vocab, size=n).tolist()


# ---------------------------------------------------------------------------------------------------
DEV = "cuda"


def env(dtype, hidden, encodings=None):
    from ai_engine_b200.parts import BuildEnv
    e = BuildEnv(hidden, dtype, torch.device(DEV))
    for k, v in (encodings or {}).items():
        e.position_encodings[k] = v
    return e


def load(part, tensors, dtype):
    from ai_engine_b200.weights import from_tensors
    part.load(from_tensors(tensors, part.tensor_specs(), dtype, DEV))
    return part


class Rig:
    """One part (with the parts it is made of) on a cache of its own (pages and state as it asks) and steps made by
    the engine's step context."""

    def __init__(self, part, dtype, page=8, pages=64, max_seqs=4):
        from ai_engine_b200.cache import PagedCache
        from ai_engine_b200.parts import CacheNeed
        from ai_engine_b200.parts.base import walk_named
        self.part = part
        needs = [CacheNeed(0, role, p.cache_request(), p.state_request()) for role, p in walk_named("p", part)
                 if p.cache_request() is not None or p.state_request() is not None]
        self.cache = PagedCache(needs, page, pages, max_seqs, 4096, dtype, DEV)
        self.err = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.have = {}
        planner = part.step_planner()
        self.planners = (planner,) if planner is not None else ()

    def admit(self):
        s = self.cache.admit()
        assert s >= 0
        self.have[s] = 0
        return s

    def finish(self, slot):
        self.cache.finish(slot)
        del self.have[slot]

    def step(self, portions):
        """portions: [(slot, n tokens)]; returns (ctx, the part's LayerCache)."""
        from ai_engine_b200.engine.step import StepContext, StepEntry
        entries = []
        for slot, n in portions:
            assert self.cache.ensure(slot, self.have[slot] + n)
            entries.append(StepEntry(slot, self.have[slot], [0] * n, []))
        ctx = StepContext(entries, self.cache, torch.device(DEV), self.err, planners=self.planners)
        return ctx, self.cache.layer_cache(0, ctx).get("p")

    def done(self, portions):
        for slot, n in portions:
            self.have[slot] += n
            self.cache.advance(slot, self.have[slot])
        assert int(self.err.item()) == 0

    def run(self, seqs, cuts):
        """Feed the rows `seqs[k]` [n_k, hidden] of request k in portions `cuts[k]`, all requests side by side (a
        request whose portions are used up sits out); returns the part's float64 outputs per request."""
        slots = [self.admit() for _ in seqs]
        at = [0] * len(seqs)
        got = [[] for _ in seqs]
        for k in range(max(len(c) for c in cuts)):
            portions, rows, who = [], [], []
            for r, c in enumerate(cuts):
                if k < len(c):
                    portions.append((slots[r], c[k]))
                    rows.append(seqs[r][at[r]:at[r] + c[k]])
                    at[r] += c[k]
                    who.append(r)
            ctx, lc = self.step(portions)
            out = self.part.forward(torch.cat(rows).to(DEV), ctx, lc)
            out = out.double()
            out = (out.sum(0) if out.dim() == 3 else out).cpu()
            o = 0
            for r, (slot, n) in zip(who, portions):
                got[r].append(out[o:o + n])
                o += n
            self.done(portions)
        for r, s in enumerate(seqs):
            assert at[r] == len(s)
        for s in slots:
            self.finish(s)
        return [torch.cat(g) for g in got]
