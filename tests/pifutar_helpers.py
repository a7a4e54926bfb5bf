"""Shared by the Pifutar tests: small configurations (none has the sizes of a published model; between them
every size, count and constant differs, some are 1), model folders with random weights, the plain
implementation as oracle, and tolerances relative to the spread of the logits."""
from __future__ import annotations

import os

import numpy as np
import torch

import plain_pifutar as pp


def _latent(heads, dim, rot_dim, vdim, rank, window=None, base=10000.0, dims=None, kv_from=None, scale=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank,
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5,
             rot=dict(base=base, dims=rot_dim if dims is None else dims))
    if window:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _moe(experts, top, ff, limit, shared=None):
    f = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))
    if shared:
        f["shared"] = dict(ff=shared[0], limit=shared[1])
    return f


def _with(layer, mlp):
    return dict(layer, mlp=mlp)


# every kind of layer; a latent cache of 72 elements a row (the plain attention kernel), experts of 40 (the float32
# grouped product), two windows on one cache, a layer without feed-forward, an expert count of 1 with top 1
CFG_X = dict(architecture="Pifutar", vocab=211, width=96, norm=dict(eps=1e-4), canon=dict(taps=4), layers=[
    _with(dict(type="gla", mixer=dict(heads=3, dim=24, vdim=40, tau=8.0)), dict(kind="dense", ff=160)),
    _with(_latent(5, 32, 8, 48, 64, window=24), _moe(6, 3, 40, 1.5, (56, 0.8))),
    _with(dict(type="retention", mixer=dict(heads=2, dim=16, vdim=24, decay=[0.9, 0.96875])), None),
    _with(_latent(3, 16, 8, 24, 64, window=17, kv_from=1), _moe(1, 1, 24, 3.0)),
    _with(_latent(2, 40, 12, 16, 48, dims=8, base=500.0), _moe(5, 2, 32, 0.7, (16, 2.0))),
    _with(_latent(5, 32, 8, 48, 64, window=9, kv_from=1), dict(kind="dense", ff=72)),
])

# no attention layer at all (no pages, state only), two taps, heads of odd sizes
CFG_Y = dict(architecture="Pifutar", vocab=130, width=128, norm=dict(eps=1e-6), canon=dict(taps=2), layers=[
    _with(dict(type="retention", mixer=dict(heads=5, dim=36, vdim=20, decay=[0.5, 0.75, 0.875, 0.9375, 0.99])),
          _moe(4, 2, 64, 2.5, (128, 1.0))),
    _with(dict(type="gla", mixer=dict(heads=1, dim=160, vdim=32, tau=4.0)), dict(kind="dense", ff=96)),
    _with(dict(type="retention", mixer=dict(heads=2, dim=8, vdim=136, decay=[1.0, 0.3])), None),
])

# the sizes the tensor-core kernels take in bfloat16: a latent of 128 with rows of 144 under 20 heads (two groups of
# 16, the second partly empty), experts of 64 on a width of 128 (the grouped tcgen05 product), one tap
CFG_Z = dict(architecture="Pifutar", vocab=257, width=128, norm=dict(eps=1e-5), canon=dict(taps=1), layers=[
    _with(_latent(20, 16, 16, 8, 128, window=70), _moe(9, 2, 64, 2.0, (64, 1.0))),
    _with(_latent(4, 48, 16, 64, 128, kv_from=0), _moe(3, 3, 128, 1.0)),
    _with(dict(type="gla", mixer=dict(heads=2, dim=64, vdim=64, tau=16.0)), dict(kind="dense", ff=256)),
    _with(_latent(8, 24, 32, 32, 64, dims=32, base=1000000.0), None),
])

CONFIGS = {"X": CFG_X, "Y": CFG_Y, "Z": CFG_Z}


def make_dir(tmp_path, name, seed=0, gain=4.0):
    """A model folder for configuration `name`: random weights N(0, 0.07) written by the engine's random-weights
    mode, norm weights N(0, 0.1) around zero, and the query projections of attention layers multiplied by
    `gain` so that scores spread and single keys stand out."""
    import ai_engine_b200 as aie
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"pifutar_{name}_{seed}_{gain}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    aie.write_random_model(aie.PifutarConfig.from_dict(CONFIGS[name]), d, seed=seed, std=0.07, norm_std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = {}
    with safe_open(path, "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith("mix.q") and gain != 1.0 and CONFIGS[name]["layers"][int(k[1:k.index(".")])]["type"] == "latent_attention":
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


def plain_logits(d, name, ids, dtype=torch.float64):
    """[len(ids), vocab] from the plain implementation (cached per folder and sequence)."""
    key = (d, tuple(ids), dtype)
    if key not in _REFS:
        _REFS[key] = pp.forward(CONFIGS[name], read_tensors(d), ids, dtype=dtype).to(torch.float64).numpy()
    return _REFS[key]


def close(got, ref, dtype, what=""):
    """Logits agree within rounding.  The float32 engine against the float64 oracle: 2e-4 of the logits' spread at
    every element.  bfloat16 against the float32 oracle on the same weights: these models are a few layers of
    cubes, clamps and normalised states on random weights, where rounding to 8 bits of mantissa at every product's
    input moves single logits by up to a tenth of the spread; the worst element may differ by 0.2 of the spread
    and the mean difference must stay under 0.03 of it (a wrong key, window or state moves whole rows by the
    spread itself)."""
    spread = max(float(np.std(ref)), 1e-3)
    diff = np.abs(np.asarray(got, dtype=np.float64) - ref)
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
