"""Pifutar configurations drawn at random (layer kinds in any order, sizes that are no multiples of 8 or 16, windows
or none, layers that read an earlier layer's cache, with and without feed-forward, shared expert or none, 1 to 5
taps): each is written with random weights, fed whole, in portions and beside a second request through the engine,
and compared with the plain implementation, in float32 and bfloat16."""
import os

import numpy as np
import pytest
import torch

import plain_pifutar as pp
from pifutar_helpers import close, ids_for, oracle_dtype, read_tensors

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.RandomState(1000 + seed)
    pick = lambda xs: xs[int(rng.randint(len(xs)))]
    width = int(pick([40, 72, 104, 136, 200]))
    n_layers = int(rng.randint(2, 7))
    layers, own = [], []          # own: latent layers with a cache of their own
    for i in range(n_layers):
        kind = pick(["latent_attention", "latent_attention", "retention", "gla"])
        if kind == "latent_attention":
            heads, dim, rot_dim = int(rng.randint(1, 10)), int(pick([8, 12, 16, 24, 40])), int(pick([4, 8, 16, 24]))
            rank = int(pick([24, 40, 64, 96, 128, 192]))
            m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=int(pick([8, 20, 32, 48])), kv_rank=rank,
                     scale=float((dim + rot_dim) ** -0.5 * pick([1.0, 0.7])),
                     rot=dict(base=float(pick([100.0, 10000.0, 500000.0])), dims=int(pick([rot_dim, rot_dim, rot_dim // 2 * 2 - 2 or 2]))))
            if rng.rand() < 0.7:
                m["mask"] = dict(size=int(rng.randint(1, 50)))
            if own and rng.rand() < 0.4:
                j = int(pick(own))
                src = layers[j]["mixer"]
                m.update(kv_from=j, kv_rank=src["kv_rank"], rot_dim=src["rot_dim"], rot=dict(src["rot"]))
                m["scale"] = float((dim + m["rot_dim"]) ** -0.5)
            else:
                own.append(i)
        elif kind == "retention":
            heads = int(rng.randint(1, 7))
            m = dict(heads=heads, dim=int(pick([4, 12, 32, 36, 130])), vdim=int(pick([4, 20, 64, 100])),
                     decay=[float(1.0 - 2.0 ** -rng.randint(1, 9)) for _ in range(heads)])
        else:
            m = dict(heads=int(rng.randint(1, 5)), dim=int(pick([8, 20, 48, 64])), vdim=int(pick([8, 24, 36, 128])),
                     tau=float(pick([1.0, 4.0, 16.0, 64.0])))
        r = rng.rand()
        if r < 0.15:
            mlp = None
        elif r < 0.4:
            mlp = dict(kind="dense", ff=int(pick([24, 50, 128, 200])))
        else:
            experts = int(rng.randint(1, 13))
            mlp = dict(kind="moe", expert=dict(ff=int(pick([8, 30, 64, 128])), limit=float(pick([0.5, 2.0, 7.0]))),
                       router=dict(experts=experts, top=int(rng.randint(1, min(experts, 4) + 1))))
            if rng.rand() < 0.6:
                mlp["shared"] = dict(ff=int(pick([16, 44, 96])), limit=float(pick([1.0, 3.0])))
        layers.append(dict(type=kind, mixer=m, mlp=mlp))
    return dict(architecture="Pifutar", vocab=int(rng.randint(50, 400)), width=width,
                norm=dict(eps=float(pick([1e-6, 1e-5, 1e-3]))), canon=dict(taps=int(rng.randint(1, 6))), layers=layers)


def folder(tmp_path, raw, seed):
    import ai_engine_b200 as aie
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"drawn{seed}")
    aie.write_random_model(aie.PifutarConfig.from_dict(raw), d, seed=seed, std=0.08, norm_std=0.1)
    t = {k: v.clone() for k, v in read_tensors(d).items()}       # copies: the file is written again below
    for k in list(t):          # attention scores that spread
        if k.endswith("mix.q") and raw["layers"][int(k[1:k.index(".")])]["type"] == "latent_attention":
            t[k] = (t[k].float() * 3.0).to(t[k].dtype)
    save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(d, "model.safetensors"))
    return d, t


def steady_rows(raw, t, ids, ref):
    """Rows at which the model itself is well conditioned: a drawn model can make q . k of a head vanish at a
    token (most often a sequence's first, where the state holds one key), and the normalised output of that head
    then turns on the last bits of its inputs.  The oracle is run twice more with every matrix nudged by noise of
    half a bfloat16 step; rows that move by more than 0.1 of the logits' spread are left out of the bfloat16
    comparison (never more than half of them), all rows stay in the float32 one."""
    g = torch.Generator().manual_seed(0)
    moved = np.zeros(len(ids))
    for _ in range(2):
        t2 = {k: (v.double() * (1 + 2.0 ** -9 * torch.randn(v.shape, generator=g, dtype=torch.float64))
                  if v.is_floating_point() and v.dim() == 2 else v) for k, v in t.items()}
        out = pp.forward(raw, t2, ids, dtype=torch.float64).numpy()
        moved = np.maximum(moved, np.abs(out - ref).max(1) / max(float(ref.std()), 1e-3))
    keep = moved <= 0.1
    assert keep.sum() >= len(ids) / 2, f"the drawn model is ill-conditioned at {int((~keep).sum())} of {len(ids)} rows"
    return keep


@pytest.mark.parametrize("seed", range(24))
def test_a_drawn_configuration(tmp_path, seed):
    from ai_engine_b200.engine.replay import Replayer

    raw = draw(seed)
    d, t = folder(tmp_path, raw, seed)
    a, b = ids_for(70, raw["vocab"], seed), ids_for(26, raw["vocab"], 100 + seed)
    for dtype in ("float32", "bfloat16"):
        ref_a = pp.forward(raw, t, a, dtype=oracle_dtype(dtype)).double().numpy()
        ref_b = pp.forward(raw, t, b, dtype=oracle_dtype(dtype)).double().numpy()
        ka = kb = slice(None)
        if dtype == "bfloat16":
            ka, kb = steady_rows(raw, t, a, ref_a), steady_rows(raw, t, b, ref_b)
        rep = Replayer(d, dtype, max_tokens=192, block_size=int([8, 16, 32][seed % 3]))
        whole = rep.run_step([dict(id="w", tokens=a, want=list(range(70)))], end=["w"]).numpy()
        close(whole[ka], ref_a[ka], dtype, f"drawn {seed} whole {raw['layers']}")
        # in portions, with a second request beside it that starts later and ends earlier
        got_a, got_b, fa, fb = [], [], 0, 0
        for k, n in enumerate([9, 2, 17, 1, 1, 30, 3, 7]):
            entries = [dict(id="a", tokens=a[fa:fa + n], want=list(range(n)))]
            if 1 <= k <= 4:
                m = [5, 1, 18, 2][k - 1]
                entries.insert(0, dict(id="b", tokens=b[fb:fb + m], want=list(range(m))))
            out = rep.run_step(entries, end=["b"] if k == 4 else []).numpy()
            if len(entries) == 2:
                got_b.append(out[:m]); out = out[m:]; fb += m
            got_a.append(out); fa += n
        close(np.concatenate(got_a)[ka], ref_a[ka], dtype, f"drawn {seed} in portions")
        close(np.concatenate(got_b)[kb], ref_b[kb], dtype, f"drawn {seed} the request beside it")
