"""Zupitar configurations drawn at random (both kinds of layer in any order, sizes that are no multiples of 8 or 16,
1 to 5 taps, a rotation that is full, partial or absent with or without stretched positions, groups of heads and of
router outputs, identity experts, with and without feed-forward or bounded logits): each is written with random
weights, fed whole, in portions and beside a second request through the engine, and compared with the plain
implementation, in float32 at every row and in bfloat16 by the rules of `zupitar_helpers.close`."""
import os

import numpy as np
import pytest
import torch

import plain_zupitar as pz
import zupitar_helpers as zh
from zupitar_helpers import close, ids_for, oracle_dtype, read_tensors

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = np.random.RandomState(2000 + seed)
    pick = lambda xs: xs[int(rng.randint(len(xs)))]
    width = int(pick([40, 72, 100, 136, 200]))

    def ssm():
        groups = int(pick([1, 1, 2, 3]))
        heads = groups * int(pick([1, 2, 3]))
        vdim = int(pick([8, 12, 20, 32, 64]))
        # (a part of very few channels divided by its own root mean square turns on the sign of single values)
        norm_groups = int(pick([1] + [g for g in (2, 3, 4, heads) if (heads * vdim) % g == 0 and heads * vdim // g >= 8]))
        return dict(heads=heads, vdim=vdim, state=int(pick([4, 12, 16, 40, 64, 128])), groups=groups,
                    conv=int(rng.randint(1, 6)), norm_groups=norm_groups)

    def attn():
        kv = int(pick([1, 1, 2, 3]))
        dim = int(pick([16, 24, 40, 64, 128]))
        m = dict(heads=kv * int(pick([1, 2, 4])), kv_heads=kv, dim=dim, vdim=dim, conv=int(rng.randint(1, 5)),
                 scale=float(dim ** -0.5 * pick([1.0, 0.6, 1.5])))
        r = rng.rand()
        if r < 0.8:
            m["rot"] = dict(base=float(pick([100.0, 10000.0, 200000.0])), dims=int(pick([dim, dim // 2, 8])))
            if rng.rand() < 0.6:
                m["rot"]["scaling"] = dict(factor=float(pick([2.0, 4.0, 1.5])))
        return m

    layers = []
    for _ in range(int(rng.randint(2, 6))):
        r = rng.rand()
        if r < 0.15:
            mlp = None
        elif r < 0.45:
            mlp = dict(kind="dense", ff=int(pick([24, 50, 128, 200])))
        else:
            count = int(pick([1, 1, 2, 3, 4]))
            per = int(rng.randint(1, 5))
            keep = int(rng.randint(1, count + 1))
            total = count * per
            identity = int(rng.randint(0, min(total, 3) + 1)) if rng.rand() < 0.6 else 0
            router = dict(experts=total - identity, top=int(rng.randint(1, min(keep * per, 4) + 1)))
            if identity:
                router["identity"] = identity
            if count > 1 or rng.rand() < 0.5:
                router["groups"] = dict(count=count, keep=keep)
            mlp = dict(kind="moe", expert=dict(ff=int(pick([8, 30, 64, 128]))), router=router)
        if rng.rand() < 0.6:
            layers.append(dict(type="parallel", mlp=mlp, mixer=dict(
                left=attn(), right=ssm(), left_scale=float(pick([1.0, 0.75, 0.5, 1.4])), right_scale=float(pick([1.0, 1.2, 0.3])))))
        else:
            layers.append(dict(type="mamba2", mixer=ssm(), mlp=mlp))
    raw = dict(architecture="Zupitar", vocab=int(rng.randint(50, 400)), width=width,
               norm=dict(eps=float(pick([1e-6, 1e-5, 1e-3]))), layers=layers)
    if rng.rand() < 0.7:
        raw["logit_softcap"] = float(pick([5.0, 12.0, 30.0]))
    return raw


def folder(tmp_path, raw, seed):
    import ai_engine_b200 as aie
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"drawn{seed}")
    aie.write_random_model(aie.ZupitarConfig.from_dict(raw), d, seed=seed, std=0.08, norm_std=0.1)
    t = {k: v.clone() for k, v in read_tensors(d).items()}       # copies: the file is written again below
    for k in list(t):          # attention scores that spread
        if k.endswith("mix.left.q"):
            t[k] = (t[k].float() * 3.0).to(t[k].dtype)
    save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(d, "model.safetensors"))
    return d, t


def reference(raw, t, ids, dtype):
    margins = []
    logits = pz.forward(raw, t, ids, dtype=dtype, margins_out=margins).double().numpy()
    m = torch.stack(margins).min(dim=0).values.double().numpy() if margins else np.full(len(ids), np.inf)
    ok = m >= zh.CLEAR
    return zh.Ref(logits, np.array([bool(ok[max(0, i - zh.AFTER):i + 1].all()) for i in range(len(ids))]))


def well_conditioned(raw, t, ids, ref):
    """Whether bfloat16 can be held to the oracle on this drawn model: the oracle is run once more with every matrix
    nudged by noise of half a bfloat16 step.  A model with several routers in a row turns many of its choices under
    such noise; if half of the rows move by more than 0.05 of the logits' spread, only float32 is compared."""
    g = torch.Generator().manual_seed(0)
    t2 = {k: (v.double() * (1 + 2.0 ** -9 * torch.randn(v.shape, generator=g, dtype=torch.float64))
              if v.is_floating_point() and v.dim() == 2 else v) for k, v in t.items()}
    out = pz.forward(raw, t2, ids, dtype=torch.float64).numpy()
    moved = np.abs(out - np.asarray(ref)).max(1) / max(float(np.std(ref)), 1e-3)
    return float(np.median(moved)) <= 0.05


@pytest.mark.parametrize("seed", range(20))
def test_a_drawn_configuration(tmp_path, seed):
    from ai_engine_b200.engine.replay import Replayer

    raw = draw(seed)
    d, t = folder(tmp_path, raw, seed)
    a, b = ids_for(70, raw["vocab"], seed), ids_for(26, raw["vocab"], 100 + seed)
    for dtype in ("float32", "bfloat16"):
        ref_a, ref_b = reference(raw, t, a, oracle_dtype(dtype)), reference(raw, t, b, oracle_dtype(dtype))
        if dtype == "bfloat16" and not well_conditioned(raw, t, a, ref_a):
            continue
        rep = Replayer(d, dtype, max_tokens=192, block_size=int([8, 16, 32][seed % 3]))
        whole = rep.run_step([dict(id="w", tokens=a, want=list(range(70)))], end=["w"]).numpy()
        close(whole, ref_a, dtype, f"drawn {seed} whole {raw['layers']}")
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
        close(np.concatenate(got_a), ref_a, dtype, f"drawn {seed} in portions")
        close(np.concatenate(got_b), ref_b, dtype, f"drawn {seed} the request beside it")
