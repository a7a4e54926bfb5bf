"""Each mechanism of the Pifutar design alone, on the GPU, against the plain implementation's function for it:
the parts are built from a PartSpec, given random tensors, and stepped with a real cache and step context, in
portions and with several requests in a batch."""
import math

import numpy as np
import pytest
import torch

import plain_pifutar as pp

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


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


def tol(dtype, ref, f32=2e-5, bf16=4e-2):
    return (f32 if dtype == torch.float32 else bf16) * max(1.0, float(ref.abs().max()))


class Rig:
    """One part with a cache of its own (pages and state as it asks) and steps made by the engine's step context."""

    def __init__(self, part, dtype, page=8, pages=64, max_seqs=4):
        from ai_engine_b200.cache import PagedCache
        from ai_engine_b200.parts import CacheNeed
        self.part = part
        self.cache = PagedCache([CacheNeed(0, "p", part.cache_request(), part.state_request())], page, pages,
                                max_seqs, 4096, dtype, DEV)
        self.err = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.have = {}

    def admit(self):
        s = self.cache.admit()
        assert s >= 0
        self.have[s] = 0
        return s

    def finish(self, slot):
        self.cache.finish(slot)
        del self.have[slot]

    def step(self, portions, ids=None):
        """portions: [(slot, n tokens)]; returns (ctx, the part's LayerCache)."""
        from ai_engine_b200.engine.step import StepContext, StepEntry
        entries = []
        for k, (slot, n) in enumerate(portions):
            assert self.cache.ensure(slot, self.have[slot] + n)
            toks = list(ids[k]) if ids is not None else [0] * n
            entries.append(StepEntry(slot, self.have[slot], toks, []))
        ctx = StepContext(entries, self.cache, torch.device(DEV), self.err)
        lc = self.cache.part_cache(0, "p", ctx)
        return ctx, lc

    def done(self, portions):
        for slot, n in portions:
            self.have[slot] += n
            self.cache.advance(slot, self.have[slot])
        assert int(self.err.item()) == 0


def as_f64(out):
    out = out.double()
    return (out.sum(0) if out.dim() == 3 else out).cpu()


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_norm_with_a_weight_stored_around_zero(dtype, offset):
    from ai_engine_b200.parts import PartSpec, RMSNorm
    D = 104
    p = RMSNorm(PartSpec("rmsnorm", dict(size=D, eps=1e-3, offset=offset, output="float32"), dict(weight="w")), env(dtype, D))
    w = (0.3 * torch.randn(D)).to(dtype)
    load(p, {"w": w}, dtype)
    x = 3 * torch.randn(7, D, device=DEV)
    out = p.forward(x.clone())
    assert out.dtype == torch.float32                 # 32-bit rows for the filter that follows
    want = pp.rms(x.double().cpu(), 1e-3) * (offset + w.double())
    assert (out.double().cpu() - want).abs().max() <= 1e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,D", [(1, 72), (2, 72), (3, 70), (5, 72), (4, 1030)])
def test_short_convolution_carries_its_tail_across_portions_and_slots(dtype, taps, D):
    """Widths that are multiples of 4 take the kernel with four channels a thread, the others one channel."""
    from ai_engine_b200.parts import CausalShortConv, PartSpec
    p = CausalShortConv(PartSpec("causal_short_conv", dict(size=D, taps=taps), dict(weight="w")), env(dtype, D))
    w = (0.5 * torch.randn(D, taps)).to(dtype)
    load(p, {"w": w}, dtype)
    rig = Rig(p, dtype, max_seqs=2)
    g = torch.Generator().manual_seed(taps)
    seqs = [torch.randn(n, D, generator=g) for n in (23, 9, 14)]
    wants = [pp.short_conv(s.double(), w.double(), torch.zeros(taps - 1, D, dtype=torch.float64))[0] for s in seqs]
    # two requests side by side in portions of unequal size (down to one token); then the first slot is
    # given back and used again by a third request, whose tail must start from zero
    a, b = rig.admit(), rig.admit()
    cuts_a, cuts_b = [1, 1, 2, 7, 1, 3, 8], [4, 1, 1, 1, 2]
    got = {a: [], b: []}
    ia = ib = 0
    for k in range(max(len(cuts_a), len(cuts_b))):
        portions, rows = [], []
        if k < len(cuts_a):
            portions.append((a, cuts_a[k])); rows.append(seqs[0][ia:ia + cuts_a[k]]); ia += cuts_a[k]
        if k < len(cuts_b):
            portions.append((b, cuts_b[k])); rows.append(seqs[1][ib:ib + cuts_b[k]]); ib += cuts_b[k]
        ctx, lc = rig.step(portions)
        out = p.forward(torch.cat(rows).to(DEV), ctx, lc)
        assert out.dtype == dtype
        at = 0
        for slot, n in portions:
            got[slot].append(out[at:at + n].double().cpu()); at += n
        rig.done(portions)
    for slot, want in ((a, wants[0]), (b, wants[1])):
        assert (torch.cat(got[slot]) - want).abs().max() <= tol(dtype, want, 1e-5, 2e-2)
    rig.finish(a)
    c = rig.admit()
    assert c == a
    ctx, lc = rig.step([(c, 14)])
    out = p.forward(seqs[2].to(DEV), ctx, lc).double().cpu()
    rig.done([(c, 14)])
    assert (out - wants[2]).abs().max() <= tol(dtype, wants[2], 1e-5, 2e-2)


def test_depth_average_keeps_every_layers_stream():
    from ai_engine_b200.kernels import ops
    T, D, L = 5, 40, 4
    g = torch.Generator().manual_seed(0)
    x0 = torch.randn(T, D, generator=g)
    deltas = [torch.randn(T, D, generator=g) for _ in range(L)]
    coefs = [torch.randn(i + 2, generator=g) for i in range(L)]
    history = torch.full((L + 1, T, D), float("nan"), device=DEV)
    x = x0.clone().to(DEV)
    history[0].copy_(x)
    streams, cur = [x0.double()], x0.double()
    for i in range(L):
        delta = deltas[i].to(DEV) if i % 2 == 0 else torch.stack([0.25 * deltas[i], 0.75 * deltas[i]]).to(DEV)   # parts
        ops.depth_average(x, delta, history, coefs[i].to(DEV), i + 1)
        streams.append(cur + deltas[i].double())
        cur = sum(coefs[i][j].double() * streams[j] for j in range(i + 2))
        assert (x.double().cpu() - cur).abs().max() < 1e-4
        assert (history[i + 1].double().cpu() - streams[-1]).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_polynorm_feed_forward(dtype):
    from ai_engine_b200.parts import PartSpec, PolyNormFF
    D, F = 72, 200
    p = PolyNormFF(PartSpec("polynorm_ff", dict(hidden_size=D, intermediate_size=F, eps=1e-4),
                            dict(up="u", down="d", act="a")), env(dtype, D))
    ts = {"u": (0.3 * torch.randn(F, D)).to(dtype), "d": (0.1 * torch.randn(D, F)).to(dtype),
          "a": torch.tensor([0.9, -0.4, 0.25, 0.1]).to(dtype)}
    load(p, ts, dtype)
    h = torch.randn(9, D).to(dtype)
    ctx = type("C", (), dict(err=torch.zeros(1, dtype=torch.int32, device=DEV)))()
    out = as_f64(p.forward(h.to(DEV), ctx))
    want = pp.dense_ff(h.double(), ts["u"].double(), ts["d"].double(), ts["a"].double(), 1e-4)
    assert (out - want).abs().max() <= tol(dtype, want, 2e-5, 4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,F,Fs,D", [(6, 3, 40, 56, 72), (1, 1, 24, 0, 72), (9, 2, 64, 64, 128), (5, 5, 128, 0, 128)])
def test_experts_chosen_by_a_table(dtype, E, top, F, Fs, D):
    """Also top = experts = 1, no shared expert, and the sizes that take the grouped tensor-core product."""
    from ai_engine_b200.parts import PartSpec, TableMoE
    V, T = 50, 77
    p = TableMoE(PartSpec("table_moe", dict(hidden_size=D, vocab_size=V, num_experts=E, top=top, intermediate_size=F,
                                            limit=0.8, shared_intermediate_size=Fs, shared_limit=0.5),
                          dict(table="t", gate="e{e}.g", up="e{e}.u", down="e{e}.d", shared_gate="s.g", shared_up="s.u",
                               shared_down="s.d", shared_sg="s.sg")), env(dtype, D))
    g = torch.Generator().manual_seed(E)
    r = lambda *s: (0.25 * torch.randn(*s, generator=g)).to(dtype)
    ts = {"t": torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)}
    for e in range(E):
        ts.update({f"e{e}.g": r(F, D), f"e{e}.u": r(F, D), f"e{e}.d": r(D, F)})
    if Fs:
        ts.update({"s.g": r(Fs, D), "s.u": r(Fs, D), "s.d": r(D, Fs), "s.sg": r(1, D)})
    load(p, ts, dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    h = torch.randn(T, D, generator=g).to(dtype)
    ctx = type("C", (), dict(err=torch.zeros(1, dtype=torch.int32, device=DEV), token_ids=ids.to(torch.int32).to(DEV)))()
    out = as_f64(p.forward(h.to(DEV), ctx))
    f = lambda n: ts[n].double()
    shared = (f("s.g"), f("s.u"), f("s.d"), f("s.sg"), 0.5) if Fs else None
    want = pp.table_moe(h.double(), ids, ts["t"], [(f(f"e{e}.g"), f(f"e{e}.u"), f(f"e{e}.d")) for e in range(E)], 0.8, shared)
    assert int(ctx.err.item()) == 0
    assert (out - want).abs().max() <= tol(dtype, want, 2e-5, 4e-2)
    # a token's output does not depend on the tokens beside it
    alone = as_f64(p.forward(h[5:6].to(DEV), type("C", (), dict(err=ctx.err, token_ids=ctx.token_ids[5:6].contiguous()))()))
    assert (alone - out[5:6]).abs().max() <= (1e-6 if dtype == torch.float32 else 2e-2) * max(1.0, float(want.abs().max()))


def latent_part(dtype, D, m, shares=False):
    from ai_engine_b200.parts import LatentAttention, PartSpec, RotaryEncoding
    e = env(dtype, D)
    rope = RotaryEncoding(PartSpec("rotary", dict(rot_dim=m["rot"]["dims"], theta=m["rot"]["base"], scaling=None,
                                                  layout="interleaved")), e)
    rope.load(None)
    e.position_encodings["r"] = rope
    window = (m.get("mask") or {}).get("size", 0)
    return LatentAttention(PartSpec("latent_attention", dict(
        hidden_size=D, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
        kv_rank=m["kv_rank"], scale=m["scale"], window=window, eps=1e-5, position_encoding="r", shares_cache=shares),
        dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o")), e)


def latent_tensors(dtype, D, m, g, gain=3.0):
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    r = lambda *s, k=1.0: (k * torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(dtype)
    return {"q": r(H * (d + dr), D, k=gain), "dkv": r(rank + dr, D), "dkv.norm": (1 + 0.2 * torch.randn(rank, generator=g)).to(dtype),
            "uk": r(H * d, rank), "uv": r(H * dv, rank), "o": r(D, H * dv)}


LATENT_CASES = [
    dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, rot=dict(base=10000.0, dims=8), mask=dict(size=11)),
    dict(heads=20, dim=16, rot_dim=16, vdim=8, kv_rank=128, scale=0.18, rot=dict(base=500000.0, dims=16), mask=dict(size=70)),
    dict(heads=4, dim=32, rot_dim=32, vdim=16, kv_rank=64, scale=0.125, rot=dict(base=100.0, dims=16)),
    # every width of the tensor-core kernel's column split: latents of 192, 256, 320, 384, 448 and 512
    dict(heads=3, dim=16, rot_dim=16, vdim=8, kv_rank=192, scale=0.2, rot=dict(base=10000.0, dims=16), mask=dict(size=33)),
    dict(heads=17, dim=8, rot_dim=32, vdim=8, kv_rank=256, scale=0.2, rot=dict(base=10000.0, dims=32), mask=dict(size=64)),
    dict(heads=2, dim=24, rot_dim=16, vdim=8, kv_rank=320, scale=0.15, rot=dict(base=10000.0, dims=16)),
    dict(heads=5, dim=16, rot_dim=16, vdim=8, kv_rank=384, scale=0.2, rot=dict(base=10000.0, dims=16), mask=dict(size=65)),
    dict(heads=1, dim=16, rot_dim=16, vdim=8, kv_rank=448, scale=0.2, rot=dict(base=10000.0, dims=16), mask=dict(size=129)),
    dict(heads=16, dim=32, rot_dim=64, vdim=16, kv_rank=512, scale=0.1, rot=dict(base=500000.0, dims=64), mask=dict(size=100)),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(LATENT_CASES)))
def test_latent_attention_windows_portions_and_batches(dtype, case):
    """Three requests in unequal portions against each alone and whole.  One token's input is scaled up so that
    its rotated key part dominates some heads' softmax for as long as the window shows it: a window that is one
    token off, at a page border or not, changes the output far beyond the tolerance."""
    m, D = LATENT_CASES[case], 64
    window = (m.get("mask") or {}).get("size", 0)
    g = torch.Generator().manual_seed(case)
    ts = latent_tensors(dtype, D, m, g)
    p = load(latent_part(dtype, D, m), ts, dtype)
    lens = (150, 37, 1 + 2 * max(window, 8))
    hs = [torch.randn(n, D, generator=g).to(dtype) for n in lens]
    for h, star in zip(hs, (40, 7, 8)):          # 40 and 8 are page borders, 7 a page's last row
        h[star] *= 8.0
    W = {k: v.double() for k, v in ts.items()}
    wants = [pp.latent_attention(h.double(), torch.arange(h.shape[0]), W, m, 1e-5, {}) for h in hs]
    rig = Rig(p, dtype, page=8, pages=64, max_seqs=3)
    slots = [rig.admit() for _ in hs]
    fed, got = [0, 0, 0], [[], [], []]
    sizes = [[64, 2, 3, 1, 1, 40, 1, 38], [5, 1, 1, 2, 28], [1, 1] + [7] * 400]
    k = 0
    while any(fed[i] < lens[i] for i in range(3)):
        portions, rows, who = [], [], []
        for i in range(3):
            if fed[i] >= lens[i] or (k % 3 == i and k % 5 == 0):        # sometimes left out of a step
                continue
            n = min(sizes[i][min(len(got[i]), len(sizes[i]) - 1)], lens[i] - fed[i])
            portions.append((slots[i], n)); rows.append(hs[i][fed[i]:fed[i] + n]); who.append((i, n))
        k += 1
        if not portions:
            continue
        ctx, lc = rig.step(portions)
        out = as_f64(p.forward(torch.cat(rows).to(DEV), ctx, lc))
        at = 0
        for i, n in who:
            got[i].append(out[at:at + n]); at += n; fed[i] += n
        rig.done(portions)
    for i in range(3):
        err = (torch.cat(got[i]) - wants[i]).abs()
        assert err.max() <= tol(dtype, wants[i], 3e-5, 5e-2), (i, int(err.max(1).values.argmax()), float(err.max()))
    if window:       # pages that the window has passed went back to the pool while the requests were live
        assert rig.cache.book.total_allocations(0) > rig.cache.book.high_water(0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_key_just_inside_and_just_outside_the_window_in_prompts_and_decoding(dtype):
    """The output at distance window - 1 from a dominant key differs from the output at distance window by the
    whole of that key's value; both must match the oracle, fed as one prompt and decoded token by token."""
    m, D = LATENT_CASES[1], 64
    w = m["mask"]["size"]
    g = torch.Generator().manual_seed(9)
    ts = latent_tensors(dtype, D, m, g, gain=4.0)
    p = load(latent_part(dtype, D, m), ts, dtype)
    star, n = 13, 13 + w + 6
    h = torch.randn(n, D, generator=g).to(dtype)
    h[star] *= 10.0
    want = pp.latent_attention(h.double(), torch.arange(n), {k: v.double() for k, v in ts.items()}, m, 1e-5, {})
    inside, outside = star + w - 1, star + w
    assert (want[inside] - want[outside]).abs().max() > 10 * tol(dtype, want, 3e-5, 5e-2)      # the edge shows
    for cuts in ([n], [star + 1] + [1] * (n - star - 1), [inside, 2, n - inside - 2]):
        rig = Rig(p, dtype, page=16, pages=16, max_seqs=1)
        s, at, outs = rig.admit(), 0, []
        for c in cuts:
            ctx, lc = rig.step([(s, c)])
            outs.append(as_f64(p.forward(h[at:at + c].to(DEV), ctx, lc)))
            rig.done([(s, c)]); at += c
        err = (torch.cat(outs) - want).abs().max(1).values
        assert err.max() <= tol(dtype, want, 3e-5, 5e-2), (cuts[:3], int(err.argmax()), float(err.max()))


def linear_part(dtype, D, kind, H, d, dv, extra):
    from ai_engine_b200.parts import DecayLinearAttention, PartSpec
    gated = kind == "gla"
    return DecayLinearAttention(PartSpec("decay_linear_attention", dict(
        hidden_size=D, num_heads=H, key_dim=d, value_dim=dv, eps=1e-5, decay=None if gated else extra, tau=extra if gated else 0.0,
        decay_rank=6, scale_on="q" if gated else "k", norm_weight=gated),
        dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a2_bias="a2.b")), env(dtype, D))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind,H,d,dv,extra", [("retention", 3, 16, 24, [0.5, 0.9, 0.99]), ("retention", 1, 100, 12, [0.97]),
                                               ("gla", 2, 24, 40, 8.0), ("gla", 1, 160, 33, 2.0), ("gla", 5, 8, 8, 16.0)])
def test_linear_attention_state_in_portions_batches_and_long_decoding(dtype, kind, H, d, dv, extra):
    D = 48
    g = torch.Generator().manual_seed(H * d)
    r = lambda *s, k=1.0: (k * torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(dtype)
    ts = {"q": r(H * d, D), "k": r(H * d, D), "v": r(H * dv, D), "g": r(H * dv, D), "o": r(D, H * dv)}
    if kind == "gla":
        ts.update({"norm": (1 + 0.2 * torch.randn(dv, generator=g)).to(dtype), "a1": r(6, D), "a2": r(H * d, 6, k=2.0),
                   "a2.b": (1.5 + torch.randn(H * d, generator=g)).to(dtype)})
    p = load(linear_part(dtype, D, kind, H, d, dv, extra), ts, dtype)
    W = {k: v.double() for k, v in ts.items()}
    m = dict(heads=H, dim=d, vdim=dv, decay=extra, tau=extra)
    fn = pp.retention if kind == "retention" else pp.gated_linear_attention
    lens = (90, 31)
    hs = [torch.randn(n, D, generator=g).to(dtype) for n in lens]
    wants = [fn(h.double(), W, m, 1e-5, torch.zeros(H, d, dv, dtype=torch.float64)) for h in hs]
    rig = Rig(p, dtype, max_seqs=2)
    slots = [rig.admit(), rig.admit()]
    cuts = [[17, 2, 1, 5] + [1] * 65, [3, 1, 1, 26]]           # a prompt in portions, then sixty-five tokens one by one
    fed, got = [0, 0], [[], []]
    for k in range(max(len(c) for c in cuts)):
        portions, rows, who = [], [], []
        for i in range(2):
            if k < len(cuts[i]):
                n = cuts[i][k]
                portions.append((slots[i], n)); rows.append(hs[i][fed[i]:fed[i] + n]); who.append((i, n))
        ctx, lc = rig.step(portions)
        out = as_f64(p.forward(torch.cat(rows).to(DEV), ctx, lc))
        at = 0
        for i, n in who:
            got[i].append(out[at:at + n]); at += n; fed[i] += n
        rig.done(portions)
    for i in range(2):
        err = (torch.cat(got[i]) - wants[i]).abs()
        assert err.max() <= tol(dtype, wants[i], 3e-5, 5e-2), (i, int(err.max(1).values.argmax()), float(err.max()))
    # a slot that is given back starts from a zero state
    rig.finish(slots[1])
    s = rig.admit()
    ctx, lc = rig.step([(s, 31)])
    out = as_f64(p.forward(hs[1].to(DEV), ctx, lc))
    assert (out - wants[1]).abs().max() <= tol(dtype, wants[1], 3e-5, 5e-2)
