"""Each mechanism of the Zupitar design alone, on the GPU, against the plain implementation's function for it: the
parts are built from a PartSpec, given random or planted tensors, and stepped with a real cache and step context,
in portions and with several requests in a batch."""
import math

import numpy as np
import pytest
import torch

import plain_zupitar as pz
from zupitar_helpers import DEV, Rig, env, load

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, ref, f32=2e-5, bf16=4e-2):
    return (f32 if dtype == torch.float32 else bf16) * max(1.0, float(ref.abs().max()))


def od(dtype):
    """The oracle's dtype: float64 against the float32 engine, float32 against bfloat16 (on the same rounded weights)."""
    return torch.float64 if dtype == torch.float32 else torch.float32


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("taps,C,lead", [(1, 40, 0), (2, 70, 8), (3, 64, 24), (4, 300, 5), (6, 33, 0)])
@pytest.mark.parametrize("act", [None, "silu"])
def test_convolution_on_a_slice_with_bias_activation_and_tail(taps, C, lead, act):
    """The input is a slice of a wider row (as the state-space mixer's x|B|C inside its projection); two requests in
    unequal portions down to one token, then a slot used again must start from a zero tail."""
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.parts import CacheNeed, StateRequest
    from ai_engine_b200.parts.base import Part

    class Holder(Part):
        def state_request(self):
            return StateRequest((taps - 1, C), torch.float32)

    rig = Rig(Holder(None, None), torch.float32, max_seqs=2)
    g = torch.Generator().manual_seed(taps)
    w, b = 0.5 * torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    seqs = [torch.randn(n, lead + C + 3, generator=g) for n in (23, 9, 14)]

    def want(s):
        y = pz.causal_conv(s[:, lead:lead + C].double(), w.double(), torch.zeros(taps - 1, C, dtype=torch.float64), b.double())[0]
        return pz.silu(y) if act else y

    rig.part.forward = lambda rows, ctx, lc: ops.causal_conv(rows[:, lead:lead + C], w.to(DEV), b.to(DEV), lc.state, ctx,
                                                             torch.float32, activation=act)
    got = rig.run(seqs[:2], [[1, 1, 2, 7, 1, 3, 8], [4, 1, 1, 1, 2]])
    for k in range(2):
        assert (got[k] - want(seqs[k])).abs().max() <= 1e-5
    got = rig.run(seqs[2:], [[14]])                    # the slots were given back: the tail starts from zero
    assert (got[0] - want(seqs[2])).abs().max() <= 1e-5


def test_convolution_writes_the_tied_columns_twice():
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.parts import StateRequest
    from ai_engine_b200.parts.base import Part

    C, dup, taps = 56, 16, 3

    class Holder(Part):
        def state_request(self):
            return StateRequest((taps - 1, C), torch.float32)

    rig = Rig(Holder(None, None), torch.float32)
    w = torch.randn(C, taps)
    x = torch.randn(11, C)
    rig.part.forward = lambda rows, ctx, lc: ops.causal_conv(rows, w.to(DEV), None, lc.state, ctx, torch.float32,
                                                             dup_from=C - dup, dup_n=dup)
    got = rig.run([x], [[4, 7]])[0]
    ref = pz.causal_conv(x.double(), w.double(), torch.zeros(taps - 1, C, dtype=torch.float64))[0]
    assert got.shape == (11, C + dup)
    assert (got[:, :C] - ref).abs().max() <= 1e-5 and torch.equal(got[:, C:], got[:, C - dup:C])


# ---------------------------------------------------------------------------------------------------
def attention_part(dtype, D, H, K, d, taps, scale, rot):
    from ai_engine_b200.parts import GQAAttention, PartSpec, RotaryEncoding
    encs = {}
    if rot is not None:
        base, dims, factor = rot
        pe = RotaryEncoding(PartSpec("rotary", dict(rot_dim=dims, theta=base,
                                                    scaling=dict(type="linear", factor=factor) if factor else None)), env(dtype, D))
        pe.load(None)
        encs["r"] = pe
    return GQAAttention(PartSpec("gqa_attention", dict(
        hidden_size=D, num_heads=H, num_kv_heads=K, head_dim=d, window=0, scale=scale,
        position_encoding="r" if rot is not None else None, qk_conv=taps, tied_values=True),
        dict(q="q", k="k", o="o", q_conv="q.conv", k_conv="k.conv")), env(dtype, D, encs))


def attention_oracle(x, t, D, H, K, d, taps, scale, rot, dtype):
    m = dict(heads=H, kv_heads=K, dim=d, conv=taps, scale=scale)
    if rot is not None:
        m["rot"] = dict(base=rot[0], dims=rot[1], scaling=dict(factor=rot[2] or 1.0))
    st = pz.State._attn(m, dtype)
    return pz.keyed_attention(x.to(dtype), m, {k: v.to(dtype) for k, v in t.items()}, st, 0)


ATTN_SHAPES = [  # D, H, K, d, taps, scale, rot
    (72, 6, 2, 32, 3, 0.3, (1000.0, 16, 2.0)),         # the plain kernel in both dtypes; a partial, stretched rotation
    (64, 4, 1, 64, 2, 0.125, (10000.0, 64, None)),     # bfloat16: the tensor-core kernels; a full rotation
    (48, 2, 2, 128, 1, 0.09, None),                    # heads of 128, one tap, no rotation
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_attention_with_tied_values_in_portions_beside_other_requests(dtype, shape):
    D, H, K, d, taps, scale, rot = shape
    g = torch.Generator().manual_seed(d)
    t = {"q": 0.3 * torch.randn(H * d, D, generator=g), "k": 0.3 * torch.randn(K * d, D, generator=g),
         "o": 0.2 * torch.randn(D, H * d, generator=g), "q.conv": 0.6 * torch.randn(H * d, taps, generator=g),
         "k.conv": 0.6 * torch.randn(K * d, taps, generator=g)}
    t = {k: v.to(dtype) for k, v in t.items()}
    part = load(attention_part(dtype, D, H, K, d, taps, scale, rot), t, dtype)
    seqs = [torch.randn(n, D, generator=g).to(dtype) for n in (150, 37, 66)]
    rig = Rig(part, dtype, page=8, pages=48)
    got = rig.run(seqs, [[70, 2, 1, 1, 9, 67], [37], [1] * 5 + [61]])
    for k, s in enumerate(seqs):
        ref = attention_oracle(s, t, D, H, K, d, taps, scale, rot, od(dtype)).double()
        assert (got[k] - ref).abs().max() <= tol(dtype, ref, 2e-5, 5e-2), (k, float((got[k] - ref).abs().max()))
    # every page came back and is used again by a second round on the same pool
    assert rig.cache.book.pages_in_use(0) == 0
    got = rig.run(seqs[:1], [[149, 1]])
    ref = attention_oracle(seqs[0], t, D, H, K, d, taps, scale, rot, od(dtype)).double()
    assert (got[0] - ref).abs().max() <= tol(dtype, ref, 2e-5, 5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("planted", [0, 3, 7, 8, 9, 200])
def test_a_far_key_that_dominates_is_found_in_prompts_and_when_decoding(dtype, planted):
    """One key among 300 carries the whole weight: the query and that key are made parallel and long, all other
    rows short.  The output at the asking token is then that key's value (the key before rotation) through W_o; an
    engine that lost the key (the first tokens, a page's edge with pages of 8, far back) would return a mix of others."""
    D, H, K, d, taps, scale = 128, 4, 2, 32, 2, 1.0
    g = torch.Generator().manual_seed(5)
    wk = torch.zeros(K * d, D)
    wk[:, :K * d] = torch.eye(K * d)                       # a key is the first K d inputs
    wq = torch.zeros(H * d, D)
    for h in range(H):                                     # a query is its group's part of the inputs behind them
        wq[h * d:(h + 1) * d, K * d + (h // 2) * d:K * d + (h // 2 + 1) * d] = torch.eye(d)
    conv = torch.zeros(1, taps)
    conv[0, -1] = 1.0                                      # the convolution passes the current token, plus a little of the last
    conv[0, 0] = 0.1
    t = {"q": wq, "k": wk, "o": 0.2 * torch.randn(D, H * d, generator=g), "q.conv": conv.repeat(H * d, 1),
         "k.conv": conv.repeat(K * d, 1)}
    t = {k: v.to(dtype) for k, v in t.items()}
    n, ask = 300, 296
    x = 0.05 * torch.randn(n, D, generator=g)
    u = torch.randn(K * d, generator=g)
    u = u / u.norm()
    x[planted, :K * d] = 6.0 * u                           # the key; the token that asks is short as a key itself
    x[ask, K * d:] = 6.0 * u
    x = x.to(dtype)
    part = load(attention_part(dtype, D, H, K, d, taps, scale, None), t, dtype)
    ref = attention_oracle(x, t, D, H, K, d, taps, scale, None, od(dtype)).double()
    # the planted key does carry the weight: the answer is its value through W_o
    value = (x[planted].double() + (0.1 * x[planted - 1].double() if planted else 0))[:K * d].view(K, d)
    alone = (value.repeat_interleave(H // K, dim=0).reshape(1, H * d) @ t["o"].double().T)[0]
    assert (ref[ask] - alone).abs().max() <= 1e-3 * float(alone.abs().max())
    for cuts in ([n], [ask] + [1] * (n - ask), [planted + 1, ask - planted - 1, 2, 2]):
        got = Rig(part, dtype, page=8, pages=48).run([x], [cuts])[0]
        assert (got[ask] - ref[ask]).abs().max() <= tol(dtype, ref, 2e-5, 3e-2), cuts[:3]
        assert (got - ref).abs().max() <= tol(dtype, ref, 2e-5, 5e-2)


# ---------------------------------------------------------------------------------------------------
def ssm_part(dtype, D, P, dv, N, G, taps, ng, eps):
    from ai_engine_b200.parts import PartSpec, ScalarDecayStateSpace
    names = dict(conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", skip="D", norm="norm", o="o")
    names["in"] = "in"
    return ScalarDecayStateSpace(PartSpec("scalar_decay_state_space", dict(
        hidden_size=D, num_heads=P, value_dim=dv, state_size=N, groups=G, taps=taps, norm_groups=ng, eps=eps), names),
        env(dtype, D))


def ssm_tensors(g, D, P, dv, N, G, taps, dtype):
    ch = P * dv + 2 * G * N
    t = {"in": 0.25 * torch.randn(2 * P * dv + 2 * G * N + P, D, generator=g), "conv": 0.5 * torch.randn(ch, taps, generator=g),
         "conv.b": 0.2 * torch.randn(ch, generator=g), "dt_bias": torch.randn(P, generator=g) - 1.0,
         "A_log": torch.randn(P, generator=g) - 1.0, "D": 1.0 + 0.3 * torch.randn(P, generator=g),
         "norm": 1.0 + 0.2 * torch.randn(P * dv, generator=g), "o": 0.2 * torch.randn(D, P * dv, generator=g)}
    return {k: v.to(dtype) for k, v in t.items()}


def ssm_oracle(x, t, P, dv, N, G, taps, ng, eps, dtype):
    m = dict(heads=P, vdim=dv, state=N, groups=G, conv=taps, norm_groups=ng)
    return pz.state_space(x.to(dtype), m, {k: v.to(dtype) for k, v in t.items()}, pz.State._ssm(m, dtype), eps)


SSM_SHAPES = [  # D, P, dv, N, G, taps, norm groups
    (40, 4, 24, 16, 2, 4, 2), (64, 3, 40, 24, 1, 2, 3), (48, 6, 8, 40, 6, 1, 1), (72, 1, 44, 12, 1, 5, 4), (128, 8, 64, 128, 2, 3, 8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SSM_SHAPES)
def test_state_space_mixer_in_portions_decoding_and_on_a_slot_used_again(dtype, shape):
    D, P, dv, N, G, taps, ng = shape
    g = torch.Generator().manual_seed(P * dv)
    t = ssm_tensors(g, D, P, dv, N, G, taps, dtype)
    part = load(ssm_part(dtype, D, P, dv, N, G, taps, ng, 1e-4), t, dtype)
    seqs = [torch.randn(n, D, generator=g).to(dtype) for n in (100, 70, 31)]
    refs = [ssm_oracle(s, t, P, dv, N, G, taps, ng, 1e-4, od(dtype)).double() for s in seqs]
    rig = Rig(part, dtype, max_seqs=2)
    # a prompt in uneven portions beside a request that decodes sixty-five tokens one by one
    got = rig.run(seqs[:2], [[33, 2, 1, 17, 2, 45], [5] + [1] * 65])
    for k in range(2):
        assert (got[k] - refs[k]).abs().max() <= tol(dtype, refs[k], 3e-5, 6e-2), (k, float((got[k] - refs[k]).abs().max()))
    got = rig.run(seqs[2:], [[31]])                    # its slot held another request's state before
    assert (got[0] - refs[2]).abs().max() <= tol(dtype, refs[2], 3e-5, 6e-2)


def test_a_slow_constant_decay_keeps_its_digits_over_a_long_prompt():
    """A head whose step size hardly changes and whose decay is near one (what carries a token a thousand places):
    rounded to float32 such a decay repeats the same rounding at every token, and a far token's share drifts by
    tokens x 3e-8.  The float32 engine works the decay out in double; whole, and with the last hundred decoded."""
    D, P, dv, N, G, taps, ng = 24, 2, 8, 8, 1, 2, 1
    g = torch.Generator().manual_seed(9)
    t = ssm_tensors(g, D, P, dv, N, G, taps, torch.float32)
    t["in"][2 * P * dv + 2 * G * N:] = 0.0                # the step size is its bias alone
    t["dt_bias"] = torch.tensor([-6.0, -5.0])             # dt = 0.0025, 0.0067
    t["A_log"] = torch.tensor([0.0, -0.5])                # decays 0.9975 and 0.9959 a token
    part = load(ssm_part(torch.float32, D, P, dv, N, G, taps, ng, 1e-5), t, torch.float32)
    n = 1500
    x = torch.randn(n, D, generator=g)
    ref = ssm_oracle(x, t, P, dv, N, G, taps, ng, 1e-5, torch.float64).double()
    for cuts in ([n], [n - 100] + [1] * 100):
        got = Rig(part, torch.float32, max_seqs=1).run([x], [cuts])[0]
        err = (got[-100:] - ref[-100:]).abs().max() / ref[-100:].abs().max()
        assert float(err) <= 4e-6, (cuts[:2], float(err))


def test_state_space_decay_and_step_size_by_hand():
    """One head of two channels and one state row: the recurrence in closed form.  The convolution's weight is zero,
    so x, B and C are constants (silu of the bias), and dt and the decay follow from dt_bias and A_log alone."""
    D, taps = 8, 1
    t = {"in": torch.zeros(2 + 2 + 2 + 1, D), "conv": torch.zeros(4, taps), "conv.b": torch.tensor([0.7, -1.1, -0.4, 1.2]),
         "dt_bias": torch.tensor([0.3]), "A_log": torch.tensor([-0.2]), "D": torch.tensor([0.5]),
         "norm": torch.tensor([1.0, 2.0]), "o": torch.zeros(D, 2)}
    t["o"][0, 0] = t["o"][1, 1] = 1.0
    t["in"][0, 0] = t["in"][1, 1] = 1.0                   # z = the first two inputs: the gates
    part = load(ssm_part(torch.float32, D, 1, 2, 1, 1, taps, 1, 0.0), t, torch.float32)
    x = torch.zeros(6, D)
    x[:, 0], x[:, 1] = 2.0, -0.5
    got = Rig(part, torch.float32).run([x], [[2, 1, 3]])[0][:, :2]
    sl = lambda v: float(pz.silu(torch.tensor(v, dtype=torch.float64)))
    x0, x1, B, C = sl(0.7), sl(-1.1), sl(-0.4), sl(1.2)
    dt = math.log1p(math.exp(0.3))
    a = math.exp(-math.exp(-0.2) * dt)
    S0 = S1 = 0.0
    want = []
    for _ in range(6):
        S0, S1 = a * S0 + dt * B * x0, a * S1 + dt * B * x1
        y0, y1 = (S0 * C + 0.5 * x0) * sl(2.0), (S1 * C + 0.5 * x1) * sl(-0.5)
        r = math.sqrt((y0 * y0 + y1 * y1) / 2)
        want.append([y0 / r, 2.0 * y1 / r])
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), atol=1e-5)


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,groups,keep,top", [(6, 3, 1, 2), (6, 3, 2, 3), (14, 2, 1, 7), (5, 1, 1, 5), (8, 8, 3, 3), (64, 64, 64, 1)])
def test_the_router_kernel_against_the_plain_router(E, groups, keep, top):
    from ai_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(E + top)
    z = 2.0 * torch.randn(97, E, generator=g)
    corr = torch.randn(E, generator=g) * 0.3 - 0.5      # choice values below zero: a group left out counts as -inf, not 0
    ids, w = ops.route_topk(z.clone().to(DEV), corr.to(DEV), groups, keep, top)
    want_ids, want_w = pz.route(z.double(), torch.eye(E, dtype=torch.float64), corr.double(), top, groups, keep)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (w.cpu().double() - want_w).abs().max() <= 1e-6


def moe_part(dtype, D, E, ident, top, F, groups, keep):
    from ai_engine_b200.parts import PartSpec, RoutedMoE
    return RoutedMoE(PartSpec("routed_moe", dict(hidden_size=D, num_experts=E, identity=ident, top=top, intermediate_size=F,
                                                 groups=groups, keep=keep),
                              dict(router="router", correction="correction", gate="e{e}.gate", up="e{e}.up", down="e{e}.down")),
                     env(dtype, D))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,E,ident,top,F,groups,keep", [(48, 5, 1, 2, 40, 3, 2), (128, 6, 2, 3, 128, 4, 2), (40, 0, 3, 2, 8, 1, 1),
                                                          (64, 1, 0, 1, 24, 1, 1), (56, 7, 5, 4, 16, 2, 1)])
def test_routed_experts_and_a_token_alone_against_in_a_batch(dtype, D, E, ident, top, F, groups, keep):
    g = torch.Generator().manual_seed(D + E)
    t = {"router": 0.8 * torch.randn(E + ident, D, generator=g), "correction": 0.1 * torch.randn(E + ident, generator=g)}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = 0.3 * torch.randn(F, D, generator=g), 0.3 * torch.randn(F, D, generator=g)
        t[f"e{e}.down"] = 0.3 * torch.randn(D, F, generator=g)
    t = {k: v.to(dtype) for k, v in t.items()}
    part = load(moe_part(dtype, D, E, ident, top, F, groups, keep), t, dtype)
    x = torch.randn(150, D, generator=g).to(dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = type("Ctx", (), dict(err=err))()
    got = part.forward(x.to(DEV), ctx).double().cpu()
    o = od(dtype)
    experts = [(t[f"e{e}.gate"].to(o), t[f"e{e}.up"].to(o), t[f"e{e}.down"].to(o)) for e in range(E)]
    ref = pz.routed_moe(x.to(o), t["router"].to(o), t["correction"].to(o), experts, ident, top, groups, keep).double()
    # the router runs in float32 on the same rounded inputs in both dtypes, so the choices are the oracle's
    assert (got - ref).abs().max() <= tol(dtype, ref, 2e-5, 4e-2)
    assert int(err.item()) == 0
    alone = part.forward(x[17:18].to(DEV), ctx).double().cpu()
    assert (alone[0] - got[17]).abs().max() <= (1e-6 if dtype == torch.float32 else 2e-2) * max(1.0, float(got[17].abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["relu", "gelu_tanh", "silu"])
def test_gated_feed_forward_with_each_activation(dtype, act):
    from ai_engine_b200.parts import PartSpec, SwiGLU
    D, F = 72, 136
    g = torch.Generator().manual_seed(F)
    t = {"g": 0.3 * torch.randn(F, D, generator=g), "u": 0.3 * torch.randn(F, D, generator=g), "d": 0.3 * torch.randn(D, F, generator=g)}
    t = {k: v.to(dtype) for k, v in t.items()}
    part = load(SwiGLU(PartSpec("swiglu", dict(hidden_size=D, intermediate_size=F, activation=act), dict(gate="g", up="u", down="d")),
                       env(dtype, D)), t, dtype)
    x = torch.randn(90, D, generator=g).to(dtype)
    ctx = type("Ctx", (), dict(err=torch.zeros(1, dtype=torch.int32, device=DEV)))()
    out = part.forward(x.to(DEV), ctx).double()
    got = (out.sum(0) if out.dim() == 3 else out).cpu()
    gelu = lambda z: 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
    fn = dict(relu=torch.relu, gelu_tanh=gelu, silu=pz.silu)[act]
    o = od(dtype)
    ref = pz.gated_ff(x.to(o), t["g"].to(o), t["u"].to(o), t["d"].to(o), fn).double()
    assert (got - ref).abs().max() <= tol(dtype, ref, 2e-5, 4e-2)


def test_bounded_logits_and_the_weighted_sum_of_two_branches():
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.parts import LMHead, PartSpec
    D, V = 40, 77
    w = torch.randn(V, D)
    head = load(LMHead(PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, softcap=3.0), dict(weight="w")), env(torch.float32, D)),
                {"w": w}, torch.float32)
    x = torch.randn(9, D)
    got = head.forward(x.to(DEV)).double().cpu()
    ref = 3.0 * torch.tanh(x.double() @ w.double().T / 3.0)
    assert (got - ref).abs().max() <= 1e-5 and float(got.abs().max()) < 3.0
    a, b = torch.randn(3, 13, 40), torch.randn(13, 40)               # the first in three unjoined parts
    s = ops.scaled_sum(a.to(DEV), 0.7, b.to(DEV), 1.3).double().cpu()
    assert (s - (0.7 * a.double().sum(0) + 1.3 * b.double())).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_mixers_side_by_side_each_with_its_own_cache(dtype):
    from ai_engine_b200.parts import ParallelMixers, PartSpec
    D, H, K, d, taps, scale, rot = ATTN_SHAPES[0]
    P, dv, N, G, staps, ng = 4, 24, 16, 2, 4, 2
    g = torch.Generator().manual_seed(77)
    ta = {"q": 0.3 * torch.randn(H * d, D, generator=g), "k": 0.3 * torch.randn(K * d, D, generator=g),
          "o": 0.2 * torch.randn(D, H * d, generator=g), "q.conv": 0.6 * torch.randn(H * d, taps, generator=g),
          "k.conv": 0.6 * torch.randn(K * d, taps, generator=g)}
    ta = {k: v.to(dtype) for k, v in ta.items()}
    ts = ssm_tensors(g, D, P, dv, N, G, staps, dtype)
    left, right = attention_part(dtype, D, H, K, d, taps, scale, rot), ssm_part(dtype, D, P, dv, N, G, staps, ng, 1e-5)
    left.spec.tensors = {k: "a." + v for k, v in left.spec.tensors.items()}
    right.spec.tensors = {k: "s." + v for k, v in right.spec.tensors.items()}
    part = ParallelMixers(PartSpec("parallel_mixers", dict(left=left.spec, right=right.spec, left_scale=0.7, right_scale=1.3)),
                          left.env)
    tensors = {**{"a." + k: v for k, v in ta.items()}, **{"s." + k: v for k, v in ts.items()}}
    load(part, tensors, dtype)
    seqs = [torch.randn(n, D, generator=g).to(dtype) for n in (60, 25)]
    got = Rig(part, dtype).run(seqs, [[30, 1, 1, 28], [2, 23]])
    for k, s in enumerate(seqs):
        o = od(dtype)
        ref = (0.7 * attention_oracle(s, ta, D, H, K, d, taps, scale, rot, o) +
               1.3 * ssm_oracle(s, ts, P, dv, N, G, staps, ng, 1e-5, o)).double()
        assert (got[k] - ref).abs().max() <= tol(dtype, ref, 3e-5, 6e-2)
