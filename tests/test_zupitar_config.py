"""The Zupitar configuration, its model builder, cache needs and random weights, and the plain implementation's own
consistency, without a device."""
import copy

import numpy as np
import pytest
import torch

import plain_zupitar as pz
from zupitar_helpers import CONFIGS, ids_for, make_dir, read_tensors


def test_config_is_found_by_its_name_and_round_trips():
    import ai_engine_b200 as aie
    from ai_engine_b200.config import load_config

    for name, raw in CONFIGS.items():
        arch, cfg = load_config(raw)
        assert arch.name == "Zupitar" and isinstance(cfg, aie.ZupitarConfig)
        assert aie.ZupitarConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.width == raw["width"] and len(cfg.layers) == len(raw["layers"])
    a = aie.ZupitarConfig.from_dict(CONFIGS["A"])
    assert a.logit_softcap == 10.0 and a.layers[0].left.rot_factor == 2.0 and a.layers[0].left.scale == 0.21
    assert a.layers[2].left.rot_dims == 0 and a.layers[2].mlp is None
    assert (a.layers[0].mlp.experts, a.layers[0].mlp.identity, a.layers[0].mlp.group_count, a.layers[0].mlp.group_keep) == (5, 1, 3, 2)
    assert (a.layers[3].mlp.identity, a.layers[3].mlp.group_count) == (0, 1)          # defaults of absent keys
    assert aie.ZupitarConfig.from_dict(CONFIGS["B"]).logit_softcap == 0.0


def test_a_missing_or_wrong_key_is_named():
    import ai_engine_b200 as aie

    def bad(name, change, match):
        raw = copy.deepcopy(CONFIGS[name])
        change(raw)
        with pytest.raises(aie.ConfigError, match=match):
            aie.ZupitarConfig.from_dict(raw)

    bad("A", lambda r: r["layers"][1]["mixer"].pop("state"), "state")
    bad("A", lambda r: r["layers"][0]["mixer"]["left"].update(vdim=48), "vdim")
    bad("A", lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=4), "kv_heads")
    bad("A", lambda r: r["layers"][0]["mixer"]["right"].update(groups=3), "groups")
    bad("A", lambda r: r["layers"][0]["mlp"]["router"].update(top=5), "top")              # two kept groups hold four
    bad("A", lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups")
    bad("A", lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=34), "rot.dims")
    bad("A", lambda r: r["layers"][1].update(type="attention"), "type")
    bad("C", lambda r: r["layers"][1]["mlp"].update(kind="glu"), "kind")
    bad("C", lambda r: r.pop("norm"), "norm")


def test_tensor_names_and_shapes_follow_the_configuration():
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.model import tensor_specs_of

    arch, cfg = load_config(CONFIGS["A"])
    specs = {s.name: tuple(s.shape) for s in tensor_specs_of(arch.build_spec(cfg))}
    assert specs["embed"] == (211, 96) and specs["head"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["l0.mix.left.q"] == (192, 96) and specs["l0.mix.left.k"] == (64, 96) and "l0.mix.left.v" not in specs
    assert specs["l0.mix.left.q.conv"] == (192, 3) and specs["l0.mix.left.k.conv"] == (64, 3)
    assert specs["l0.mix.right.in"] == (2 * 96 + 2 * 32 + 4, 96) and specs["l0.mix.right.conv"] == (96 + 64, 4)
    assert specs["l0.mix.right.conv.b"] == (160,) and specs["l0.mix.right.A_log"] == (4,)
    assert specs["l1.mix.in"] == (2 * 120 + 2 * 24 + 3, 96) and specs["l1.mix.norm"] == (120,) and specs["l1.mix.o"] == (96, 120)
    assert specs["l0.mlp.router"] == (6, 96) and specs["l0.mlp.correction"] == (6,)
    assert "l0.mlp.e4.down" in specs and "l0.mlp.e5.down" not in specs                    # the sixth output is an identity expert
    assert specs["l1.mlp.gate"] == (80, 96) and specs["l0.norm1b"] == (96,) and specs["l1.norm2b"] == (96,)
    assert "l2.norm2" not in specs and "l2.norm2b" not in specs and "l2.mlp.gate" not in specs
    arch, cfg = load_config(CONFIGS["C"])
    specs = {s.name for s in tensor_specs_of(arch.build_spec(cfg))}
    assert "l0.mlp.router" in specs and not any(n.startswith("l0.mlp.e") for n in specs)    # only identity experts


def test_cache_needs_pages_for_attention_and_slots_for_state():
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.base import KVRequest
    from ai_engine_b200.parts.model import Model

    arch, cfg = load_config(CONFIGS["A"])
    model = Model(arch.build_spec(cfg), torch.float32, device="cpu")
    needs = {(n.run, n.role): n for n in model.cache_requests()}
    assert set(needs) == {(0, "mixer.left"), (0, "mixer.right"), (1, "mixer"), (2, "mixer.left"), (2, "mixer.right"), (3, "mixer")}
    assert needs[0, "mixer.left"].kv == KVRequest(2, 32, 0) and needs[0, "mixer.left"].state.shape == (2, 256)
    assert needs[2, "mixer.left"].kv == KVRequest(3, 16, 0) and needs[2, "mixer.left"].state.shape == (0, 96)
    right = needs[0, "mixer.right"].state
    assert right["tail"].shape == (3, 160) and right["S"].shape == (4, 16, 24) and right["S"].dtype == torch.float32
    assert needs[1, "mixer"].kv is None and needs[1, "mixer"].state["S"].shape == (3, 24, 40)
    assert not model.pads_decode_rows()            # a repeated row would race on its slot's state
    cache = PagedCache(model.cache_requests(), 8, 16, 2, 128, torch.float32, "cpu")
    assert len(cache.groups) == 2                  # two head shapes: two pools with block tables of their own
    assert cache.state[0, "mixer.right"]["S"].shape == (2, 4, 16, 24)
    slot = cache.admit()
    cache.state[1, "mixer"]["tail"][slot] += 1.0
    cache.finish(slot)
    assert cache.admit() == slot and float(cache.state[1, "mixer"]["tail"][slot].abs().sum()) == 0.0    # a slot starts at zero
    arch, cfg = load_config(CONFIGS["C"])
    model = Model(arch.build_spec(cfg), torch.float32, device="cpu")
    assert all(n.kv is None for n in model.cache_requests()) and model.keeps_state()


def test_linear_scaling_divides_every_frequency():
    from ai_engine_b200.parts.rope import rotary_inv_freq

    plain = rotary_inv_freq(8, 100.0)
    np.testing.assert_allclose(plain, [1.0, 100.0 ** -0.25, 0.1, 100.0 ** -0.75], rtol=1e-6)
    np.testing.assert_allclose(rotary_inv_freq(8, 100.0, dict(type="linear", factor=4.0)), plain / 4.0, rtol=1e-6)
    with pytest.raises(ValueError):
        rotary_inv_freq(8, 100.0, dict(type="cubic", factor=4.0))


def test_the_plain_implementation_continues_from_its_own_state(tmp_path):
    """Random weights written by the engine's random-weights mode are read back by name, and the oracle gives the
    same logits whether a sequence is fed whole, in portions, or token by token."""
    for name in ("A", "C"):
        d = make_dir(tmp_path, name)
        raw, t = CONFIGS[name], read_tensors(d)
        ids = ids_for(19, raw["vocab"], 3)
        whole = pz.forward(raw, t, ids)
        assert whole.shape == (19, raw["vocab"]) and bool(torch.isfinite(whole).all())
        if raw.get("logit_softcap"):
            assert float(whole.abs().max()) < raw["logit_softcap"]
        for cuts in ([7, 1, 2, 9], [1] * 19):
            st, out, at = pz.State(raw, torch.float64), [], 0
            for c in cuts:
                out.append(pz.forward(raw, t, ids[at:at + c], state=st))
                at += c
            assert float((torch.cat(out) - whole).abs().max()) < 1e-9


def test_the_router_of_the_plain_implementation_by_hand():
    # six outputs in three groups of two; corrections make every choice value negative except in group 1
    h = torch.eye(6, dtype=torch.float64)[:1]
    w = torch.zeros(6, 6, dtype=torch.float64)
    w[:, 0] = torch.tensor([2.0, 0.0, 1.0, 1.5, 0.5, 0.0])
    s = torch.softmax(w[:, 0], 0)
    corr = torch.tensor([-1.0, -1.0, 0.0, 0.0, -1.0, -0.9])
    ids, weights = pz.route(h, w, corr, top=2, group_count=3, group_keep=1)
    assert ids.tolist() == [[3, 2]] and torch.allclose(weights[0], s[[3, 2]])       # weights without the correction
    # two groups kept: the best groups are 1 and 0 (-1 + s0 > -0.9 + s5); group 2's larger values do not count
    ids, _ = pz.route(h, w, corr, top=3, group_count=3, group_keep=2)
    assert ids.tolist() == [[3, 2, 0]]
    ids, _ = pz.route(h, w, torch.zeros(6, dtype=torch.float64), top=2, group_count=1, group_keep=1)
    assert ids.tolist() == [[0, 3]]
