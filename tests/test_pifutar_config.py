"""The Pifutar configuration, its model builder and its random weights, without a device."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_pifutar as pp
from pifutar_helpers import CONFIGS, ids_for, make_dir, read_tensors


def test_config_is_found_by_its_name_and_round_trips():
    import ai_engine_b200 as aie
    from ai_engine_b200.config import load_config

    for name, raw in CONFIGS.items():
        arch, cfg = load_config(raw)
        assert arch.name == "Pifutar" and isinstance(cfg, aie.PifutarConfig)
        again = aie.PifutarConfig.from_dict(cfg.to_dict())
        assert again == cfg
        assert cfg.width == raw["width"] and cfg.taps == raw["canon"]["taps"] and len(cfg.layers) == len(raw["layers"])


def test_a_missing_or_wrong_key_is_named():
    import ai_engine_b200 as aie

    bad = copy.deepcopy(CONFIGS["X"])
    del bad["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(aie.ConfigError, match="kv_rank"):
        aie.PifutarConfig.from_dict(bad)
    bad = copy.deepcopy(CONFIGS["X"])
    bad["layers"][3]["mixer"]["kv_from"] = 4          # a later layer
    with pytest.raises(aie.ConfigError, match="kv_from"):
        aie.PifutarConfig.from_dict(bad)
    bad = copy.deepcopy(CONFIGS["X"])
    bad["layers"][3]["mixer"]["kv_rank"] = 32         # differs from the layer it reads
    with pytest.raises(aie.ConfigError, match="kv_from"):
        aie.PifutarConfig.from_dict(bad)
    bad = copy.deepcopy(CONFIGS["Y"])
    bad["layers"][0]["mixer"]["decay"] = [0.5]
    with pytest.raises(aie.ConfigError, match="decay"):
        aie.PifutarConfig.from_dict(bad)
    bad = copy.deepcopy(CONFIGS["Y"])
    bad["layers"][0]["type"] = "softmax"
    with pytest.raises(aie.ConfigError, match="type"):
        aie.PifutarConfig.from_dict(bad)


def test_tensor_names_and_shapes_follow_the_configuration():
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.model import tensor_specs_of

    arch, cfg = load_config(CONFIGS["X"])
    specs = {s.name: tuple(s.shape) for s in tensor_specs_of(arch.build_spec(cfg))}
    assert specs["embed"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["l1.mix.q"] == (5 * 40, 96) and specs["l1.mix.dkv"] == (72, 96) and specs["l1.mix.uk"] == (160, 64)
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs          # reads layer 1's cache
    assert "l2.norm2" not in specs and "l2.canon2" not in specs                  # no feed-forward
    assert specs["l0.mix.a2"] == (72, 16) and specs["l0.mix.a2.b"] == (72,) and specs["l0.mix.norm"] == (40,)
    assert specs["l4.mlp.e4.down"] == (96, 32) and specs["l4.mlp.table"] == (211, 2) and specs["l4.mlp.shared.sg"] == (1, 96)
    assert specs["l3.dwa"] == (5,) and specs["l0.canon1"] == (96, 4) and specs["l0.mlp.act"] == (4,)
    assert "lm_head" not in " ".join(specs)


def test_cache_needs_windows_shared_rows_and_state():
    from ai_engine_b200.cache import PagedCache
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.model import Model

    arch, cfg = load_config(CONFIGS["X"])
    model = Model(arch.build_spec(cfg), torch.float32, device="cpu")
    needs = model.cache_requests()
    kv = {n.run: n for n in needs if n.role == "mixer" and (n.kv is not None or n.cache_from is not None)}
    # layer 1's rows must outlive the widest window of the layers that read them (24, 17, 9)
    assert kv[1].kv.window == 24 and kv[1].kv.planes == 1 and kv[1].kv.head_dim == 72 and kv[1].kv.kv_heads == 1
    assert kv[3].cache_from == 1 and kv[5].cache_from == 1 and kv[4].kv.window == 0 and kv[4].kv.head_dim == 60
    state = {(n.run, n.role): n.state.shape for n in needs if n.state is not None}
    assert state[0, "mixer"] == (3, 24, 40) and state[2, "mixer"] == (2, 16, 24)
    assert state[0, "mixer_filter"] == (3, 96) and state[1, "ffn_filter"] == (3, 96) and (2, "ffn_filter") not in state
    cache = PagedCache(needs, 8, 16, 4, 128, torch.float32, allocate=False)
    assert len(cache.groups) == 2 and cache.where[3, "mixer"] == cache.where[1, "mixer"] and not cache.writes[5, "mixer"]
    # a model without attention asks for no pages at all
    arch, cfg = load_config(CONFIGS["Y"])
    needs = Model(arch.build_spec(cfg), torch.float32, device="cpu").cache_requests()
    assert all(n.kv is None for n in needs) and len(PagedCache(needs, 8, 4, 2, 64, torch.float32, allocate=False).groups) == 0


def test_random_weights_can_be_read_back_and_tables_have_distinct_rows(tmp_path):
    d = make_dir(tmp_path, "X")
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    assert raw["architecture"] == "Pifutar"
    t = read_tensors(d)
    table = t["l1.mlp.table"]
    assert table.dtype == torch.int32 and table.shape == (211, 3) and int(table.max()) < 6 and int(table.min()) >= 0
    assert all(len(set(r)) == 3 for r in table.tolist())
    assert abs(float(t["l1.norm1"].float().mean())) < 0.05 and float(t["l1.norm1"].float().std()) > 0.05
    logits = pp.forward(raw, t, ids_for(7, 211, 0), dtype=torch.float32)
    assert logits.shape == (7, 211) and bool(torch.isfinite(logits).all())


def test_the_plain_implementation_continues_from_its_state(tmp_path):
    """The oracle itself: a sequence in one call equals the same sequence in portions carried by its state."""
    for name in ("X", "Y"):
        d = make_dir(tmp_path, name)
        t, raw = read_tensors(d), CONFIGS[name]
        ids = ids_for(40, raw["vocab"], 5)
        whole = pp.forward(raw, t, ids).numpy()
        st, parts = pp.State(), []
        for a, b in ((0, 3), (3, 4), (4, 6), (6, 21), (21, 22), (22, 40)):
            parts.append(pp.forward(raw, t, ids[a:b], st).numpy())
        assert np.abs(np.concatenate(parts) - whole).max() < 1e-9
