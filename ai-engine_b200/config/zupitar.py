"""ZupitarConfig: the typed configuration of a Zupitar model.

config.json names the architecture under `architecture`, the sizes `vocab` and `width`, `norm.eps`,
`logit_softcap` and a list `layers`.  A layer has a `type` (parallel | mamba2), the sizes and constants of its
mixer under `mixer` (for `parallel`: `left`, an attention, `right`, a state-space mixer, and their weights
`left_scale`, `right_scale`), and its feed-forward under `mlp` (null: none; kind dense | moe).  Every size and
constant of a model is read here; a missing or ill-typed key is a ConfigError that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from .base import ConfigError, get_float, get_int

LAYER_TYPES = ("parallel", "mamba2")


def _obj(raw: dict, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where}`{key}` is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}`{key}` must be an object, got {v!r}")
    return v


@dataclass(frozen=True)
class KeyedAttentionConfig:
    """Softmax attention whose values are its keys: no value projection, a short convolution behind the query and
    key projections, a rotation of the first `rot_dims` elements of a head with evenly stretched positions."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    rot_base: float = 10000.0
    rot_dims: int = 0
    rot_factor: float = 1.0

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "KeyedAttentionConfig":
        heads, kv_heads, dim = get_int(m, "heads"), get_int(m, "kv_heads"), get_int(m, "dim")
        vdim = get_int(m, "vdim", dim)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads = {heads} is not a multiple of kv_heads = {kv_heads}")
        if vdim != dim:
            raise ConfigError(f"config.json: {where}vdim = {vdim} differs from dim = {dim}, but the values are the keys")
        rot = _obj(m, "rot", where, required=False) or {}
        rot_dims = get_int(rot, "dims", 0, minimum=0)
        if rot_dims > dim or rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} must be even and at most dim = {dim}")
        scaling = _obj(rot, "scaling", where + "rot.", required=False) or {}
        factor = get_float(scaling, "factor", 1.0)
        if factor <= 0:
            raise ConfigError(f"config.json: {where}rot.scaling.factor must be positive, got {factor}")
        return cls(heads, kv_heads, dim, vdim, get_int(m, "conv"), get_float(m, "scale", float(dim) ** -0.5),
                   get_float(rot, "base", 10000.0), rot_dims, factor)

    def to_dict(self) -> dict:
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, conv=self.conv, scale=self.scale)
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
            if self.rot_factor != 1.0:
                d["rot"]["scaling"] = dict(factor=self.rot_factor)
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "StateSpaceConfig":
        heads, vdim, groups = get_int(m, "heads"), get_int(m, "vdim"), get_int(m, "groups", 1)
        norm_groups = get_int(m, "norm_groups", 1)
        if heads % groups:
            raise ConfigError(f"config.json: {where}heads = {heads} is not a multiple of groups = {groups}")
        if (heads * vdim) % norm_groups:
            raise ConfigError(f"config.json: {where}heads * vdim = {heads * vdim} does not divide into "
                              f"norm_groups = {norm_groups}")
        return cls(heads, vdim, get_int(m, "state"), groups, get_int(m, "conv"), norm_groups)

    def to_dict(self) -> dict:
        return dict(heads=self.heads, vdim=self.vdim, state=self.state, groups=self.groups, conv=self.conv,
                    norm_groups=self.norm_groups)


@dataclass(frozen=True)
class ZupitarFeedForward:
    kind: str                          # dense | moe
    ff: int = 0                        # dense: width; moe: an expert's width
    experts: int = 0                   # experts with tensors
    identity: int = 0                  # router outputs behind them that hand the input on
    top: int = 0
    group_count: int = 1
    group_keep: int = 1

    @classmethod
    def from_dict(cls, f: dict, where: str) -> "ZupitarFeedForward":
        kind = f.get("kind")
        if kind == "dense":
            return cls("dense", get_int(f, "ff"))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind `{kind}` is not known (dense, moe)")
        ex, ro = _obj(f, "expert", where + "mlp."), _obj(f, "router", where + "mlp.")
        experts, top = get_int(ro, "experts", minimum=0), get_int(ro, "top")
        identity = get_int(ro, "identity", 0, minimum=0)
        gr = _obj(ro, "groups", where + "mlp.router.", required=False) or {}
        count, keep = get_int(gr, "count", 1), get_int(gr, "keep", 1)
        total = experts + identity
        if total < 1 or total % count or keep > count or top > total // count * keep:
            raise ConfigError(f"config.json: {where}mlp.router: {total} outputs (experts + identity) must divide into "
                              f"groups.count = {count} groups, of which groups.keep = {keep} hold at least top = {top}")
        return cls("moe", get_int(ex, "ff"), experts, identity, top, count, keep)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        return dict(kind="moe", expert=dict(ff=self.ff),
                    router=dict(experts=self.experts, identity=self.identity, top=self.top,
                                groups=dict(count=self.group_count, keep=self.group_keep)))


@dataclass(frozen=True)
class ZupitarLayer:
    type: str
    left: Optional[KeyedAttentionConfig]            # parallel only
    right: StateSpaceConfig                         # the state-space mixer (the only one of a mamba2 layer)
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[ZupitarFeedForward] = None

    def to_dict(self) -> dict:
        if self.type == "parallel":
            mixer = dict(left=self.left.to_dict(), right=self.right.to_dict(), left_scale=self.left_scale,
                         right_scale=self.right_scale)
        else:
            mixer = self.right.to_dict()
        return dict(type=self.type, mixer=mixer, mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class ZupitarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float = 0.0                      # 0: the logits are left as they are
    layers: Tuple[ZupitarLayer, ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20          # nothing in the design bounds a sequence; the cache does
    eos_token_ids: Tuple[int, ...] = ()

    ARCHITECTURE = "Zupitar"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZupitarConfig":
        norm = _obj(raw, "norm", "")
        ls = raw.get("layers")
        if not isinstance(ls, list) or not ls:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers: List[ZupitarLayer] = []
        for i, l in enumerate(ls):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = l.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type `{kind}` is not known ({', '.join(LAYER_TYPES)})")
            m = _obj(l, "mixer", where)
            ff = _obj(l, "mlp", where, required=False)
            mlp = ZupitarFeedForward.from_dict(ff, where) if ff else None
            if kind == "parallel":
                w = where + "mixer."
                layers.append(ZupitarLayer(kind, KeyedAttentionConfig.from_dict(_obj(m, "left", w), w + "left."),
                                           StateSpaceConfig.from_dict(_obj(m, "right", w), w + "right."),
                                           get_float(m, "left_scale", 1.0), get_float(m, "right_scale", 1.0), mlp))
            else:
                layers.append(ZupitarLayer(kind, None, StateSpaceConfig.from_dict(m, where + "mixer."), mlp=mlp))
        softcap = get_float(raw, "logit_softcap", 0.0)
        if softcap < 0:
            raise ConfigError(f"config.json: `logit_softcap` must be positive, got {softcap}")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        return cls(get_int(raw, "vocab"), get_int(raw, "width"), get_float(norm, "eps"), softcap, tuple(layers),
                   get_int(raw, "max_position_embeddings", 1 << 20), eos)

    def to_dict(self) -> dict:
        d = dict(architecture=self.ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 layers=[l.to_dict() for l in self.layers])
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
