"""PifutarConfig: the typed configuration of a Pifutar model.

config.json names the architecture under `architecture`, the sizes `vocab` and `width`, `norm.eps`,
`canon.taps` (taps of the short convolution in front of every sublayer) and a list `layers`.  A layer has a
`type` (latent_attention | retention | gla), the sizes and constants of its mixer under `mixer`, and its
feed-forward under `mlp` (null: none; kind dense | moe).  Every size and constant of a model is read here;
a missing or ill-typed key is a ConfigError that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from .base import ConfigError, get_float, get_int

MIXER_TYPES = ("latent_attention", "retention", "gla")


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
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query/key elements a head
    rot_dim: int             # rotated query/key elements a head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    window: int              # 0: every earlier key
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, m: dict, where: str) -> "LatentAttentionConfig":
        heads, dim, rot_dim = get_int(m, "heads"), get_int(m, "dim", minimum=0), get_int(m, "rot_dim", minimum=0)
        rot = _obj(m, "rot", where, required=rot_dim > 0) or {}
        rot_dims = get_int(rot, "dims", rot_dim, minimum=0)
        if rot_dims > rot_dim or rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} must be even and at most rot_dim = {rot_dim}")
        mask = _obj(m, "mask", where, required=False)
        kv_from = m.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {where}`kv_from` must be a layer index, got {kv_from!r}")
        return cls(heads, dim, rot_dim, get_int(m, "vdim"), get_int(m, "kv_rank"),
                   get_float(m, "scale", float(dim + rot_dim) ** -0.5),
                   get_int(mask, "size", 0, minimum=0) if mask else 0,
                   get_float(rot, "base", 10000.0), rot_dims, kv_from)

    def to_dict(self) -> dict:
        d = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, kv_rank=self.kv_rank,
                 scale=self.scale, rot=dict(base=self.rot_base, dims=self.rot_dims))
        if self.window:
            d["mask"] = dict(size=self.window)
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class LinearAttentionConfig:
    """retention: `decay` per head; gla: `tau` (the decay's rank is the shape of its first projection)."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...] = ()
    tau: float = 0.0
    decay_rank: int = 16

    @classmethod
    def from_dict(cls, m: dict, kind: str, where: str) -> "LinearAttentionConfig":
        heads = get_int(m, "heads")
        if kind == "retention":
            decay = m.get("decay")
            if not isinstance(decay, list) or len(decay) != heads or any(
                    isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
                raise ConfigError(f"config.json: {where}`decay` must list one number per head ({heads})")
            return cls(heads, get_int(m, "dim"), get_int(m, "vdim"), tuple(float(x) for x in decay))
        tau = get_float(m, "tau")
        if tau <= 0:
            raise ConfigError(f"config.json: {where}`tau` must be positive, got {tau}")
        return cls(heads, get_int(m, "dim"), get_int(m, "vdim"), (), tau, get_int(m, "decay_rank", 16))

    def to_dict(self) -> dict:
        d = dict(heads=self.heads, dim=self.dim, vdim=self.vdim)
        if self.decay:
            d["decay"] = list(self.decay)
        else:
            d.update(tau=self.tau, decay_rank=self.decay_rank)
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                          # dense | moe
    ff: int = 0                        # dense: width; moe: an expert's width
    limit: float = 0.0                 # moe: clamp of an expert's operands
    experts: int = 0
    top: int = 0
    shared_ff: int = 0                 # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, f: dict, where: str) -> "FeedForwardConfig":
        kind = f.get("kind")
        if kind == "dense":
            return cls("dense", get_int(f, "ff"))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind `{kind}` is not known (dense, moe)")
        ex, ro = _obj(f, "expert", where), _obj(f, "router", where)
        sh = _obj(f, "shared", where, required=False)
        experts, top = get_int(ro, "experts"), get_int(ro, "top")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top = {top} exceeds router.experts = {experts}")
        return cls("moe", get_int(ex, "ff"), get_float(ex, "limit"), experts, top,
                   get_int(sh, "ff") if sh else 0, get_float(sh, "limit") if sh else 0.0)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        d = dict(kind="moe", expert=dict(ff=self.ff, limit=self.limit),
                 router=dict(experts=self.experts, top=self.top))
        if self.shared_ff:
            d["shared"] = dict(ff=self.shared_ff, limit=self.shared_limit)
        return d


@dataclass(frozen=True)
class PifutarLayer:
    type: str
    mixer: object                                   # LatentAttentionConfig | LinearAttentionConfig
    mlp: Optional[FeedForwardConfig] = None

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class PifutarConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int
    layers: Tuple[PifutarLayer, ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20          # nothing in the design bounds a sequence; the cache does
    eos_token_ids: Tuple[int, ...] = ()

    ARCHITECTURE = "Pifutar"

    @classmethod
    def from_dict(cls, raw: dict) -> "PifutarConfig":
        norm, canon = _obj(raw, "norm", ""), _obj(raw, "canon", "")
        ls = raw.get("layers")
        if not isinstance(ls, list) or not ls:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers: List[PifutarLayer] = []
        for i, l in enumerate(ls):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = l.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type `{kind}` is not known ({', '.join(MIXER_TYPES)})")
            m = _obj(l, "mixer", where)
            mixer = (LatentAttentionConfig.from_dict(m, where) if kind == "latent_attention"
                     else LinearAttentionConfig.from_dict(m, kind, where))
            ff = _obj(l, "mlp", where, required=False)
            layers.append(PifutarLayer(kind, mixer, FeedForwardConfig.from_dict(ff, where) if ff else None))
        for i, l in enumerate(layers):
            j = getattr(l.mixer, "kv_from", None)
            if j is None:
                continue
            src = layers[j].mixer if j < i else None
            if (src is None or layers[j].type != "latent_attention" or src.kv_from is not None
                    or (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) !=
                    (l.mixer.kv_rank, l.mixer.rot_dim, l.mixer.rot_base, l.mixer.rot_dims)):
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} must name an earlier latent-attention "
                                  f"layer with a cache of its own and the same kv_rank, rot_dim and rotation")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        return cls(get_int(raw, "vocab"), get_int(raw, "width"), get_float(norm, "eps"), get_int(canon, "taps"),
                   tuple(layers), get_int(raw, "max_position_embeddings", 1 << 20), eos)

    def to_dict(self) -> dict:
        d = dict(architecture=self.ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 canon=dict(taps=self.taps), layers=[l.to_dict() for l in self.layers])
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
