"""FokisunConfig: the typed configuration of a Fokisun model.

config.json names the architecture under `architecture`, the sizes `vocab` and `width`, `norm.eps`,
`residual_mult`, `logit_scale` and a list `layers`.  A layer has a `type` (latent_attention | hgrn2 | attention), the
sizes and constants of its mixer under `mixer`, and its feed-forward under `mlp` (null: none; kind dense | moe).
Every size and constant of a model is read here; a missing or ill-typed key is a ConfigError that names it.  Keys
that may be absent mean "none": no window, no rotation, no scaling, no value mixing, one group, no shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .base import ConfigError, get_bool, get_float, get_int

LAYER_TYPES = ("latent_attention", "hgrn2", "attention")


def _obj(raw: dict, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where}`{key}` is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}`{key}` must be an object, got {v!r}")
    return v


def _named(fn, where: str):
    """Run a reader and put the place in front of its complaint."""
    try:
        return fn()
    except ConfigError as e:
        raise ConfigError(str(e).replace("config.json: ", f"config.json: {where}", 1)) from None


@dataclass(frozen=True)
class FokisunMixer:
    """Sizes of a mixer.  hgrn2: heads of `dim` gate/query channels and `vdim` value channels.  attention: heads query
    heads and kv_heads key/value heads, keys of `dim`, values of `vdim`, the score's scale, the window (0: all keys),
    the rotation over the first rot_dims elements of a head (0: none) with its base and the factor all frequencies
    are divided by, v_mix.  latent_attention: heads with `dim` unrotated and `rot_dim` rotated query/key elements,
    values of `vdim`, latents of kv_rank and q_rank, the scale, the rotation."""
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0
    scale: float = 0.0
    window: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_factor: float = 1.0
    v_mix: bool = False
    rot_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0

    @classmethod
    def from_dict(cls, kind: str, m: dict, where: str) -> "FokisunMixer":
        heads, dim, vdim = get_int(m, "heads"), get_int(m, "dim"), get_int(m, "vdim")
        if kind == "hgrn2":
            return cls(heads, dim, vdim)
        rot = _obj(m, "rot", where, required=False) or {}
        rot_dims = get_int(rot, "dims", 0, minimum=0)
        rot_base = get_float(rot, "base", 10000.0)
        scaling = _obj(rot, "scaling", where + "rot.", required=False) or {}
        rot_factor = get_float(scaling, "factor", 1.0)
        if rot_dims % 2:
            raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} must be even")
        scale = get_float(m, "scale")
        if kind == "attention":
            kv_heads = get_int(m, "kv_heads", heads)
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}heads = {heads} is not a multiple of kv_heads = {kv_heads}")
            if rot_dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} exceeds dim = {dim}")
            mask = _obj(m, "mask", where, required=False) or {}
            return cls(heads, dim, vdim, kv_heads=kv_heads, scale=scale, window=get_int(mask, "size", 0, minimum=0),
                       rot_dims=rot_dims, rot_base=rot_base, rot_factor=rot_factor, v_mix=get_bool(m, "v_mix", False))
        rot_dim = get_int(m, "rot_dim", 0, minimum=0)
        if rot_dims > rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} exceeds rot_dim = {rot_dim}")
        return cls(heads, dim, vdim, scale=scale, rot_dims=rot_dims, rot_base=rot_base, rot_factor=rot_factor,
                   rot_dim=rot_dim, kv_rank=get_int(m, "kv_rank"), q_rank=get_int(m, "q_rank"))

    def to_dict(self, kind: str) -> dict:
        d = dict(heads=self.heads, dim=self.dim, vdim=self.vdim)
        if kind == "hgrn2":
            return d
        d["scale"] = self.scale
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
            if self.rot_factor != 1.0:
                d["rot"]["scaling"] = dict(factor=self.rot_factor)
        if kind == "attention":
            d["kv_heads"] = self.kv_heads
            if self.window:
                d["mask"] = dict(size=self.window)
            if self.v_mix:
                d["v_mix"] = True
        else:
            d.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank, q_rank=self.q_rank)
        return d


@dataclass(frozen=True)
class FokisunFF:
    """A feed-forward.  dense: width `ff`.  moe: `experts` experts of width `ff` of which a token uses `top`, in
    `group_count` groups of which `group_keep` stay open, weights times `scale`; a shared expert of width
    `shared_ff` (0: none)."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    group_count: int = 1
    group_keep: int = 1
    scale: float = 1.0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, f: dict, where: str) -> "FokisunFF":
        kind = f.get("kind")
        if kind == "dense":
            return cls("dense", get_int(f, "ff"))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}kind `{kind}` is not known (dense, moe)")
        ff = _named(lambda: get_int(_obj(f, "expert", where), "ff"), where + "expert.")
        r = _obj(f, "router", where)
        groups = _obj(r, "groups", where + "router.", required=False) or {}
        shared = _obj(f, "shared", where, required=False)

        def read():
            experts, top = get_int(r, "experts"), get_int(r, "top")
            count = get_int(groups, "count", 1)
            keep = get_int(groups, "keep", count)
            if experts % count or keep > count or top > experts // count * keep:
                raise ConfigError(f"config.json: {experts} experts do not divide into {count} groups of which {keep} "
                                  f"are kept for {top} choices")
            return cls("moe", ff, experts, top, count, keep, get_float(r, "scale", 1.0),
                       get_int(shared, "ff") if shared else 0)
        return _named(read, where + "router.")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        d = dict(kind="moe", expert=dict(ff=self.ff),
                 router=dict(experts=self.experts, top=self.top, scale=self.scale,
                             groups=dict(count=self.group_count, keep=self.group_keep)))
        if self.shared_ff:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class FokisunLayer:
    type: str
    mixer: FokisunMixer
    mlp: Optional[FokisunFF] = None

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(self.type), mlp=self.mlp.to_dict() if self.mlp else None)


@dataclass(frozen=True)
class FokisunConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    layers: Tuple[FokisunLayer, ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20          # nothing in the design bounds a sequence; the cache does
    eos_token_ids: Tuple[int, ...] = ()

    ARCHITECTURE = "Fokisun"

    @classmethod
    def from_dict(cls, raw: dict) -> "FokisunConfig":
        norm = _obj(raw, "norm", "")
        ls = raw.get("layers")
        if not isinstance(ls, list) or not ls:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = []
        mixed = None
        for i, l in enumerate(ls):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = l.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type `{kind}` is not known ({', '.join(LAYER_TYPES)})")
            m = _obj(l, "mixer", where)
            mixer = _named(lambda: FokisunMixer.from_dict(kind, m, where + "mixer."), where + "mixer.")
            if mixer.v_mix:
                if mixed is not None and (mixer.kv_heads, mixer.vdim) != mixed:
                    raise ConfigError(f"config.json: {where}mixer: layers that mix values need kv_heads = {mixed[0]} and "
                                      f"vdim = {mixed[1]} like the first of them")
                mixed = (mixer.kv_heads, mixer.vdim)
            f = _obj(l, "mlp", where, required=False)
            layers.append(FokisunLayer(kind, mixer, FokisunFF.from_dict(f, where + "mlp.") if f else None))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        return cls(get_int(raw, "vocab"), get_int(raw, "width"), _named(lambda: get_float(norm, "eps"), "norm."),
                   get_float(raw, "residual_mult", 1.0), get_float(raw, "logit_scale", 1.0), tuple(layers),
                   get_int(raw, "max_position_embeddings", 1 << 20), eos)

    def to_dict(self) -> dict:
        d = dict(architecture=self.ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 residual_mult=self.residual_mult, logit_scale=self.logit_scale,
                 layers=[l.to_dict() for l in self.layers])
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
