"""TizodraConfig: the typed configuration of a Tizodra model.

config.json names the architecture under `architecture`, the sizes `vocab` and `width`, `norm.eps`, `logit_scale`,
a list `layers` and, optionally, `loop`: the layers start .. stop - 1 run `times` times in a row.  A layer has a
`type` (attention | delta), the sizes and constants of its mixer under `mixer`, and its feed-forward under `mlp`
(null: none; kind dense).  Every size and constant of a model is read here; a missing or ill-typed key is a
ConfigError that names it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from .base import ConfigError, get_float, get_int

LAYER_TYPES = ("attention", "delta")


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
class TizodraMixer:
    """Sizes of a mixer.  attention: heads query heads and kv_heads key/value heads, keys of `dim`, values of `vdim`,
    the score's scale, the window (`window` keys, the first `keep_first` always seen; window 0: all keys).  delta:
    heads value heads of `vdim`, kv_heads query/key heads of `dim`, `conv` taps."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float = 0.0
    window: int = 0
    keep_first: int = 0
    conv: int = 0

    @classmethod
    def from_dict(cls, kind: str, m: dict, where: str) -> "TizodraMixer":
        heads, kv_heads = get_int(m, "heads"), get_int(m, "kv_heads")
        dim, vdim = get_int(m, "dim"), get_int(m, "vdim")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads = {heads} is not a multiple of kv_heads = {kv_heads}")
        if kind == "delta":
            return cls(heads, kv_heads, dim, vdim, conv=get_int(m, "conv"))
        mask = _obj(m, "mask", where, required=False) or {}
        window, keep = get_int(mask, "size", 0, minimum=0), get_int(mask, "keep_first", 0, minimum=0)
        return cls(heads, kv_heads, dim, vdim, scale=get_float(m, "scale"), window=window, keep_first=keep)

    def to_dict(self, kind: str) -> dict:
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim)
        if kind == "delta":
            d["conv"] = self.conv
        else:
            d["scale"] = self.scale
            if self.window:
                d["mask"] = dict(size=self.window, keep_first=self.keep_first)
        return d


@dataclass(frozen=True)
class TizodraLayer:
    type: str
    mixer: TizodraMixer
    ff: int = 0                          # the dense feed-forward's width; 0: the layer has none

    def to_dict(self) -> dict:
        return dict(type=self.type, mixer=self.mixer.to_dict(self.type),
                    mlp=dict(kind="dense", ff=self.ff) if self.ff else None)


@dataclass(frozen=True)
class TizodraConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float = 1.0
    layers: Tuple[TizodraLayer, ...] = field(default_factory=tuple)
    loop_start: int = 0                  # layers loop_start .. loop_stop - 1 run loop_times times in a row;
    loop_stop: int = 0                   # loop_times 0: the model has no loop
    loop_times: int = 0
    max_position_embeddings: int = 1 << 20          # nothing in the design bounds a sequence; the cache does
    eos_token_ids: Tuple[int, ...] = ()

    ARCHITECTURE = "Tizodra"

    @classmethod
    def from_dict(cls, raw: dict) -> "TizodraConfig":
        norm = _obj(raw, "norm", "")
        ls = raw.get("layers")
        if not isinstance(ls, list) or not ls:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers: List[TizodraLayer] = []
        for i, l in enumerate(ls):
            where = f"layers[{i}]."
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = l.get("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type `{kind}` is not known ({', '.join(LAYER_TYPES)})")
            mixer = TizodraMixer.from_dict(kind, _obj(l, "mixer", where), where + "mixer.")
            f = _obj(l, "mlp", where, required=False)
            ff = 0
            if f:
                if f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind `{f.get('kind')}` is not known (dense)")
                ff = get_int(f, "ff")
            layers.append(TizodraLayer(kind, mixer, ff))
        loop = _obj(raw, "loop", "", required=False)
        start = stop = times = 0
        if loop:
            start, stop = get_int(loop, "start", minimum=0), get_int(loop, "stop", minimum=0)
            times = get_int(loop, "times", minimum=1)
            if not start < stop <= len(layers):
                raise ConfigError(f"config.json: loop.start = {start} and loop.stop = {stop} must name layers "
                                  f"(0 <= start < stop <= {len(layers)})")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (eos,)
        return cls(get_int(raw, "vocab"), get_int(raw, "width"), get_float(norm, "eps"),
                   get_float(raw, "logit_scale", 1.0), tuple(layers), start, stop, times,
                   get_int(raw, "max_position_embeddings", 1 << 20), eos)

    def to_dict(self) -> dict:
        d = dict(architecture=self.ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 logit_scale=self.logit_scale, layers=[l.to_dict() for l in self.layers])
        if self.loop_times:
            d["loop"] = dict(start=self.loop_start, stop=self.loop_stop, times=self.loop_times)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def run_order(self) -> List[int]:
        """The layers in the order they run: the loop's layers `loop_times` times in a row, the others once."""
        n = len(self.layers)
        if not self.loop_times:
            return list(range(n))
        return (list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, n)))
