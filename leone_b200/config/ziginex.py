"""Typed configuration of the Ziginex decoder.

Its ``config.json`` names the model under ``architecture`` and describes every layer on its own
(``layers``: a list of ``{"type", "mixer", "mlp"}``).  Top-level keys: ``vocab``, ``width``,
``norm.eps`` and, optionally, ``token_side.dim`` (the width of every layer's slice of the second
token table).

Mixer type ``parallel``: ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``softcap`` (optional), ``rot`` (``base``, ``dims``; optional), ``mask.size`` (the chunk; optional)) and
``right`` (gated delta rule: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` taps).
Mixer type ``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``,
``scale``, ``rot`` (``base``, ``dims``, optionally ``scaling`` with ``factor``, ``original``, ``fast``,
``slow``).

``mlp`` is ``null``, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"}, "router":
{"experts", "top", "identity", "groups": {"count", "keep"}}}`` (``identity`` and ``groups`` optional).

The file gives no limit on positions; ``max_positions`` (not a key of the design) bounds the
engine's block tables and defaults to 2**20.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .base import ConfigReader, InvalidValue, ModelConfig, UnsupportedField, WrongType

DEFAULT_MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("parallel", "latent_attention")


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_json(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


def _read_rot(r: ConfigReader, limit: int, what: str):
    """``(base, dims, scaling)`` of a ``rot`` section, ``(10000.0, 0, None)`` without one."""
    rot = r.section("rot", optional=True)
    if rot is None:
        return 10000.0, 0, None
    base, dims = rot.positive_float("base"), rot.positive_int("dims")
    if dims % 2 or dims > limit:
        raise InvalidValue(f"{rot.where}: 'dims' ({dims}) must be even and at most {what} ({limit})")
    sc = rot.section("scaling", optional=True)
    scaling = None
    if sc is not None:
        scaling = YarnScaling(sc.positive_float("factor"), sc.positive_float("original"), sc.positive_float("fast"),
                              sc.positive_float("slow"))
    return base, dims, scaling


def _rot_json(base, dims, scaling):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        out["scaling"] = scaling.to_json()
    return out


@dataclass(frozen=True)
class LeftMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float               # 0: no cap
    rot_base: float
    rot_dims: int                # 0: no rotation
    chunk: int                   # 0: every earlier position is seen

    def to_json(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.softcap:
            out["softcap"] = self.softcap
        if self.rot_dims:
            out["rot"] = _rot_json(self.rot_base, self.rot_dims, None)
        if self.chunk:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class RightMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                    # taps of the convolution on q, k and v; 0: none

    def to_json(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim}
        if self.conv:
            out["conv"] = self.conv
        return out


@dataclass(frozen=True)
class ParallelMixer:
    left: LeftMixer
    right: RightMixer

    def to_json(self):
        return {"left": self.left.to_json(), "right": self.right.to_json()}


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[YarnScaling]

    def to_json(self):
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "q_rank": self.q_rank, "scale": self.scale, "rot": _rot_json(self.rot_base, self.rot_dims, self.rot_scaling)}


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoeMlp:
    expert_ff: int
    experts: int
    top: int
    identity: int                # router outputs past the experts whose expert passes its input on
    groups: int                  # 1: no groups
    groups_kept: int

    def to_json(self):
        router = {"experts": self.experts, "top": self.top}
        if self.identity:
            router["identity"] = self.identity
        if self.groups > 1:
            router["groups"] = {"count": self.groups, "keep": self.groups_kept}
        return {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": router}


@dataclass(frozen=True)
class ZiginexLayer:
    type: str
    mixer: Union[ParallelMixer, LatentMixer]
    mlp: Union[None, DenseMlp, MoeMlp]

    def to_json(self):
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json()}


def _heads(r: ConfigReader):
    heads, kv_heads = r.positive_int("heads"), r.positive_int("kv_heads")
    if heads % kv_heads:
        raise InvalidValue(f"{r.where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    return heads, kv_heads


def _read_parallel(r: ConfigReader) -> ParallelMixer:
    lr, rr = r.section("left"), r.section("right")
    heads, kv_heads = _heads(lr)
    dim = lr.positive_int("dim")
    base, dims, scaling = _read_rot(lr, dim, "dim")
    if scaling is not None:
        raise UnsupportedField(f"{lr.where}: this mixer's rotation has no 'scaling'")
    mask = lr.section("mask", optional=True)
    cap = lr.number("softcap", 0.0)
    if cap < 0:
        raise InvalidValue(f"{lr.where}: 'softcap' ({cap}) must not be negative")
    left = LeftMixer(heads, kv_heads, dim, lr.positive_int("vdim"), lr.positive_float("scale"), float(cap), base, dims,
                     0 if mask is None else mask.positive_int("size"))
    rheads, rkv = _heads(rr)
    conv = rr.optional_int("conv") or 0
    if not 0 <= conv <= 16:
        raise InvalidValue(f"{rr.where}: 'conv' ({conv}) must be between 0 and 16 taps")
    return ParallelMixer(left, RightMixer(rheads, rkv, rr.positive_int("dim"), rr.positive_int("vdim"), conv))


def _read_latent(r: ConfigReader) -> LatentMixer:
    rot_dim = r.positive_int("rot_dim")
    base, dims, scaling = _read_rot(r, rot_dim, "rot_dim")
    if dims != rot_dim:
        raise InvalidValue(f"{r.where}: the rotated part turns as a whole: rot.dims ({dims}) must equal rot_dim ({rot_dim})")
    return LatentMixer(r.positive_int("heads"), r.positive_int("dim"), rot_dim, r.positive_int("vdim"),
                       r.positive_int("kv_rank"), r.positive_int("q_rank"), r.positive_float("scale"), base, dims, scaling)


def _read_mlp(r: Optional[ConfigReader]):
    if r is None:
        return None
    kind = r.string("kind")
    if kind == "dense":
        return DenseMlp(r.positive_int("ff"))
    if kind != "moe":
        raise UnsupportedField(f"{r.where}: mlp kind '{kind}' is not supported (dense, moe)")
    router = r.section("router")
    experts, top = router.positive_int("experts"), router.positive_int("top")
    identity = router.optional_int("identity") or 0
    if identity < 0:
        raise InvalidValue(f"{router.where}: 'identity' ({identity}) must not be negative")
    groups = router.section("groups", optional=True)
    count, keep = (1, 1) if groups is None else (groups.positive_int("count"), groups.positive_int("keep"))
    outputs = experts + identity
    if outputs % count or keep > count or top > outputs // count * keep:
        raise InvalidValue(f"{router.where}: {outputs} router outputs in {count} groups, {keep} kept, {top} chosen")
    return MoeMlp(r.section("expert").positive_int("ff"), experts, top, identity, count, keep)


@dataclass(frozen=True)
class ZiginexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    side_dim: int = 0            # 0: no per-layer token input
    layers: Tuple[ZiginexLayer, ...] = ()
    max_positions: int = DEFAULT_MAX_POSITIONS

    ARCHITECTURE = "Ziginex"

    def to_json_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": [layer.to_json() for layer in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZiginexConfig":
        r = ConfigReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise WrongType("config.json: 'layers' must be a non-empty list of layer descriptions")
        layers = []
        for i, entry in enumerate(layers_raw):
            lr = ConfigReader(entry, f"config.json: layers[{i}]")
            kind = lr.string("type")
            if kind not in MIXER_TYPES:
                raise UnsupportedField(f"{lr.where}: mixer type '{kind}' is not supported ({', '.join(MIXER_TYPES)})")
            mixer = _read_parallel(lr.section("mixer")) if kind == "parallel" else _read_latent(lr.section("mixer"))
            layers.append(ZiginexLayer(kind, mixer, _read_mlp(lr.section("mlp", optional=True))))
        side = r.section("token_side", optional=True)
        return cls(architecture=cls.ARCHITECTURE, vocab=r.positive_int("vocab"), width=r.positive_int("width"),
                   norm_eps=r.section("norm").positive_float("eps"),
                   side_dim=0 if side is None else side.positive_int("dim"), layers=tuple(layers),
                   max_positions=r.positive_int("max_positions", DEFAULT_MAX_POSITIONS))
