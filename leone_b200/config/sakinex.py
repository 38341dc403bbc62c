"""Typed configuration of the Sakinex decoder.

Its ``config.json`` names the model under ``architecture`` and describes every layer on its own
(``layers``: a list of ``{"type", "mixer", "mlp"}``).  Top-level keys: ``vocab``, ``width``,
``norm.eps``, ``residual_mult`` and, optionally, ``canon.taps`` (the short convolution in front of
every sublayer) and ``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop-1`` run ``times``
times in a row with the same weights).

Mixer type ``parallel``: ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``conv`` (taps of the convolution on q, k and v; optional), ``rot`` (``base``, ``dims``, optionally
``scaling`` with ``factor``, ``original``, ``fast``, ``slow``), ``mask`` (``size``, ``pool``)),
``right`` (minGRU: ``width``), ``left_scale``, ``right_scale``.

``mlp`` is ``null`` or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared":
{"ff"}}`` (``shared`` optional).

The file gives no limit on positions; ``max_positions`` (not a key of the design) bounds the
engine's block tables and defaults to 2**20.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigReader, InvalidValue, ModelConfig, UnsupportedField, WrongType

DEFAULT_MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("parallel",)


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_json(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class LeftMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                    # taps of the convolution on q, k and v; 0: none
    rot_base: float
    rot_dims: int                # 0: no rotation
    rot_scaling: Optional[YarnScaling]
    mask_size: int
    mask_pool: int

    def to_json(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
               "mask": {"size": self.mask_size, "pool": self.mask_pool}}
        if self.conv:
            out["conv"] = self.conv
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                out["rot"]["scaling"] = self.rot_scaling.to_json()
        return out


@dataclass(frozen=True)
class ParallelMixer:
    left: LeftMixer
    right_width: int
    left_scale: float
    right_scale: float

    def to_json(self):
        return {"left": self.left.to_json(), "right": {"width": self.right_width}, "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class MoeMlp:
    expert_ff: int
    experts: int
    top: int
    shared_ff: int               # 0: no shared expert

    def to_json(self):
        out = {"kind": "moe", "expert": {"ff": self.expert_ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_json(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class SakinexLayer:
    type: str
    mixer: ParallelMixer
    mlp: Optional[MoeMlp]

    def to_json(self):
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json()}


def _read_left(r: ConfigReader) -> LeftMixer:
    heads, kv_heads, dim = r.positive_int("heads"), r.positive_int("kv_heads"), r.positive_int("dim")
    if heads % kv_heads:
        raise InvalidValue(f"{r.where}: 'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    rot = r.section("rot", optional=True)
    base, dims, scaling = 10000.0, 0, None
    if rot is not None:
        base, dims = rot.positive_float("base"), rot.positive_int("dims")
        if dims % 2 or dims > dim:
            raise InvalidValue(f"{rot.where}: 'dims' ({dims}) must be even and at most dim ({dim})")
        sc = rot.section("scaling", optional=True)
        if sc is not None:
            scaling = YarnScaling(sc.positive_float("factor"), sc.positive_float("original"), sc.positive_float("fast"),
                                  sc.positive_float("slow"))
    mask = r.section("mask")
    conv = r.optional_int("conv") or 0
    if not 0 <= conv <= 16:
        raise InvalidValue(f"{r.where}: 'conv' ({conv}) must be between 0 and 16 taps")
    return LeftMixer(heads, kv_heads, dim, r.positive_int("vdim"), r.positive_float("scale"), conv, base, dims, scaling,
                     mask.positive_int("size"), mask.positive_int("pool"))


def _read_mixer(kind: str, r: ConfigReader) -> ParallelMixer:
    if kind not in MIXER_TYPES:
        raise UnsupportedField(f"{r.where}: mixer type '{kind}' is not supported ({', '.join(MIXER_TYPES)})")
    return ParallelMixer(_read_left(r.section("left")), r.section("right").positive_int("width"),
                         r.number("left_scale", 1.0), r.number("right_scale", 1.0))


def _read_mlp(r: Optional[ConfigReader]) -> Optional[MoeMlp]:
    if r is None:
        return None
    kind = r.string("kind")
    if kind != "moe":
        raise UnsupportedField(f"{r.where}: mlp kind '{kind}' is not supported (moe)")
    router = r.section("router")
    experts, top = router.positive_int("experts"), router.positive_int("top")
    if top > experts:
        raise InvalidValue(f"{router.where}: 'top' ({top}) exceeds 'experts' ({experts})")
    shared = r.section("shared", optional=True)
    return MoeMlp(r.section("expert").positive_int("ff"), experts, top, 0 if shared is None else shared.positive_int("ff"))


@dataclass(frozen=True)
class SakinexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    canon_taps: int = 0          # 0: no convolution in front of the sublayers
    layers: Tuple[SakinexLayer, ...] = ()
    loop: Optional[Loop] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    ARCHITECTURE = "Sakinex"

    def to_json_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "layers": [layer.to_json() for layer in self.layers]}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            out["loop"] = self.loop.to_json()
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        lp = self.loop
        return tuple(range(lp.start)) + tuple(range(lp.start, lp.stop)) * lp.times + tuple(range(lp.stop, n))

    def later_pass_starts(self) -> Tuple[int, ...]:
        """Positions of the run order at which a pass over the looped layers begins, the first pass left out."""
        if self.loop is None:
            return ()
        lp = self.loop
        return tuple(lp.start + k * (lp.stop - lp.start) for k in range(1, lp.times))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SakinexConfig":
        r = ConfigReader(raw)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise WrongType("config.json: 'layers' must be a non-empty list of layer descriptions")
        layers = []
        for i, entry in enumerate(layers_raw):
            lr = ConfigReader(entry, f"config.json: layers[{i}]")
            kind = lr.string("type")
            layers.append(SakinexLayer(kind, _read_mixer(kind, lr.section("mixer")),
                                       _read_mlp(lr.section("mlp", optional=True))))
        loop = None
        lr = r.section("loop", optional=True)
        if lr is not None:
            start = lr.optional_int("start")
            stop, times = lr.positive_int("stop"), lr.positive_int("times")
            if start is None or not 0 <= start < stop <= len(layers):
                raise InvalidValue(f"{lr.where}: layers {start} .. {stop} - 1 are not a span of the {len(layers)} layers")
            loop = Loop(start, stop, times)
        canon = r.section("canon", optional=True)
        taps = 0 if canon is None else canon.positive_int("taps")
        if taps > 16:
            raise InvalidValue(f"config.json: canon.taps ({taps}) must be at most 16")
        return cls(architecture=cls.ARCHITECTURE, vocab=r.positive_int("vocab"), width=r.positive_int("width"),
                   norm_eps=r.section("norm").positive_float("eps"), residual_mult=r.number("residual_mult", 1.0),
                   canon_taps=taps, layers=tuple(layers), loop=loop,
                   max_positions=r.positive_int("max_positions", DEFAULT_MAX_POSITIONS))
