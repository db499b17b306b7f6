"""`KoridraConfig`: the hyper-parameters of a Koridra decoder.

config.json of this design is nested: top level `architecture` (a string),
`vocab`, `width`, `max_positions`, `norm.eps`, `postln_alpha`, and `layers`, a
list with one object per layer: `type` ("lightning" or "parallel"), `mixer`
(the mixer's sizes and constants) and `mlp` ({"kind": "dense", "ff": F} or null
for a layer without feed-forward).  Every size and constant is read from there;
nothing is fixed in code.

  lightning mixer:  heads, dim, vdim, decay (one factor per head)
  parallel mixer:   left  {heads, kv_heads, dim, vdim, scale, mask.size,
                           rot {dims, base, scaling {factor, original, fast, slow} or absent}}
                    right {heads, dim, vdim, tau[, gate_rank]}  (the gate's inner width is otherwise
                           taken from the checkpoint's tensor shapes)
                    left_scale, right_scale
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Tuple

from .base import ConfigError, KeyReader

ARCHITECTURE = "Koridra"


def _sub(r: KeyReader, key: str, required: bool = True) -> KeyReader | None:
    """The object under `key` as a reader of its own (errors name the whole path)."""
    if not r.has(key):
        if required:
            raise ConfigError(f"{r.where}: missing required key {key!r}")
        r.used.add(key)
        return None
    r.used.add(key)
    return KeyReader(r.raw[key], f"{r.where}: {key}")


def _finite(where: str, **values: float) -> None:
    for k, v in values.items():
        if not math.isfinite(v):
            raise ConfigError(f"{where}: key {k!r} must be finite, found {v}")


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class SoftmaxBranch:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int | None                 # mask.size: keys are seen within the query's chunk of this many positions
    rot_dims: int
    rot_base: float
    rot_scaling: YarnScaling | None


@dataclass(frozen=True)
class GatedLinearBranch:
    heads: int
    dim: int
    vdim: int
    tau: float
    gate_rank: int | None = None      # inner width of the decay gate; a checkpoint's tensor shape gives it


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxBranch
    right: GatedLinearBranch
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class KoridraLayer:
    type: str
    mixer: object
    ff: int | None                    # width of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class KoridraConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    postln_alpha: float
    layers: Tuple[KoridraLayer, ...]
    raw: dict = field(default_factory=dict, compare=False, repr=False)
    architectures: Tuple[str, ...] = (ARCHITECTURE,)
    ignored_keys: Tuple[str, ...] = field(default=(), compare=False)

    # names the engine's generic code asks every configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "KoridraConfig":
        r = KeyReader(raw, where)
        r.used.update(("architecture", "architectures"))
        V = r.integer("vocab", min_value=1)
        d = r.integer("width", min_value=1)
        max_pos = r.integer("max_positions", min_value=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        alpha = r.number("postln_alpha")
        _finite(where, postln_alpha=alpha, eps=eps)
        r.used.add("layers")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list of layer objects")
        layers = []
        for i, lraw in enumerate(raw["layers"]):
            lw = f"{where}: layers[{i}]"
            lr = KeyReader(lraw, lw)
            kind = lr.raw.get("type")
            lr.used.add("type")
            mr = _sub(lr, "mixer")
            if kind == "lightning":
                mixer = _lightning(mr)
            elif kind == "parallel":
                mixer = _parallel(mr)
            else:
                raise ConfigError(f"{lw}: type = {kind!r}; known types: lightning, parallel")
            fr = _sub(lr, "mlp", required=False)
            ff = None
            if fr is not None:
                fk = fr.raw.get("kind")
                fr.used.add("kind")
                if fk != "dense":
                    raise ConfigError(f"{fr.where}: kind = {fk!r}; known kinds: dense")
                ff = fr.integer("ff", min_value=1)
            layers.append(KoridraLayer(kind, mixer, ff))
        return cls(vocab=V, width=d, max_positions=max_pos, norm_eps=eps, postln_alpha=alpha, layers=tuple(layers),
                   raw=dict(raw), ignored_keys=tuple(r.unused()))

    def to_dict(self) -> dict:
        """A config.json dictionary that `from_dict` reads back to an equal configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "lightning":
                mixer = dict(heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay))
            else:
                L, R = m.left, m.right
                rot = dict(dims=L.rot_dims, base=L.rot_base)
                if L.rot_scaling is not None:
                    s = L.rot_scaling
                    rot["scaling"] = dict(factor=s.factor, original=s.original, fast=s.fast, slow=s.slow)
                left = dict(heads=L.heads, kv_heads=L.kv_heads, dim=L.dim, vdim=L.vdim, scale=L.scale, rot=rot)
                if L.chunk is not None:
                    left["mask"] = dict(size=L.chunk)
                right = dict(heads=R.heads, dim=R.dim, vdim=R.vdim, tau=R.tau)
                if R.gate_rank is not None:
                    right["gate_rank"] = R.gate_rank
                mixer = dict(left=left, right=right,
                             left_scale=m.left_scale, right_scale=m.right_scale)
            layers.append(dict(type=l.type, mixer=mixer, mlp=None if l.ff is None else dict(kind="dense", ff=l.ff)))
        return dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, max_positions=self.max_positions,
                    norm=dict(eps=self.norm_eps), postln_alpha=self.postln_alpha, layers=layers)

    def describe(self) -> dict:
        kinds = [l.type + ("" if l.ff is not None else " (no feed-forward)") for l in self.layers]
        return dict(vocab=self.vocab, width=self.width, max_positions=self.max_positions, norm_eps=self.norm_eps,
                    postln_alpha=self.postln_alpha, n_layers=len(self.layers), layer_types=kinds,
                    feed_forward_widths=[l.ff for l in self.layers])


def _lightning(r: KeyReader) -> LightningMixer:
    H = r.integer("heads", min_value=1)
    dk = r.integer("dim", min_value=1)
    dv = r.integer("vdim", min_value=1)
    r.used.add("decay")
    dec = r.raw.get("decay")
    if (not isinstance(dec, list) or len(dec) != H or
            not all(isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(x) for x in dec)):
        raise ConfigError(f"{r.where}: key 'decay' must be a list of {H} numbers (one per head), found {dec!r}")
    return LightningMixer(H, dk, dv, tuple(float(x) for x in dec))


def _parallel(r: KeyReader) -> ParallelMixer:
    lr, rr = _sub(r, "left"), _sub(r, "right")
    H = lr.integer("heads", min_value=1)
    G = lr.integer("kv_heads", default=H, min_value=1)
    if H % G:
        raise ConfigError(f"{lr.where}: heads {H} is not a multiple of kv_heads {G}")
    dim = lr.integer("dim", min_value=1)
    vdim = lr.integer("vdim", default=dim, min_value=1)
    if vdim != dim:
        raise ConfigError(f"{lr.where}: vdim {vdim} differs from dim {dim}, but the values of this mixer are its keys")
    scale = lr.number("scale", default=1.0 / math.sqrt(dim))
    mask = _sub(lr, "mask", required=False)
    chunk = mask.integer("size", min_value=1) if mask is not None else None
    rot = _sub(lr, "rot", required=False)
    rot_dims, rot_base, scaling = 0, 1.0, None
    if rot is not None:
        rot_dims = rot.integer("dims", min_value=0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{rot.where}: dims {rot_dims} must be even and at most the head size {dim}")
        rot_base = rot.number("base", positive=True)
        sr = _sub(rot, "scaling", required=False)
        if sr is not None:
            scaling = YarnScaling(sr.number("factor", positive=True), sr.number("original", positive=True),
                                  sr.number("fast", positive=True), sr.number("slow", positive=True))
    left = SoftmaxBranch(H, G, dim, vdim, scale, chunk, rot_dims, rot_base, scaling)
    right = GatedLinearBranch(rr.integer("heads", min_value=1), rr.integer("dim", min_value=1),
                              rr.integer("vdim", min_value=1), rr.number("tau", positive=True),
                              rr.optional_integer("gate_rank", min_value=1))
    ls, rs = r.number("left_scale", default=1.0), r.number("right_scale", default=1.0)
    _finite(r.where, left_scale=ls, right_scale=rs, scale=scale)
    return ParallelMixer(left, right, ls, rs)
